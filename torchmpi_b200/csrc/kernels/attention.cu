// Causal self-attention forward (softmax(Q K^T / sqrt(d)) V, head size 64) as one tcgen05 kernel.
//
// The reference has no attention (its models are MNIST networks, examples/mnist/*.lua); the GPT-2 configuration
// of this package needs one, and it is a contraction, so it belongs on the tensor cores.  One CTA handles one
// block of 128 queries of one (batch, head) and walks the key / value blocks up to its diagonal:
//
//   warp 0     TMA producer: the Q tile once, then K tiles of 128 keys through a two-stage ring and V tiles through
//              one buffer (V of the next block is fetched while its scores are exponentiated)
//   warp 1     MMA issuer:   S = Q K^T (128 x 128, fp32, tensor memory), then O_j = P V (128 x 64, tensor memory)
//   warps 2-9  softmax:      two threads per query row (tcgen05.ld 32x32b gives a thread its own row, so there are no
//                            shuffles; both read the whole row for its maximum, each exponentiates 64 of the 128
//                            scores): running maximum, P = exp2(scaled S - max) written as bf16 into shared memory
//                            in the K-major 128-byte-swizzled layout that the second MMA reads, then the running
//                            output acc = acc * alpha + O_j in registers (32 of the 64 columns per thread)
//
// S for block j + 1 is issued as soon as the softmax warps have read S of block j, so the tensor core works on it
// while they exponentiate, and the row maximum of block j + 1 is found while the tensor core multiplies P_j by V; a
// quarter of the exponentials run as a cubic on the FMA pipe because the special-function unit (which also packs
// fp32 pairs into bf16) is the busiest pipe of this kernel.  Two CTAs fit on an SM (256 tensor-memory columns and 96 KB of shared memory each), so
// one CTA's softmax overlaps the other's MMAs.  Q, K and V are read where the fused QKV projection left them
// ([B * T, 3 C], one tensor map per operand) and the output is written as [B * T, C]: no transposes around the
// kernel.  Every wait is bounded; a CTA that gives up records where in the status word and frees its tensor memory.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <mutex>
#include "sm100_ptx.cuh"
#include "attn_util.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"

using namespace tmpi;

namespace tmpi {
int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
}

namespace attn {
using namespace attn_util;

constexpr int BQ = 128, BKV = 128, D = 64, THREADS = 320, UMMA_K = 16;
constexpr int TILE_BYTES = 128 * D * 2;                       // a 128 x 64 bf16 tile: 16 KB
constexpr int P_BYTES = BQ * BKV * 2;                         // 32 KB: two K-major chunks of 64 keys
constexpr int SMEM_TILES = TILE_BYTES * 4 + P_BYTES;          // Q, K x 2, V, P
constexpr int V_OFF = TILE_BYTES * 3;                          // P follows the one or two V buffers
constexpr int SMEM_SHARED = 256;                              // the barrier block follows the tiles
constexpr int TMEM_COLS = 256;                                // S: columns 0-127, O_j: columns 128-191
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;

struct alignas(128) Shared {
  uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full, s_empty, p_full, o_full;
  uint64_t pair[4];            // the 64 threads that share 32 rows meet here (bounded, unlike a named barrier)
  uint32_t tmem_base;
  int error;
};
static_assert(sizeof(Shared) <= SMEM_SHARED, "barrier block");

struct Params {
  int B, T, H, q_blocks;
  int v_stages;                // 1 or 2 V buffers (2 prefetches V a block ahead and costs 16 KB of shared memory)
  float scale_log2;            // softmax scale times log2(e)
  __nv_bfloat16* out;          // [B * T, ld_out], head h at columns h * 64
  int ld_out;
  float* lse;                  // [B, H, T]: natural-log sum of exponentials of the scaled scores
  int* status;
  unsigned long long* trace;   // optional: time stamps of the phases of CTA 0 (see tmpi_attention_set_trace)
};

__device__ __forceinline__ void fail(Shared* sh, const Params& p, int where) {
  atomicExch(&sh->error, where);
  if (p.status) atomicCAS(p.status, 0, 3000 + where);
}

// Phase time stamps of one CTA for tuning: slot = (block * 16 + event), written by one thread per role.
__device__ __forceinline__ void stamp(const Params& p, int j, int ev) {
  if (p.trace && blockIdx.x == 0) p.trace[j * 16 + ev] = sm100::now_ns();
}

#define ATTN_WAIT(bar, parity, where) \
  do { if (!sm100::mbar_wait((bar), (parity), kWaitBudgetNs) || sh->error) { fail(sh, p, (where)); return; } } while (0)

__device__ void producer(Shared* sh, unsigned char* tiles, const Params& p, const CUtensorMap* mq, const CUtensorMap* mk,
                         const CUtensorMap* mv, int b, int h, int qblk) {
  const int row0 = b * p.T;
  sm100::mbar_expect_tx(&sh->q_full, TILE_BYTES);
  sm100::tma_load_2d(tiles, mq, h * D, row0 + qblk * BQ, &sh->q_full);
  auto load_k = [&](int j) {
    sm100::mbar_expect_tx(&sh->k_full[j & 1], TILE_BYTES);
    sm100::tma_load_2d(tiles + TILE_BYTES * (1 + (j & 1)), mk, h * D, row0 + j * BKV, &sh->k_full[j & 1]);
  };
  load_k(0);
  for (int j = 0; j <= qblk; ++j) {
    if (j < qblk) {                                                        // K runs one block ahead of V
      if (j + 1 >= 2) ATTN_WAIT(&sh->k_empty[(j + 1) & 1], (((j + 1) >> 1) - 1) & 1, 1);   // S of block j - 1 has read this stage
      load_k(j + 1);
    }
    const int vs = p.v_stages == 2 ? (j & 1) : 0, vuse = p.v_stages == 2 ? (j >> 1) : j;
    if (vuse >= 1) ATTN_WAIT(&sh->v_empty[vs], (vuse - 1) & 1, 13);        // the P V that read this buffer is done
    sm100::mbar_expect_tx(&sh->v_full[vs], TILE_BYTES);
    sm100::tma_load_2d(tiles + V_OFF + vs * TILE_BYTES, mv, h * D, row0 + j * BKV, &sh->v_full[vs]);
  }
}

__device__ void mma_issuer(Shared* sh, unsigned char* tiles, const Params& p, int qblk) {
  const uint32_t tmem_s = sh->tmem_base, tmem_o = sh->tmem_base + 128;
  const uint32_t q_addr = sm100::smem_u32(tiles), p_addr = sm100::smem_u32(tiles + V_OFF + p.v_stages * TILE_BYTES);
  constexpr uint32_t idesc_s = sm100::make_idesc_f16(BQ, BKV, true);            // Q and K both K-major
  constexpr uint32_t idesc_o = sm100::make_idesc_f16(BQ, D, true, true);        // P K-major, V MN-major (d contiguous)
  // descriptors of every operand slice, built once
  uint64_t dq[D / UMMA_K], dk[2][D / UMMA_K], dp[BKV / UMMA_K], dv[2][BKV / UMMA_K];
  const uint32_t v_addr = sm100::smem_u32(tiles + V_OFF);
#pragma unroll
  for (int k = 0; k < D / UMMA_K; ++k) {
    dq[k] = sm100::make_desc_sw128(q_addr + k * UMMA_K * 2);
    dk[0][k] = sm100::make_desc_sw128(sm100::smem_u32(tiles + TILE_BYTES) + k * UMMA_K * 2);
    dk[1][k] = sm100::make_desc_sw128(sm100::smem_u32(tiles + 2 * TILE_BYTES) + k * UMMA_K * 2);
  }
#pragma unroll
  for (int k = 0; k < BKV / UMMA_K; ++k) {
    dp[k] = sm100::make_desc_sw128(p_addr + (k >> 2) * TILE_BYTES + (k & 3) * UMMA_K * 2);
    dv[0][k] = sm100::make_desc_sw128_mn(v_addr + k * UMMA_K * 128, TILE_BYTES, 1024);
    dv[1][k] = sm100::make_desc_sw128_mn(v_addr + TILE_BYTES + k * UMMA_K * 128, TILE_BYTES, 1024);
  }
  auto issue_s = [&](int j) {
    if (j & 1) {
#pragma unroll
      for (int k = 0; k < D / UMMA_K; ++k) sm100::umma_f16(tmem_s, dq[k], dk[1][k], idesc_s, k > 0 ? 1u : 0u);
    } else {
#pragma unroll
      for (int k = 0; k < D / UMMA_K; ++k) sm100::umma_f16(tmem_s, dq[k], dk[0][k], idesc_s, k > 0 ? 1u : 0u);
    }
    sm100::umma_commit(&sh->s_full);
    sm100::umma_commit(&sh->k_empty[j & 1]);
  };
  ATTN_WAIT(&sh->q_full, 0, 2);
  ATTN_WAIT(&sh->k_full[0], 0, 3);
  sm100::tc_fence_after();
  issue_s(0);
  for (int j = 0; j <= qblk; ++j) {
    if (j < qblk) {                      // S of the next block, as soon as this block's S has been read
      ATTN_WAIT(&sh->s_empty, j & 1, 4);
      stamp(p, j, 8);
      ATTN_WAIT(&sh->k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, 5);
      sm100::tc_fence_after();
      issue_s(j + 1);
      stamp(p, j, 9);
    }
    ATTN_WAIT(&sh->p_full, j & 1, 6);
    stamp(p, j, 10);
    const int vs = p.v_stages == 2 ? (j & 1) : 0, vuse = p.v_stages == 2 ? (j >> 1) : j;
    ATTN_WAIT(&sh->v_full[vs], vuse & 1, 14);
    stamp(p, j, 11);
    sm100::tc_fence_after();
    if (vs) {
#pragma unroll
      for (int k = 0; k < BKV / UMMA_K; ++k) sm100::umma_f16(tmem_o, dp[k], dv[1][k], idesc_o, k > 0 ? 1u : 0u);
    } else {
#pragma unroll
      for (int k = 0; k < BKV / UMMA_K; ++k) sm100::umma_f16(tmem_o, dp[k], dv[0][k], idesc_o, k > 0 ? 1u : 0u);
    }
    sm100::umma_commit(&sh->o_full);
    sm100::umma_commit(&sh->v_empty[vs]);
    stamp(p, j, 12);
  }
}

// One thread's 64 scores of a block: P = exp2(S * c2 + nmc) as bf16 into the swizzled K-major tile; returns their sum.
// DIAG: the block on the diagonal, where a key after the query gives 0 and whole chunks of 32 keys may be masked
// for the warp (then there is nothing to load or exponentiate).
template <bool DIAG>
__device__ __forceinline__ float exp_pass(Shared* sh, uint32_t (&r)[32], uint32_t tmem_s, unsigned char* p_row, int row, int half,
                                          int last_row, float c2, float nmc) {
  const unsigned long long c2x2 = pack2(__float_as_uint(c2), __float_as_uint(c2));
  const unsigned long long nmc2 = pack2(__float_as_uint(nmc), __float_as_uint(nmc));
  unsigned long long rs2 = 0ull;                          // two partial sums (0.f, 0.f)
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    const int key0 = half * 64 + c * 32;
    const bool masked = DIAG && key0 > last_row;           // warp-uniform
    if (!masked) {
      sm100::tmem_ld_32x32(tmem_s + c * 32, r);
      sm100::tmem_ld_wait();
    }
    if (c == 1) {                                         // S is in registers: the next S may overwrite it
      sm100::tc_fence_before();
      sm100::mbar_arrive(&sh->s_empty);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {                          // eight keys = one 16-byte unit of the swizzled row
      uint32_t w[4] = {0u, 0u, 0u, 0u};
      if (!masked) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = u * 8 + 2 * q;
          float a0, a1;
          unpack2(fma2(pack2(r[i], r[i + 1]), c2x2, nmc2), a0, a1);
          // a quarter of the exponentials on the FMA pipe, the rest on the special-function unit
          float e0 = q == 3 ? ex2_fma(a0) : ex2(a0);
          float e1 = q == 3 ? ex2_fma(a1) : ex2(a1);
          if (DIAG) {
            if (key0 + i > row) e0 = 0.f;
            if (key0 + i + 1 > row) e1 = 0.f;
          }
          rs2 = add2(rs2, pack2(__float_as_uint(e0), __float_as_uint(e1)));
          __nv_bfloat162 hh = __floats2bfloat162_rn(e0, e1);
          w[q] = *reinterpret_cast<uint32_t*>(&hh);
        }
      }
      const int unit = c * 4 + u;
      *reinterpret_cast<uint4*>(p_row + ((unit ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
  float rs0, rs1;
  unpack2(rs2, rs0, rs1);
  return rs0 + rs1;
}

// Two threads per query row: the warps with the same (warp & 3) read the same 32 tensor-memory lanes; `half` picks
// which 64 of the 128 score columns a thread exponentiates (and which 32 of the 64 output columns it accumulates).
// Both read the whole row for its maximum (tensor-memory reads are cheap and this needs no exchange); each keeps
// the partial row sum of its own columns, and the two are added once at the end through shared memory.
__device__ void softmax_rows(Shared* sh, unsigned char* tiles, const Params& p, int b, int h, int qblk, int quarter, int half,
                             int lane) {
  const int row = quarter * 32 + lane;
  const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
  const uint32_t tmem_row = sh->tmem_base + lane_base, tmem_s = tmem_row + half * 64;
  const uint32_t tmem_o = sh->tmem_base + 128 + lane_base + half * 32;
  unsigned char* p_tile = tiles + V_OFF + p.v_stages * TILE_BYTES;
  unsigned char* p_row = p_tile + half * TILE_BYTES + row * 128;      // chunk `half`: keys 64 half ...
  float* xch = reinterpret_cast<float*>(p_tile);     // the P tile, once the last MMA has read it
  const float c2 = p.scale_log2;
  float m = -INFINITY, l = 0.f;
  unsigned long long acc2[D / 4];                         // this thread's 32 output columns, two per register pair
#pragma unroll
  for (int i = 0; i < D / 4; ++i) acc2[i] = 0ull;
  uint32_t r[32];
  const int last_row = quarter * 32 + 31;                 // a chunk of keys beyond it is masked for the whole warp
  // the maximum of the row over block j (on the diagonal block a key after the query is masked)
  auto row_max = [&](int j, float mx) {
    const bool diag = j == qblk;
#pragma unroll 1
    for (int c = 0; c < BKV / 32; ++c) {
      if (diag && c * 32 > last_row) break;
      sm100::tmem_ld_32x32(tmem_row + c * 32, r);
      sm100::tmem_ld_wait();
      if (!diag) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx = max3(mx, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (c * 32 + i <= row) mx = fmaxf(mx, __uint_as_float(r[i]));
      }
    }
    return mx;
  };
  const bool tracer = row == 0 && half == 0;
  if (tracer) stamp(p, 0, 0);
  ATTN_WAIT(&sh->s_full, 0, 7);
  if (tracer) stamp(p, 0, 1);
  sm100::tc_fence_after();
  float mx = row_max(0, m);
  for (int j = 0; j <= qblk; ++j) {
    const bool diag = j == qblk;
    if (tracer) stamp(p, j, 2);
    const float alpha = ex2((m - mx) * c2);             // 0 for the first block (m = -inf)
    const float nmc = -mx * c2;
    // second pass: P = exp2(S * c2 - max * c2) as bf16 into the swizzled K-major tile
    const float rs = diag ? exp_pass<true>(sh, r, tmem_s, p_row, row, half, last_row, c2, nmc)
                          : exp_pass<false>(sh, r, tmem_s, p_row, row, half, last_row, c2, nmc);
    l = l * alpha + rs;
    m = mx;
    if (tracer) stamp(p, j, 3);
    sm100::fence_proxy_async_smem();                      // the MMA reads P through the async proxy
    sm100::mbar_arrive(&sh->p_full);
    if (tracer) stamp(p, j, 4);
    // while the tensor core multiplies P by V: the maximum of the next block's scores, which are already there
    if (j < qblk) {
      ATTN_WAIT(&sh->s_full, (j + 1) & 1, 7);
      if (tracer) stamp(p, j + 1, 1);
      sm100::tc_fence_after();
      mx = row_max(j + 1, m);
    }
    // running output: this thread's 32 columns
    ATTN_WAIT(&sh->o_full, j & 1, 8);
    if (tracer) stamp(p, j, 5);
    sm100::tc_fence_after();
    sm100::tmem_ld_32x32(tmem_o, r);
    sm100::tmem_ld_wait();
    const unsigned long long al2 = pack2(__float_as_uint(alpha), __float_as_uint(alpha));
#pragma unroll
    for (int i = 0; i < 16; ++i) acc2[i] = fma2(acc2[i], al2, pack2(r[2 * i], r[2 * i + 1]));
    if (tracer) stamp(p, j, 6);
    sm100::tc_fence_before();
  }
  // the row sum is the sum of the two halves' partial sums (the last o_full says that the MMAs are done with P)
  xch[half * 128 + row] = l;
  sm100::mbar_arrive(&sh->pair[quarter]);
  ATTN_WAIT(&sh->pair[quarter], 0, 11);
  l += xch[(half ^ 1) * 128 + row];
  const float inv = 1.f / l;
  const size_t grow = (size_t)b * p.T + (size_t)qblk * BQ + row;
  __nv_bfloat16* o = p.out + grow * p.ld_out + h * D + half * 32;
#pragma unroll
  for (int u = 0; u < D / 16; ++u) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a0, a1;
      unpack2(acc2[u * 4 + i], a0, a1);
      __nv_bfloat162 hh = __floats2bfloat162_rn(a0 * inv, a1 * inv);
      w[i] = *reinterpret_cast<uint32_t*>(&hh);
    }
    *reinterpret_cast<uint4*>(o + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
  }
  if (p.lse && half == 0) p.lse[((size_t)b * p.H + h) * p.T + (size_t)qblk * BQ + row] = m * c2 * 0.6931471805599453f + __logf(l);
}

__global__ void __launch_bounds__(THREADS, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];   // no static shared memory: the tiles start aligned
  unsigned char* tiles = smem_raw;
  Shared* sh = (Shared*)(smem_raw + SMEM_TILES + (p.v_stages - 1) * TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the longest rows of blocks (near the end of the sequence) start first
  const int bh = blockIdx.x % (p.B * p.H);
  const int qblk = p.q_blocks - 1 - blockIdx.x / (p.B * p.H);
  const int b = bh / p.H, h = bh - b * p.H;
  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(&map_q);
    sm100::tma_prefetch_desc(&map_k);
    sm100::tma_prefetch_desc(&map_v);
    sm100::mbar_init(&sh->q_full, 1);
    for (int s = 0; s < 2; ++s) { sm100::mbar_init(&sh->k_full[s], 1); sm100::mbar_init(&sh->k_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { sm100::mbar_init(&sh->v_full[s], 1); sm100::mbar_init(&sh->v_empty[s], 1); }
    sm100::mbar_init(&sh->s_full, 1);
    sm100::mbar_init(&sh->s_empty, 256);
    sm100::mbar_init(&sh->p_full, 256);
    sm100::mbar_init(&sh->o_full, 1);
    for (int q = 0; q < 4; ++q) sm100::mbar_init(&sh->pair[q], 64);
    sh->error = 0;
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(&sh->tmem_base, TMEM_COLS);
    sm100::tmem_relinquish();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();

  // the swizzled tiles need a 1024-byte aligned base
  const bool fits = (sm100::smem_u32(tiles) & 1023u) == 0;
  if (!fits) {
    if (threadIdx.x == 0) fail(sh, p, 9);
  } else if (warp == 0) {
    if (sm100::elect_one()) producer(sh, tiles, p, &map_q, &map_k, &map_v, b, h, qblk);
  } else if (warp == 1) {
    if (sm100::elect_one()) mma_issuer(sh, tiles, p, qblk);
  } else {
    softmax_rows(sh, tiles, p, b, h, qblk, warp & 3, (warp - 2) >> 2, lane);
  }
  __syncwarp();
  sm100::tc_fence_before();
  __syncthreads();
  if (sh->error && warp == 0 && sm100::elect_one()) {
    const unsigned long long t0 = sm100::now_ns();
    while (sm100::now_ns() - t0 < 200000000ull) { __nanosleep(1000); }   // copies in flight land within microseconds
  }
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(sh->tmem_base, TMEM_COLS);
  }
}

}  // namespace attn

static unsigned long long* g_attn_trace = nullptr;
static int g_attn_v_stages = 1;
static int attn_smem_bytes() { return attn::SMEM_TILES + (g_attn_v_stages - 1) * attn::TILE_BYTES + attn::SMEM_SHARED; }

static int* attn_status_word(int** host_out = nullptr) {
  static int* dev_ptr = nullptr;
  static int* host_ptr = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    if (cudaHostAlloc((void**)&host_ptr, sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
      *host_ptr = 0;
      cudaHostGetDevicePointer((void**)&dev_ptr, host_ptr, 0);
    }
  });
  if (host_out) *host_out = host_ptr;
  return dev_ptr;
}

extern "C" {

// out[b, t, h, :] = sum_s softmax_s(scale * q[b, t, h, :] . k[b, s, h, :], s <= t) v[b, s, h, :] for bf16 q, k, v given
// as [B * T, H * 64] matrices with a common row pitch of ld_qkv elements (for instance the three column blocks of a
// fused QKV projection); out is [B * T, ld_out]; lse (optional) is [B, H, T] fp32.  T must be a multiple of 128.
int tmpi_attention_fwd(const void* q, const void* k, const void* v, int64_t ld_qkv, void* out, int64_t ld_out, float* lse,
                       int B, int T, int H, float scale, void* stream) {
  if (B < 1 || H < 1 || T < 128 || T % 128) return fail(TMPI_ERR_UNSUPPORTED, "attention: T=%d must be a positive multiple of 128", T);
  if (ld_out % 8 || ((uintptr_t)out & 15)) return fail(TMPI_ERR_INVALID, "attention: the output must be 16-byte aligned with a pitch that is a multiple of 8");
  if ((int64_t)B * H * (T / 128) > 0x7fffffffLL) return fail(TMPI_ERR_INVALID, "attention: too many blocks");
  CUtensorMap mq, mk, mv;
  int st;
  const uint64_t rows = (uint64_t)B * T, cols = (uint64_t)H * attn::D;
  if ((st = make_tmap_bf16(&mq, q, rows, cols, (uint64_t)ld_qkv, 128))) return st;
  if ((st = make_tmap_bf16(&mk, k, rows, cols, (uint64_t)ld_qkv, 128))) return st;
  if ((st = make_tmap_bf16(&mv, v, rows, cols, (uint64_t)ld_qkv, 128))) return st;
  cudaError_t ae = cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn_smem_bytes());
  if (ae == cudaSuccess)          // two CTAs per SM need the largest shared-memory carve-out
    ae = cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (ae != cudaSuccess) return fail(TMPI_ERR_CUDA, "attention: shared memory attribute: %s", cudaGetErrorString(ae));
  attn::Params p;
  p.B = B; p.T = T; p.H = H; p.q_blocks = T / attn::BQ;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)out; p.ld_out = (int)ld_out; p.lse = lse;
  p.status = attn_status_word();
  p.trace = g_attn_trace;
  const int grid = B * H * p.q_blocks;
  p.v_stages = g_attn_v_stages;
  attn::attention_fwd_kernel<<<grid, attn::THREADS, attn_smem_bytes(), (cudaStream_t)stream>>>(mq, mk, mv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
}

// Resident CTAs of the attention kernel per SM (2 when shared memory and registers allow the intended overlap).
int tmpi_attention_ctas_per_sm(void) {
  int n = 0;
  cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn_smem_bytes());
  cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn::attention_fwd_kernel, attn::THREADS, attn_smem_bytes()) != cudaSuccess) return -1;
  return n;
}

// Tuning aid: with a device buffer of (T / 128) * 16 64-bit words, CTA 0 of every later launch (the last query block
// of the first batch and head) records the time of each phase of each key block (ns): 0 waits for S, 1 has S, 2 row
// maximum known, 3 P written, 4 P announced, 5 has O_j, 6 output updated; MMA thread: 8 S was read, 9 next S issued,
// 10 has P, 11 has V, 12 P V issued.  nullptr switches it off.
// Tuning aid: one or two V buffers per CTA (see Params::v_stages).
void tmpi_attention_set_v_stages(int n) { g_attn_v_stages = n == 2 ? 2 : 1; }

void tmpi_attention_set_trace(void* device_buffer) { g_attn_trace = (unsigned long long*)device_buffer; }

// Non-zero after an attention CTA gave up on a bounded wait (3000 + the point where it happened); clears it.
int tmpi_attention_status(void) {
  int* host = nullptr;
  attn_status_word(&host);
  if (!host) return 0;
  int v = *(volatile int*)host;
  if (v) *(volatile int*)host = 0;
  return v;
}

}  // extern "C"
