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
//                            shuffles; the two halves of a row exchange their maxima through shared memory): running
//                            maximum, P = exp2(scaled S - max) written as bf16 into shared memory in the K-major
//                            128-byte-swizzled layout that the second MMA reads, then the running output
//                            acc = acc * alpha + O_j in registers
//
// S for block j + 1 is issued as soon as the softmax warps have read S of block j, so the tensor core works on it
// while they exponentiate; two CTAs fit on an SM (256 tensor-memory columns and 96 KB of shared memory each), so
// one CTA's softmax overlaps the other's MMAs.  Q, K and V are read where the fused QKV projection left them
// ([B * T, 3 C], one tensor map per operand) and the output is written as [B * T, C]: no transposes around the
// kernel.  Every wait is bounded; a CTA that gives up records where in the status word and frees its tensor memory.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <mutex>
#include "sm100_ptx.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"

using namespace tmpi;

namespace tmpi {
int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
}

namespace attn {

constexpr int BQ = 128, BKV = 128, D = 64, THREADS = 320, UMMA_K = 16;
constexpr int TILE_BYTES = 128 * D * 2;                       // a 128 x 64 bf16 tile: 16 KB
constexpr int P_BYTES = BQ * BKV * 2;                         // 32 KB: two K-major chunks of 64 keys
constexpr int SMEM_TILES = TILE_BYTES * 4 + P_BYTES;          // Q, K x 2, V, P
constexpr int V_OFF = TILE_BYTES * 3, P_OFF = TILE_BYTES * 4;
constexpr int SMEM_DYNAMIC = SMEM_TILES + 128;                // the barrier block follows the tiles
constexpr int TMEM_COLS = 256;                                // S: columns 0-127, O_j: columns 128-191
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;

struct alignas(128) Shared {
  uint64_t q_full, k_full[2], k_empty[2], v_full, v_empty, s_full, s_empty, p_full, o_full;
  uint64_t pair[4];            // the 64 threads that share 32 rows meet here (bounded, unlike a named barrier)
  uint32_t tmem_base;
  int error;
};
static_assert(sizeof(Shared) == 128, "barrier block");

struct Params {
  int B, T, H, q_blocks;
  float scale_log2;            // softmax scale times log2(e)
  __nv_bfloat16* out;          // [B * T, ld_out], head h at columns h * 64
  int ld_out;
  float* lse;                  // [B, H, T]: natural-log sum of exponentials of the scaled scores
  int* status;
};

__device__ __forceinline__ void fail(Shared* sh, const Params& p, int where) {
  atomicExch(&sh->error, where);
  if (p.status) atomicCAS(p.status, 0, 3000 + where);
}

#define ATTN_WAIT(bar, parity, where) \
  do { if (!sm100::mbar_wait((bar), (parity), kWaitBudgetNs) || sh->error) { fail(sh, p, (where)); return; } } while (0)

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

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
    if (j >= 1) ATTN_WAIT(&sh->v_empty, (j - 1) & 1, 13);                  // P V of block j - 1 has read V
    sm100::mbar_expect_tx(&sh->v_full, TILE_BYTES);
    sm100::tma_load_2d(tiles + V_OFF, mv, h * D, row0 + j * BKV, &sh->v_full);
  }
}

__device__ void mma_issuer(Shared* sh, unsigned char* tiles, const Params& p, int qblk) {
  const uint32_t tmem_s = sh->tmem_base, tmem_o = sh->tmem_base + 128;
  const uint32_t q_addr = sm100::smem_u32(tiles), p_addr = sm100::smem_u32(tiles + P_OFF);
  constexpr uint32_t idesc_s = sm100::make_idesc_f16(BQ, BKV, true);            // Q and K both K-major
  constexpr uint32_t idesc_o = sm100::make_idesc_f16(BQ, D, true, true);        // P K-major, V MN-major (d contiguous)
  auto issue_s = [&](int j) {
    const uint32_t k_addr = sm100::smem_u32(tiles + TILE_BYTES * (1 + (j & 1)));
#pragma unroll
    for (int k = 0; k < D / UMMA_K; ++k)
      sm100::umma_f16(tmem_s, sm100::make_desc_sw128(q_addr + k * UMMA_K * 2), sm100::make_desc_sw128(k_addr + k * UMMA_K * 2),
                      idesc_s, k > 0 ? 1u : 0u);
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
      ATTN_WAIT(&sh->k_full[(j + 1) & 1], ((j + 1) >> 1) & 1, 5);
      sm100::tc_fence_after();
      issue_s(j + 1);
    }
    ATTN_WAIT(&sh->p_full, j & 1, 6);
    ATTN_WAIT(&sh->v_full, j & 1, 14);
    sm100::tc_fence_after();
    const uint32_t v_addr = sm100::smem_u32(tiles + V_OFF);
#pragma unroll
    for (int k = 0; k < BKV / UMMA_K; ++k)
      sm100::umma_f16(tmem_o, sm100::make_desc_sw128(p_addr + (k >> 2) * TILE_BYTES + (k & 3) * UMMA_K * 2),
                      sm100::make_desc_sw128_mn(v_addr + k * UMMA_K * 128, TILE_BYTES, 1024), idesc_o, k > 0 ? 1u : 0u);
    sm100::umma_commit(&sh->o_full);
    sm100::umma_commit(&sh->v_empty);
  }
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
  unsigned char* p_row = tiles + P_OFF + half * TILE_BYTES + row * 128;      // chunk `half`: keys 64 half ...
  float* xch = reinterpret_cast<float*>(tiles + P_OFF);     // the P tile, once the last MMA has read it
  const float c2 = p.scale_log2;
  float m = -INFINITY, l = 0.f;
  float acc[D / 2];
#pragma unroll
  for (int i = 0; i < D / 2; ++i) acc[i] = 0.f;
  uint32_t r[32];
  for (int j = 0; j <= qblk; ++j) {
    const bool diag = j == qblk;
    ATTN_WAIT(&sh->s_full, j & 1, 7);
    sm100::tc_fence_after();
    // first pass over the whole row: its maximum (a masked entry is a key after the query)
    float mx = m;
#pragma unroll 1
    for (int c = 0; c < BKV / 32; ++c) {
      sm100::tmem_ld_32x32(tmem_row + c * 32, r);
      sm100::tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (!diag || c * 32 + i <= row) mx = fmaxf(mx, __uint_as_float(r[i]));
    }
    const float alpha = ex2((m - mx) * c2);             // 0 for the first block (m = -inf)
    const float mc = mx * c2;
    float rs = 0.f;
    // second pass: P = exp2(S * c2 - max * c2) as bf16 into the swizzled K-major tile
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      sm100::tmem_ld_32x32(tmem_s + c * 32, r);
      sm100::tmem_ld_wait();
      if (c == 1) {                                       // S is in registers: the next S may overwrite it
        sm100::tc_fence_before();
        sm100::mbar_arrive(&sh->s_empty);
      }
      const int key0 = half * 64 + c * 32;
#pragma unroll
      for (int u = 0; u < 4; ++u) {                        // eight keys = one 16-byte unit of the swizzled row
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int i = u * 8 + 2 * q;
          float e0 = ex2(fmaf(__uint_as_float(r[i]), c2, -mc));
          float e1 = ex2(fmaf(__uint_as_float(r[i + 1]), c2, -mc));
          if (diag) {
            if (key0 + i > row) e0 = 0.f;
            if (key0 + i + 1 > row) e1 = 0.f;
          }
          rs += e0 + e1;
          __nv_bfloat162 hh = __floats2bfloat162_rn(e0, e1);
          w[q] = *reinterpret_cast<uint32_t*>(&hh);
        }
        const int unit = c * 4 + u;
        *reinterpret_cast<uint4*>(p_row + ((unit ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    l = l * alpha + rs;
    m = mx;
    sm100::fence_proxy_async();                           // the MMA reads P through the async proxy
    sm100::mbar_arrive(&sh->p_full);
    // running output: this thread's 32 columns
    ATTN_WAIT(&sh->o_full, j & 1, 8);
    sm100::tc_fence_after();
    sm100::tmem_ld_32x32(tmem_o, r);
    sm100::tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) acc[i] = fmaf(acc[i], alpha, __uint_as_float(r[i]));
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
      __nv_bfloat162 hh = __floats2bfloat162_rn(acc[u * 8 + 2 * i] * inv, acc[u * 8 + 2 * i + 1] * inv);
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
  Shared* sh = (Shared*)(smem_raw + SMEM_TILES);
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
    sm100::mbar_init(&sh->v_full, 1);
    sm100::mbar_init(&sh->v_empty, 1);
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
  cudaError_t ae = cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_DYNAMIC);
  if (ae == cudaSuccess)          // two CTAs per SM need the largest shared-memory carve-out
    ae = cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (ae != cudaSuccess) return fail(TMPI_ERR_CUDA, "attention: shared memory attribute: %s", cudaGetErrorString(ae));
  attn::Params p;
  p.B = B; p.T = T; p.H = H; p.q_blocks = T / attn::BQ;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.out = (__nv_bfloat16*)out; p.ld_out = (int)ld_out; p.lse = lse;
  p.status = attn_status_word();
  const int grid = B * H * p.q_blocks;
  attn::attention_fwd_kernel<<<grid, attn::THREADS, attn::SMEM_DYNAMIC, (cudaStream_t)stream>>>(mq, mk, mv, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "attention launch: %s", cudaGetErrorString(e));
}

// Resident CTAs of the attention kernel per SM (2 when shared memory and registers allow the intended overlap).
int tmpi_attention_ctas_per_sm(void) {
  int n = 0;
  cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, attn::SMEM_DYNAMIC);
  cudaFuncSetAttribute(attn::attention_fwd_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, attn::attention_fwd_kernel, attn::THREADS, attn::SMEM_DYNAMIC) != cudaSuccess) return -1;
  return n;
}

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
