// Causal self-attention backward (head size 64) as one tcgen05 kernel: dQ, dK, dV from Q, K, V, dO, the forward's
// log-sum-exp and delta = rowsum(dO * O).
//
// One CTA owns one block of 128 keys of one (batch, head) and walks the query blocks from its diagonal to the end
// of the sequence.  Per pair (query block i, key block j), five MMAs with fp32 accumulators in tensor memory:
//
//   S  = Q_i K_j^T            dP = dO_i V_j^T                       (128 x 128 each; read by the softmax warps)
//   dV += P^T dO_i            dK += dS^T Q_i                        (128 keys x 64, accumulated over i, read once)
//   dQ_ij = dS K_j                                                  (128 queries x 64, added to a fp32 dQ buffer)
//
// with P = exp(scale S - lse) and dS = scale P (dP - delta) computed by eight warps (two threads per query row, 64
// keys each) and written as bf16 into two shared-memory tiles laid out [query][key] with the 128-byte swizzle: the
// tensor core reads them K-major for dS K_j and MN-major (transposed) for P^T dO_i and dS^T Q_i, so nothing is
// transposed by hand.  Q_i and dO_i arrive by TMA through a two-stage ring, K_j and V_j once.  S and dP of the next
// pair are issued as soon as the softmax warps have read the current ones.
//
// dQ receives contributions from every key block: each CTA adds its 128 x 64 tile to a fp32 buffer with vector
// reductions (red.global.add.v4.f32), so the low bits of dQ depend on the order in which CTAs arrive; dK and dV are
// bit-reproducible.  Every wait is bounded; a CTA that gives up records where and frees its tensor memory.
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

namespace attnb {
using namespace attn_util;

constexpr int BLK = 128, D = 64, THREADS = 320, UMMA_K = 16;
constexpr int TILE = BLK * D * 2;                             // a 128 x 64 bf16 tile: 16 KB
constexpr int K_OFF = 0, V_OFF = TILE, Q_OFF = 2 * TILE, DO_OFF = 4 * TILE, P_OFF = 6 * TILE, DS_OFF = 8 * TILE;
constexpr int SMEM_TILES = 10 * TILE;                         // K, V, Q x 2, dO x 2, P (32 KB), dS (32 KB)
constexpr int SMEM_SHARED = 256;
constexpr int TMEM_COLS = 512;                                // S 0, dP 128, dV 256, dK 320, dQ 384
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;

struct alignas(128) Shared {
  uint64_t kv_full, qd_full[2], qd_empty[2], sdp_full, sdp_empty, pds_full, dq_full, dq_empty, all_done;
  uint32_t tmem_base;
  int error;
};
static_assert(sizeof(Shared) <= SMEM_SHARED, "barrier block");

struct Params {
  int B, T, H, blocks;
  float scale, scale_log2;
  const float* lse;            // [B, H, T], natural log
  const float* delta;          // [B, H, T]
  float* dq_acc;               // [B * T, H * 64] fp32, zeroed by the caller
  __nv_bfloat16* dk;           // [B * T, ld_dkv], head h at columns h * 64
  __nv_bfloat16* dv;
  int ld_dkv;
  int* status;
};

__device__ __forceinline__ void fail(Shared* sh, const Params& p, int where) {
  atomicExch(&sh->error, where);
  if (p.status) atomicCAS(p.status, 0, 3100 + where);
}

#define ATTNB_WAIT(bar, parity, where) \
  do { if (!sm100::mbar_wait((bar), (parity), kWaitBudgetNs) || sh->error) { fail(sh, p, (where)); return; } } while (0)

__device__ void producer(Shared* sh, unsigned char* tiles, const Params& p, const CUtensorMap* mq, const CUtensorMap* mk,
                         const CUtensorMap* mv, const CUtensorMap* mdo, int b, int h, int jblk) {
  const int row0 = b * p.T;
  sm100::mbar_expect_tx(&sh->kv_full, 2 * TILE);
  sm100::tma_load_2d(tiles + K_OFF, mk, h * D, row0 + jblk * BLK, &sh->kv_full);
  sm100::tma_load_2d(tiles + V_OFF, mv, h * D, row0 + jblk * BLK, &sh->kv_full);
  int n = 0;
  for (int i = jblk; i < p.blocks; ++i, ++n) {
    const int st = n & 1;
    if (n >= 2) ATTNB_WAIT(&sh->qd_empty[st], ((n >> 1) - 1) & 1, 1);
    sm100::mbar_expect_tx(&sh->qd_full[st], 2 * TILE);
    sm100::tma_load_2d(tiles + Q_OFF + st * TILE, mq, h * D, row0 + i * BLK, &sh->qd_full[st]);
    sm100::tma_load_2d(tiles + DO_OFF + st * TILE, mdo, h * D, row0 + i * BLK, &sh->qd_full[st]);
  }
}

__device__ void mma_issuer(Shared* sh, unsigned char* tiles, const Params& p, int jblk) {
  const uint32_t t_s = sh->tmem_base, t_dp = t_s + 128, t_dv = t_s + 256, t_dk = t_s + 320, t_dq = t_s + 384;
  const uint32_t k_addr = sm100::smem_u32(tiles + K_OFF), v_addr = sm100::smem_u32(tiles + V_OFF);
  const uint32_t p_addr = sm100::smem_u32(tiles + P_OFF), ds_addr = sm100::smem_u32(tiles + DS_OFF);
  constexpr uint32_t idesc_s = sm100::make_idesc_f16(BLK, BLK, true);                 // both operands K-major
  constexpr uint32_t idesc_t = sm100::make_idesc_f16(BLK, D, true, true, true);       // A and B MN-major (transposed reads)
  constexpr uint32_t idesc_q = sm100::make_idesc_f16(BLK, D, true, true, false);      // A K-major, B MN-major
  const int pairs = p.blocks - jblk;
  auto issue_sdp = [&](int n) {
    const uint32_t q_addr = sm100::smem_u32(tiles + Q_OFF + (n & 1) * TILE), do_addr = sm100::smem_u32(tiles + DO_OFF + (n & 1) * TILE);
#pragma unroll
    for (int k = 0; k < D / UMMA_K; ++k)
      sm100::umma_f16(t_s, sm100::make_desc_sw128(q_addr + k * UMMA_K * 2), sm100::make_desc_sw128(k_addr + k * UMMA_K * 2),
                      idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
    for (int k = 0; k < D / UMMA_K; ++k)
      sm100::umma_f16(t_dp, sm100::make_desc_sw128(do_addr + k * UMMA_K * 2), sm100::make_desc_sw128(v_addr + k * UMMA_K * 2),
                      idesc_s, k > 0 ? 1u : 0u);
    sm100::umma_commit(&sh->sdp_full);
  };
  ATTNB_WAIT(&sh->kv_full, 0, 2);
  ATTNB_WAIT(&sh->qd_full[0], 0, 3);
  sm100::tc_fence_after();
  issue_sdp(0);
  for (int n = 0; n < pairs; ++n) {
    if (n + 1 < pairs) {                 // S and dP of the next pair, as soon as this pair's have been read
      ATTNB_WAIT(&sh->sdp_empty, n & 1, 4);
      ATTNB_WAIT(&sh->qd_full[(n + 1) & 1], ((n + 1) >> 1) & 1, 5);
      sm100::tc_fence_after();
      issue_sdp(n + 1);
    }
    ATTNB_WAIT(&sh->pds_full, n & 1, 6);
    if (n > 0) ATTNB_WAIT(&sh->dq_empty, (n - 1) & 1, 7);        // the previous dQ tile has been read
    sm100::tc_fence_after();
    const uint32_t q_addr = sm100::smem_u32(tiles + Q_OFF + (n & 1) * TILE), do_addr = sm100::smem_u32(tiles + DO_OFF + (n & 1) * TILE);
    // K dimension = the 128 queries of the block: 16 rows of 128 bytes per step in every [query][...] tile
#pragma unroll
    for (int k = 0; k < BLK / UMMA_K; ++k) {
      const uint64_t a_p = sm100::make_desc_sw128_mn(p_addr + k * UMMA_K * 128, TILE, 1024);     // P^T: keys x queries
      const uint64_t b_do = sm100::make_desc_sw128_mn(do_addr + k * UMMA_K * 128, TILE, 1024);   // dO: queries x d
      sm100::umma_f16(t_dv, a_p, b_do, idesc_t, (n > 0 || k > 0) ? 1u : 0u);
    }
#pragma unroll
    for (int k = 0; k < BLK / UMMA_K; ++k) {
      const uint64_t a_ds = sm100::make_desc_sw128_mn(ds_addr + k * UMMA_K * 128, TILE, 1024);   // dS^T
      const uint64_t b_q = sm100::make_desc_sw128_mn(q_addr + k * UMMA_K * 128, TILE, 1024);     // Q: queries x d
      sm100::umma_f16(t_dk, a_ds, b_q, idesc_t, (n > 0 || k > 0) ? 1u : 0u);
    }
    // K dimension = the 128 keys: dS read K-major (two chunks of 64 keys), K_j read MN-major
#pragma unroll
    for (int k = 0; k < BLK / UMMA_K; ++k) {
      const uint64_t a_ds = sm100::make_desc_sw128(ds_addr + (k >> 2) * TILE + (k & 3) * UMMA_K * 2);
      const uint64_t b_k = sm100::make_desc_sw128_mn(k_addr + k * UMMA_K * 128, TILE, 1024);
      sm100::umma_f16(t_dq, a_ds, b_k, idesc_q, k > 0 ? 1u : 0u);
    }
    sm100::umma_commit(&sh->dq_full);                // also: P, dS and this stage of Q / dO are free again
    sm100::umma_commit(&sh->qd_empty[n & 1]);
  }
  sm100::umma_commit(&sh->all_done);
}

// Two threads per query row (warps with the same warp & 3 share 32 tensor-memory lanes); `half` picks 64 of the 128
// keys of the pair and 32 of the 64 columns of dQ (and, at the end, of dK / dV, where the rows are keys).
__device__ void softmax_rows(Shared* sh, unsigned char* tiles, const Params& p, int b, int h, int jblk, int quarter, int half,
                             int lane) {
  const int row = quarter * 32 + lane;
  const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
  const uint32_t t_s = sh->tmem_base + lane_base + half * 64, t_dp = t_s + 128;
  const uint32_t t_dv = sh->tmem_base + lane_base + 256 + half * 32, t_dk = t_dv + 64, t_dq = t_dv + 128;
  unsigned char* p_row = tiles + P_OFF + half * TILE + row * 128;
  unsigned char* ds_row = tiles + DS_OFF + half * TILE + row * 128;
  const float c2 = p.scale_log2, scale = p.scale;
  const int last_row = quarter * 32 + 31;
  uint32_t rs[32], rp[32];
  int n = 0;
  for (int i = jblk; i < p.blocks; ++i, ++n) {
    const bool diag = i == jblk;
    const size_t stat = ((size_t)b * p.H + h) * p.T + (size_t)i * BLK + row;
    const float nl2 = -p.lse[stat] * 1.4426950408889634f, delta = p.delta[stat];
    ATTNB_WAIT(&sh->sdp_full, n & 1, 8);
    sm100::tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      const int key0 = half * 64 + c * 32;
      const bool masked = diag && key0 > last_row;         // warp-uniform: every key of the chunk is after the query
      if (!masked) {
        sm100::tmem_ld_32x32(t_s + c * 32, rs);
        sm100::tmem_ld_32x32(t_dp + c * 32, rp);
        sm100::tmem_ld_wait();
      }
      if (c == 1) {                                       // S and dP are in registers: the next pair may overwrite them
        sm100::tc_fence_before();
        sm100::mbar_arrive(&sh->sdp_empty);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        uint32_t wp[4] = {0u, 0u, 0u, 0u}, wd[4] = {0u, 0u, 0u, 0u};
        if (!masked) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int e = u * 8 + 2 * q;
            float p0 = ex2(fmaf(__uint_as_float(rs[e]), c2, nl2)), p1 = ex2(fmaf(__uint_as_float(rs[e + 1]), c2, nl2));
            if (diag) {
              if (key0 + e > row) p0 = 0.f;
              if (key0 + e + 1 > row) p1 = 0.f;
            }
            const float d0 = p0 * (__uint_as_float(rp[e]) - delta) * scale, d1 = p1 * (__uint_as_float(rp[e + 1]) - delta) * scale;
            __nv_bfloat162 hp = __floats2bfloat162_rn(p0, p1), hd = __floats2bfloat162_rn(d0, d1);
            wp[q] = *reinterpret_cast<uint32_t*>(&hp);
            wd[q] = *reinterpret_cast<uint32_t*>(&hd);
          }
        }
        const int off = ((c * 4 + u) ^ (row & 7)) << 4;
        *reinterpret_cast<uint4*>(p_row + off) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
        *reinterpret_cast<uint4*>(ds_row + off) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
      }
    }
    sm100::fence_proxy_async_smem();                      // the MMAs read P and dS through the async proxy
    sm100::mbar_arrive(&sh->pds_full);
    // this pair's share of dQ: 32 columns of this thread's query row, added to the fp32 buffer
    ATTNB_WAIT(&sh->dq_full, n & 1, 9);
    sm100::tc_fence_after();
    sm100::tmem_ld_32x32(t_dq, rs);
    sm100::tmem_ld_wait();
    sm100::tc_fence_before();
    sm100::mbar_arrive(&sh->dq_empty);
    float* dq = p.dq_acc + ((size_t)b * p.T + (size_t)i * BLK + row) * (p.H * D) + h * D + half * 32;
#pragma unroll
    for (int u = 0; u < 8; ++u)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + 4 * u), "f"(__uint_as_float(rs[4 * u])),
                   "f"(__uint_as_float(rs[4 * u + 1])), "f"(__uint_as_float(rs[4 * u + 2])), "f"(__uint_as_float(rs[4 * u + 3]))
                   : "memory");
  }
  // dV and dK of this key block: the accumulator rows are keys now
  ATTNB_WAIT(&sh->all_done, 0, 10);
  sm100::tc_fence_after();
  const size_t grow = (size_t)b * p.T + (size_t)jblk * BLK + row;
  auto store = [&](uint32_t taddr, __nv_bfloat16* base) {
    sm100::tmem_ld_32x32(taddr, rs);
    sm100::tmem_ld_wait();
    __nv_bfloat16* o = base + grow * p.ld_dkv + h * D + half * 32;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(rs[u * 8 + 2 * e]), __uint_as_float(rs[u * 8 + 2 * e + 1]));
        w[e] = *reinterpret_cast<uint32_t*>(&hh);
      }
      *reinterpret_cast<uint4*>(o + u * 8) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  };
  store(t_dv, p.dv);
  store(t_dk, p.dk);
}

__global__ void __launch_bounds__(THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do, const Params p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = smem_raw;
  Shared* sh = (Shared*)(smem_raw + SMEM_TILES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // key blocks near the start of the sequence meet the most query blocks: they start first
  const int bh = blockIdx.x % (p.B * p.H);
  const int jblk = blockIdx.x / (p.B * p.H);
  const int b = bh / p.H, h = bh - b * p.H;
  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(&map_q);
    sm100::tma_prefetch_desc(&map_k);
    sm100::tma_prefetch_desc(&map_v);
    sm100::tma_prefetch_desc(&map_do);
    sm100::mbar_init(&sh->kv_full, 1);
    for (int s = 0; s < 2; ++s) { sm100::mbar_init(&sh->qd_full[s], 1); sm100::mbar_init(&sh->qd_empty[s], 1); }
    sm100::mbar_init(&sh->sdp_full, 1);
    sm100::mbar_init(&sh->sdp_empty, 256);
    sm100::mbar_init(&sh->pds_full, 256);
    sm100::mbar_init(&sh->dq_full, 1);
    sm100::mbar_init(&sh->dq_empty, 256);
    sm100::mbar_init(&sh->all_done, 1);
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

  const bool aligned = (sm100::smem_u32(tiles) & 1023u) == 0;     // the swizzled tiles need a 1024-byte aligned base
  if (!aligned) {
    if (threadIdx.x == 0) fail(sh, p, 11);
  } else if (warp == 0) {
    if (sm100::elect_one()) producer(sh, tiles, p, &map_q, &map_k, &map_v, &map_do, b, h, jblk);
  } else if (warp == 1) {
    if (sm100::elect_one()) mma_issuer(sh, tiles, p, jblk);
  } else {
    softmax_rows(sh, tiles, p, b, h, jblk, warp & 3, (warp - 2) >> 2, lane);
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

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d]: one thread per (row, head), 128-byte reads.
__global__ void __launch_bounds__(256)
attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, int64_t ld_o, int64_t ld_do,
                       float* __restrict__ delta, int B, int T, int H) {
  const long long total = (long long)B * T * H;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const int h = (int)(idx % H);
    const long long r = idx / H;                                 // b * T + t
    const uint4* po = reinterpret_cast<const uint4*>(o + r * ld_o + h * D);
    const uint4* pd = reinterpret_cast<const uint4*>(dout + r * ld_do + h * D);
    float acc = 0.f;
#pragma unroll
    for (int u = 0; u < D / 8; ++u) {
      const uint4 a = __ldg(po + u), g = __ldg(pd + u);
      const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wg[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc = fmaf(__uint_as_float(wa[e] << 16), __uint_as_float(wg[e] << 16), acc);
        acc = fmaf(__uint_as_float(wa[e] & 0xffff0000u), __uint_as_float(wg[e] & 0xffff0000u), acc);
      }
    }
    const int b = (int)(r / T), t = (int)(r - (long long)b * T);
    delta[((size_t)b * H + h) * T + t] = acc;
  }
}

}  // namespace attnb

static int* attnb_status_word(int** host_out = nullptr) {
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

// Gradients of tmpi_attention_fwd.  q, k, v as there (common row pitch ld_qkv); o and dout are [B * T, H * 64] with
// their own pitches; lse [B, H, T] from the forward; delta [B, H, T] is scratch (written here); dq_acc is a zeroed
// fp32 [B * T, H * 64] buffer that receives dQ; dk and dv are bf16 [B * T, ld_dkv] (for instance the K and V column
// blocks of the gradient of a packed QKV projection).
int tmpi_attention_bwd(const void* q, const void* k, const void* v, int64_t ld_qkv, const void* o, int64_t ld_o,
                       const void* dout, int64_t ld_do, const float* lse, float* delta, float* dq_acc, void* dk, void* dv,
                       int64_t ld_dkv, int B, int T, int H, float scale, void* stream) {
  if (B < 1 || H < 1 || T < 128 || T % 128) return fail(TMPI_ERR_UNSUPPORTED, "attention backward: T=%d must be a positive multiple of 128", T);
  if (ld_dkv % 8 || ((uintptr_t)dk & 15) || ((uintptr_t)dv & 15) || ((uintptr_t)dq_acc & 15) || ld_o % 8 || ld_do % 8 ||
      ((uintptr_t)o & 15) || ((uintptr_t)dout & 15))
    return fail(TMPI_ERR_INVALID, "attention backward: operands must be 16-byte aligned with pitches that are multiples of 8");
  if ((int64_t)B * H * (T / 128) > 0x7fffffffLL) return fail(TMPI_ERR_INVALID, "attention backward: too many blocks");
  cudaStream_t s = (cudaStream_t)stream;
  const long long rows_heads = (long long)B * T * H;
  const int dgrid = (int)std::min<long long>((rows_heads + 255) / 256, 148 * 8);
  attnb::attention_delta_kernel<<<dgrid, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, ld_o, ld_do, delta, B, T, H);
  CUtensorMap mq, mk, mv, mdo;
  int st;
  const uint64_t rows = (uint64_t)B * T, cols = (uint64_t)H * attnb::D;
  if ((st = make_tmap_bf16(&mq, q, rows, cols, (uint64_t)ld_qkv, 128))) return st;
  if ((st = make_tmap_bf16(&mk, k, rows, cols, (uint64_t)ld_qkv, 128))) return st;
  if ((st = make_tmap_bf16(&mv, v, rows, cols, (uint64_t)ld_qkv, 128))) return st;
  if ((st = make_tmap_bf16(&mdo, dout, rows, cols, (uint64_t)ld_do, 128))) return st;
  const int smem = attnb::SMEM_TILES + attnb::SMEM_SHARED;
  cudaError_t ae = cudaFuncSetAttribute(attnb::attention_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (ae != cudaSuccess) return fail(TMPI_ERR_CUDA, "attention backward: shared memory attribute: %s", cudaGetErrorString(ae));
  attnb::Params p;
  p.B = B; p.T = T; p.H = H; p.blocks = T / attnb::BLK;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.ld_dkv = (int)ld_dkv;
  p.status = attnb_status_word();
  attnb::attention_bwd_kernel<<<B * H * p.blocks, attnb::THREADS, smem, s>>>(mq, mk, mv, mdo, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "attention backward launch: %s", cudaGetErrorString(e));
}

// Non-zero after a CTA of the attention backward gave up on a bounded wait (3100 + the point where); clears it.
int tmpi_attention_bwd_status(void) {
  int* host = nullptr;
  attnb_status_word(&host);
  if (!host) return 0;
  int v = *(volatile int*)host;
  if (v) *(volatile int*)host = 0;
  return v;
}

}  // extern "C"
