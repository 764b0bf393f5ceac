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
// with P = exp(scale S - lse) and dS = scale P (dP - delta) computed by sixteen warps (four threads per query row, 32
// keys each) and written as bf16 into two shared-memory tiles laid out [query][key] with the 128-byte swizzle: the
// tensor core reads them K-major for dS K_j and MN-major (transposed) for P^T dO_i and dS^T Q_i, so nothing is
// transposed by hand.  Q_i and dO_i arrive by TMA through a two-stage ring, K_j and V_j once.  S and dP of the next
// pair are issued as soon as the softmax warps have read the current ones, and P and dS are double-buffered, so the
// softmax of pair n + 1 runs while the tensor core works on the three products of pair n.
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

constexpr int BLK = 128, D = 64, SOFTMAX_WARPS = 16, THREADS = 64 + SOFTMAX_WARPS * 32, UMMA_K = 16;
constexpr int TILE = BLK * D * 2;                             // a 128 x 64 bf16 tile: 16 KB
constexpr int K_OFF = 0, V_OFF = TILE, Q_OFF = 2 * TILE, DO_OFF = 4 * TILE, P_OFF = 6 * TILE, DS_OFF = 10 * TILE;
constexpr int SMEM_TILES = 14 * TILE;                         // K, V, Q x 2, dO x 2, P x 2 (32 KB each), dS x 2: 224 KB
constexpr int SMEM_SHARED = 256;
constexpr int TMEM_COLS = 512;                                // S 0, dP 128, dV 256, dK 320, dQ 384
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;

struct alignas(128) Shared {
  uint64_t kv_full, qd_full[2], qd_empty[2], sdp_full, sdp_empty, pds_full[2], dq_full, dq_empty, all_done;
  uint32_t tmem_base;
  int error;
};
static_assert(sizeof(Shared) <= SMEM_SHARED, "barrier block");

struct Params {
  int B, T, H, blocks;
  float scale, scale_log2;
  const float* lse;            // [B, H, T], natural log
  const float* delta;          // [B, H, T]
  float* dq_acc;               // [B * T, H * 64] fp32, cleared by the delta kernel
  __nv_bfloat16* dk;           // [B * T, ld_dkv], head h at columns h * 64
  __nv_bfloat16* dv;
  int ld_dkv;
  int* status;
  unsigned long long* trace;   // optional: time stamps of the phases of CTA 0 (see tmpi_attention_bwd_set_trace)
};

__device__ __forceinline__ void fail(Shared* sh, const Params& p, int where) {
  atomicExch(&sh->error, where);
  if (p.status) atomicCAS(p.status, 0, 3100 + where);
}

// Phase time stamps of one CTA for tuning: slot = (pair * 16 + event), written by one thread per role.
__device__ __forceinline__ void stamp(const Params& p, int n, int ev) {
  if (p.trace && blockIdx.x == 0) p.trace[n * 16 + ev] = sm100::now_ns();
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
  constexpr uint32_t idesc_s = sm100::make_idesc_f16(BLK, BLK, true);                 // both operands K-major
  constexpr uint32_t idesc_t = sm100::make_idesc_f16(BLK, D, true, true, true);       // A and B MN-major (transposed reads)
  constexpr uint32_t idesc_q = sm100::make_idesc_f16(BLK, D, true, true, false);      // A K-major, B MN-major
  const int pairs = p.blocks - jblk;
  // Descriptors: one per operand tile, built once; a slice further into the tile only adds to the address field
  // (bytes / 16 in the low 14 bits; shared memory is far smaller than the field, so nothing carries out of it).
  auto at = [](uint64_t desc, uint32_t bytes) { return desc + (uint64_t)(bytes >> 4); };
  const uint64_t k_kmaj = sm100::make_desc_sw128(k_addr), v_kmaj = sm100::make_desc_sw128(v_addr);
  const uint64_t k_mn = sm100::make_desc_sw128_mn(k_addr, TILE, 1024);
  uint64_t q_kmaj[2], do_kmaj[2], q_mn[2], do_mn[2], p_mn[2], ds_mn[2], ds_kmaj[2];
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const uint32_t q_addr = sm100::smem_u32(tiles + Q_OFF + s * TILE), do_addr = sm100::smem_u32(tiles + DO_OFF + s * TILE);
    const uint32_t p_addr = sm100::smem_u32(tiles + P_OFF + s * 2 * TILE), ds_addr = sm100::smem_u32(tiles + DS_OFF + s * 2 * TILE);
    q_kmaj[s] = sm100::make_desc_sw128(q_addr);
    do_kmaj[s] = sm100::make_desc_sw128(do_addr);
    q_mn[s] = sm100::make_desc_sw128_mn(q_addr, TILE, 1024);
    do_mn[s] = sm100::make_desc_sw128_mn(do_addr, TILE, 1024);
    p_mn[s] = sm100::make_desc_sw128_mn(p_addr, TILE, 1024);
    ds_mn[s] = sm100::make_desc_sw128_mn(ds_addr, TILE, 1024);
    ds_kmaj[s] = sm100::make_desc_sw128(ds_addr);
  }
  auto issue_sdp = [&](int n) {
    const uint64_t dq = (n & 1) ? q_kmaj[1] : q_kmaj[0], dd = (n & 1) ? do_kmaj[1] : do_kmaj[0];
#pragma unroll
    for (int k = 0; k < D / UMMA_K; ++k)
      sm100::umma_f16(t_s, at(dq, k * UMMA_K * 2), at(k_kmaj, k * UMMA_K * 2), idesc_s, k > 0 ? 1u : 0u);
#pragma unroll
    for (int k = 0; k < D / UMMA_K; ++k)
      sm100::umma_f16(t_dp, at(dd, k * UMMA_K * 2), at(v_kmaj, k * UMMA_K * 2), idesc_s, k > 0 ? 1u : 0u);
    sm100::umma_commit(&sh->sdp_full);
  };
  auto issue_products = [&](int n) {
    const int s = n & 1;
    const uint64_t a_p = s ? p_mn[1] : p_mn[0], a_ds = s ? ds_mn[1] : ds_mn[0], a_dsk = s ? ds_kmaj[1] : ds_kmaj[0];
    const uint64_t b_do = s ? do_mn[1] : do_mn[0], b_q = s ? q_mn[1] : q_mn[0];
    const uint32_t acc = n > 0 ? 1u : 0u;
    // K dimension = the 128 queries of the block: 16 rows of 128 bytes per step in every [query][...] tile
#pragma unroll
    for (int k = 0; k < BLK / UMMA_K; ++k)      // dV += P^T dO
      sm100::umma_f16(t_dv, at(a_p, k * UMMA_K * 128), at(b_do, k * UMMA_K * 128), idesc_t, k > 0 ? 1u : acc);
#pragma unroll
    for (int k = 0; k < BLK / UMMA_K; ++k)      // dK += dS^T Q
      sm100::umma_f16(t_dk, at(a_ds, k * UMMA_K * 128), at(b_q, k * UMMA_K * 128), idesc_t, k > 0 ? 1u : acc);
    // K dimension = the 128 keys: dS read K-major (two chunks of 64 keys), K_j read MN-major
#pragma unroll
    for (int k = 0; k < BLK / UMMA_K; ++k)      // dQ_ij = dS K_j
      sm100::umma_f16(t_dq, at(a_dsk, (k >> 2) * TILE + (k & 3) * UMMA_K * 2), at(k_mn, k * UMMA_K * 128), idesc_q, k > 0 ? 1u : 0u);
    sm100::umma_commit(&sh->dq_full);                // also: these P / dS buffers and this stage of Q / dO are free again
    sm100::umma_commit(&sh->qd_empty[s]);
  };
  ATTNB_WAIT(&sh->kv_full, 0, 2);
  ATTNB_WAIT(&sh->qd_full[0], 0, 3);
  sm100::tc_fence_after();
  issue_sdp(0);
  int next_sdp = 1;                                  // the next pair whose S and dP are to be issued
  for (int n = 0; n < pairs; ++n) {
    // Two things may become possible, in either order: S and dP of pair n + 1 (its Q and dO have landed and the
    // softmax warps have read pair n's), and the three products of pair n (its P and dS are written and the previous
    // dQ tile has been collected).  Whichever is ready goes first, so a late TMA load does not hold up the products.
    const unsigned long long t0 = sm100::now_ns();
    bool products_done = false;
    unsigned spins = 0;
    while (!products_done || (next_sdp == n + 1 && n + 1 < pairs)) {
      if (next_sdp == n + 1 && n + 1 < pairs && sm100::mbar_try_wait(&sh->sdp_empty, n & 1) &&
          sm100::mbar_try_wait(&sh->qd_full[(n + 1) & 1], ((n + 1) >> 1) & 1)) {
        if (!products_done) stamp(p, n, 8);
        sm100::tc_fence_after();
        issue_sdp(n + 1);
        ++next_sdp;
        stamp(p, n, 9);
      } else if (!products_done && sm100::mbar_try_wait(&sh->pds_full[n & 1], (n >> 1) & 1) &&
                 (n == 0 || sm100::mbar_try_wait(&sh->dq_empty, (n - 1) & 1))) {
        stamp(p, n, 10);
        sm100::tc_fence_after();
        issue_products(n);
        products_done = true;
        stamp(p, n, 12);
      } else if ((++spins & 255u) == 0 && (sm100::now_ns() - t0 > kWaitBudgetNs || sh->error)) {
        fail(sh, p, 6);
        return;
      }
    }
  }
  sm100::umma_commit(&sh->all_done);
}

// Four threads per query row (warps with the same warp & 3 share 32 tensor-memory lanes); `part` picks 32 of the 128
// keys of the pair and 16 of the 64 columns of dQ (and, at the end, of dK / dV, where the rows are keys).
__device__ void softmax_rows(Shared* sh, unsigned char* tiles, const Params& p, int b, int h, int jblk, int quarter, int part,
                             int lane) {
  const int row = quarter * 32 + lane;
  const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
  const uint32_t t_s = sh->tmem_base + lane_base + part * 32, t_dp = t_s + 128;
  const uint32_t t_dv = sh->tmem_base + lane_base + 256 + part * 16, t_dk = t_dv + 64, t_dq = t_dv + 128;
  const float c2 = p.scale_log2, scale = p.scale;
  const int key0 = part * 32;
  const int tile_off = (part >> 1) * TILE + row * 128;    // which 64-key chunk of the [query][key] tiles
  const int unit0 = (part & 1) * 4;                       // first 16-byte unit of this thread's keys in the row
  const bool masked_diag = key0 > quarter * 32 + 31;      // on the diagonal block: every key of the chunk is after the query
  uint32_t rs[32], rp[32];
  const int pairs = p.blocks - jblk;
  const bool tracer = row == 0 && part == 0;
  // P and dS of pair n (query block jblk + n) into the buffers n & 1
  auto softmax_pair = [&](int n) -> bool {
    const int i = jblk + n;
    const bool diag = n == 0;
    unsigned char* p_row = tiles + P_OFF + (n & 1) * 2 * TILE + tile_off;
    unsigned char* ds_row = tiles + DS_OFF + (n & 1) * 2 * TILE + tile_off;
    const size_t stat = ((size_t)b * p.H + h) * p.T + (size_t)i * BLK + row;
    const float nl2 = -p.lse[stat] * 1.4426950408889634f, delta = p.delta[stat];
    if (tracer) stamp(p, n, 0);
    if (!sm100::mbar_wait(&sh->sdp_full, n & 1, kWaitBudgetNs) || sh->error) { fail(sh, p, 8); return false; }
    if (tracer) stamp(p, n, 1);
    sm100::tc_fence_after();
    const bool masked = diag && masked_diag;               // warp-uniform: nothing to load or exponentiate
    if (!masked) {
      sm100::tmem_ld_32x32(t_s, rs);
      sm100::tmem_ld_32x32(t_dp, rp);
      sm100::tmem_ld_wait();
    }
    sm100::tc_fence_before();                              // S and dP are in registers: the next pair may overwrite them
    sm100::mbar_arrive(&sh->sdp_empty);
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
      const int off = ((unit0 + u) ^ (row & 7)) << 4;
      *reinterpret_cast<uint4*>(p_row + off) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
      *reinterpret_cast<uint4*>(ds_row + off) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
    }
    sm100::fence_proxy_async_smem();                      // the MMAs read P and dS through the async proxy
    sm100::mbar_arrive(&sh->pds_full[n & 1]);
    if (tracer) stamp(p, n, 2);
    return true;
  };
  if (!softmax_pair(0)) return;
  uint32_t rq[16];
  for (int n = 0; n < pairs; ++n) {
    // the next pair's P and dS while the tensor core multiplies this pair's (its buffers were freed by the MMAs of
    // pair n - 1, whose dQ this thread has already collected)
    if (n + 1 < pairs && !softmax_pair(n + 1)) return;
    // this pair's share of dQ: 16 columns of this thread's query row, added to the fp32 buffer
    if (tracer) stamp(p, n, 3);
    ATTNB_WAIT(&sh->dq_full, n & 1, 9);
    if (tracer) stamp(p, n, 4);
    sm100::tc_fence_after();
    sm100::tmem_ld_32x16(t_dq, rq);
    sm100::tmem_ld_wait();
    sm100::tc_fence_before();
    sm100::mbar_arrive(&sh->dq_empty);
    float* dq = p.dq_acc + ((size_t)b * p.T + (size_t)(jblk + n) * BLK + row) * (p.H * D) + h * D + part * 16;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dq + 4 * u), "f"(__uint_as_float(rq[4 * u])),
                   "f"(__uint_as_float(rq[4 * u + 1])), "f"(__uint_as_float(rq[4 * u + 2])), "f"(__uint_as_float(rq[4 * u + 3]))
                   : "memory");
    if (tracer) stamp(p, n, 5);
  }
  // dV and dK of this key block: the accumulator rows are keys now
  ATTNB_WAIT(&sh->all_done, 0, 10);
  sm100::tc_fence_after();
  const size_t grow = (size_t)b * p.T + (size_t)jblk * BLK + row;
  auto store = [&](uint32_t taddr, __nv_bfloat16* base) {
    sm100::tmem_ld_32x16(taddr, rq);
    sm100::tmem_ld_wait();
    __nv_bfloat16* o = base + grow * p.ld_dkv + h * D + part * 16;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      uint32_t w[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(rq[u * 8 + 2 * e]), __uint_as_float(rq[u * 8 + 2 * e + 1]));
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
    sm100::mbar_init(&sh->sdp_empty, SOFTMAX_WARPS * 32);
    for (int s = 0; s < 2; ++s) sm100::mbar_init(&sh->pds_full[s], SOFTMAX_WARPS * 32);
    sm100::mbar_init(&sh->dq_full, 1);
    sm100::mbar_init(&sh->dq_empty, SOFTMAX_WARPS * 32);
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

// delta[b, h, t] = sum_d dO[b, t, h, d] * O[b, t, h, d]: eight threads per (row, head), one 16-byte load of O and of
// dO each (a warp reads four whole 128-byte lines of each tensor per instruction), three shuffles; the same threads
// clear their 64 entries of the fp32 dQ buffer, so the caller need not.
__global__ void __launch_bounds__(256)
attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, int64_t ld_o, int64_t ld_do,
                       float* __restrict__ delta, float* __restrict__ dq_acc, int B, int T, int H) {
  const long long total = (long long)B * T * H;                  // (row, head) pairs; blockDim.x / 8 of them per block and step
  const int sub = threadIdx.x & 7;
  for (long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 3; idx < total;
       idx += ((long long)gridDim.x * blockDim.x) >> 3) {
    const int h = (int)(idx % H);
    const long long r = idx / H;                                 // b * T + t
    const uint4 a = __ldg(reinterpret_cast<const uint4*>(o + r * ld_o + h * D) + sub);
    const uint4 g = __ldg(reinterpret_cast<const uint4*>(dout + r * ld_do + h * D) + sub);
    const uint32_t wa[4] = {a.x, a.y, a.z, a.w}, wg[4] = {g.x, g.y, g.z, g.w};
    float acc = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      acc = fmaf(__uint_as_float(wa[e] << 16), __uint_as_float(wg[e] << 16), acc);
      acc = fmaf(__uint_as_float(wa[e] & 0xffff0000u), __uint_as_float(wg[e] & 0xffff0000u), acc);
    }
    const unsigned group = 0xffu << (threadIdx.x & 24);          // the eight lanes of this (row, head)
    acc += __shfl_xor_sync(group, acc, 1);
    acc += __shfl_xor_sync(group, acc, 2);
    acc += __shfl_xor_sync(group, acc, 4);
    if (sub == 0) {
      const int b = (int)(r / T), t = (int)(r - (long long)b * T);
      delta[((size_t)b * H + h) * T + t] = acc;
    }
    float4* z = reinterpret_cast<float4*>(dq_acc + (size_t)r * (H * D) + h * D) + sub * 2;
    z[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    z[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// dq[r, c] = bf16(dq_acc[r, c]): the fp32 sums of the reductions rounded into the Q block of the packed gradient.
__global__ void __launch_bounds__(256)
attention_dq_round_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, int64_t ld_dq, long long rows, int cols) {
  const int groups = cols / 8;
  const long long total = rows * groups;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / groups;
    const int c = (int)(idx - r * groups) * 8;
    const float4 a = *reinterpret_cast<const float4*>(acc + r * cols + c), b = *reinterpret_cast<const float4*>(acc + r * cols + c + 4);
    __nv_bfloat162 h0 = __floats2bfloat162_rn(a.x, a.y), h1 = __floats2bfloat162_rn(a.z, a.w);
    __nv_bfloat162 h2 = __floats2bfloat162_rn(b.x, b.y), h3 = __floats2bfloat162_rn(b.z, b.w);
    uint4 u;
    u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
    u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
    *reinterpret_cast<uint4*>(dq + r * ld_dq + c) = u;
  }
}

}  // namespace attnb

static unsigned long long* g_attnb_trace = nullptr;

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
// their own pitches; lse [B, H, T] from the forward; delta [B, H, T] is scratch (written here); dq_acc is a fp32
// [B * T, H * 64] buffer (cleared here) that receives dQ; dq (optional), dk and dv are bf16 [B * T, ld_dkv] (for instance
// the column blocks of the gradient of a packed QKV projection): dk and dv are written by the main kernel, dq by a last
// pass that rounds dq_acc.
int tmpi_attention_bwd(const void* q, const void* k, const void* v, int64_t ld_qkv, const void* o, int64_t ld_o,
                       const void* dout, int64_t ld_do, const float* lse, float* delta, float* dq_acc, void* dq, void* dk,
                       void* dv, int64_t ld_dkv, int B, int T, int H, float scale, void* stream) {
  if (B < 1 || H < 1 || T < 128 || T % 128) return fail(TMPI_ERR_UNSUPPORTED, "attention backward: T=%d must be a positive multiple of 128", T);
  if (ld_dkv % 8 || ((uintptr_t)dk & 15) || ((uintptr_t)dv & 15) || ((uintptr_t)dq_acc & 15) || ld_o % 8 || ld_do % 8 ||
      ((uintptr_t)o & 15) || ((uintptr_t)dout & 15))
    return fail(TMPI_ERR_INVALID, "attention backward: operands must be 16-byte aligned with pitches that are multiples of 8");
  if ((int64_t)B * H * (T / 128) > 0x7fffffffLL) return fail(TMPI_ERR_INVALID, "attention backward: too many blocks");
  cudaStream_t s = (cudaStream_t)stream;
  const long long rows_heads = (long long)B * T * H;
  const int dgrid = (int)std::min<long long>((rows_heads * 8 + 255) / 256, 148 * 8);
  attnb::attention_delta_kernel<<<dgrid, 256, 0, s>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, ld_o, ld_do, delta, dq_acc, B, T, H);
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
  p.trace = g_attnb_trace;
  attnb::attention_bwd_kernel<<<B * H * p.blocks, attnb::THREADS, smem, s>>>(mq, mk, mv, mdo, p);
  if (dq) {
    if ((uintptr_t)dq & 15) return fail(TMPI_ERR_INVALID, "attention backward: dq must be 16-byte aligned");
    const long long groups = (long long)rows * (cols / 8);
    const int cgrid = (int)std::min<long long>((groups + 255) / 256, 148 * 8);
    attnb::attention_dq_round_kernel<<<cgrid, 256, 0, s>>>(dq_acc, (__nv_bfloat16*)dq, ld_dkv, (long long)rows, (int)cols);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "attention backward launch: %s", cudaGetErrorString(e));
}

// Tuning aid: with a device buffer of (T / 128) * 16 64-bit words, CTA 0 of every later launch (the first key block of
// the first batch and head, which meets every query block) records the time of each phase of each pair (ns):
// 0 waits for S and dP, 1 has them, 2 P and dS announced, 3 waits for dQ, 4 has it, 5 reductions issued; MMA thread:
// 8 S and dP were read, 9 next S and dP issued, 10 has P and dS, 11 dQ tile free, 12 three products issued.
void tmpi_attention_bwd_set_trace(void* device_buffer) { g_attnb_trace = (unsigned long long*)device_buffer; }

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
