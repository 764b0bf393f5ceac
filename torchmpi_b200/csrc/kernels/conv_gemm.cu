// Convolutions of channels-last bf16 activations as implicit GEMMs on the tcgen05 tensor cores.
//
//   forward   Y[p, co]  = sum_{tap, ci} X[pixel(p) + tap, ci] * W[co, tap, ci]
//   dgrad     dX[p, ci] = sum_{tap, co} dY[pixel(p) + tap, co] * W[co, flipped tap, ci]      (stride 1)
//   wgrad     dW[co, tap, ci] = sum_p dY[p, co] * X[pixel(p) + tap, ci]                       (split over p)
//
// p runs over the output pixels (n, ho, wo) in memory order, so Y, dX and dW are plain row-major
// matrices and no patch matrix is ever written.  A 1x1 / stride-1 convolution reads its activation
// with ordinary 2-D TMA tiles; every other shape reads it with im2col-mode TMA loads, which walk 128
// (or 64) consecutive filter positions and fetch one tap of each, with zeros outside the image.  The
// weight is read as it lies in a channels-last Conv2d parameter ([Cout, R, S, Cin]): K-major for
// forward, MN-major for dgrad.  wgrad reads both operands MN-major (pixels are its K).
//
// One persistent CTA per SM, 320 threads: a TMA producer warp, an MMA issuer warp (128 x N tiles,
// N <= 256, two accumulators in tensor memory) and eight epilogue warps in two groups, one group per
// accumulator.  Most of these products are bound by memory or by the latency of the loads, not by the
// tensor cores, so the shared memory goes to loads in flight: the ring has as many stages as fit
// (up to 12), and when one column tile covers the output and the whole weight fits beside five
// stages, the weight is loaded once and stays resident while only the activation streams.  The
// epilogue warps work independently (own staging tile, no barrier between warps), two tiles drain at a
// time.  Epilogues:
//   store    bf16 rows: each warp transposes its 32 x 64 slice through a swizzled staging tile and
//            writes full 128-byte lines; optionally the per-channel sum and sum of squares of the
//            stored values (the batch statistics of the batch-norm that follows, accumulated per lane
//            in registers over all tiles of the CTA and written as one partial row per CTA: no atomics,
//            fixed order), and optionally
//            "+ R" for a second gradient that flows into the same tensor (added to the rounded product,
//            as a separate accumulation kernel would);
//   split-K  fp32 partial tiles to a workspace, summed in slice order by a second small kernel
//            (deterministic).
// The three passes of a framework convolution go to library kernels; the reference itself has no
// convolution (its only model is nn.Linear, examples/mnist/mnist_allreduce.lua:31).
// Every mbarrier wait is bounded; a CTA that gives up records a status word, drains and returns.
#include <cuda_bf16.h>
#include <algorithm>
#include <cstring>
#include <mutex>
#include "sm100_ptx.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"

namespace tmpi {

int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
int gemm_sm_count();

namespace conv {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16, MAX_STAGES = 12, TMEM_COLS = 512;
constexpr int EPI_WARPS = 8, THREADS = 32 * (2 + EPI_WARPS);
constexpr int A_BYTES = BM * BK * 2;
constexpr int CHUNK_BYTES = 64 * BK * 2;                      // one 64 x 64 box of an MN-major operand
constexpr int SLICE = 64, WARP_STAGING_BYTES = 32 * SLICE * 2, STAGING_BYTES = EPI_WARPS * WARP_STAGING_BYTES;
constexpr size_t SMEM_LIMIT = 232448;
constexpr size_t SMEM_FIXED = 1024 /*alignment slack*/ + 512 /*barriers*/ + STAGING_BYTES;
constexpr unsigned long long kWaitBudgetNs = 4000000000ull;

enum { A_TILED = 0, A_IM2COL = 1, A_MN = 2 };
enum { B_K = 0, B_MN = 2, B_MN_IM2COL = 3 };
enum { EPI_STATS = 1, EPI_ADD = 2, EPI_SPLITK = 4 };

struct Shared {
  uint64_t full[MAX_STAGES], empty[MAX_STAGES], acc_full[2], acc_empty[2], b_full;
  uint32_t tmem_base;
  int error;
};
static_assert(sizeof(Shared) <= 512, "barrier block");

struct Problem {
  int M, N;                    // rows and columns of the product
  int tiles_m, tiles_n;
  int k_blocks_total;          // 64-wide K blocks of the whole product
  int k_per_slice, slices;     // split-K (wgrad); slices == 1 otherwise
  int mma_n;                   // N of the MMA and columns staged per tile (multiple of 16, of 64 for MN-major B)
  int a_mode, b_mode;
  int taps, S;                 // filter taps (R * S) and filter width
  int cblocks;                 // K blocks per tap (channels of the K dimension / 64)
  int Cb;                      // channels per tap in the weight / in the N index of wgrad
  int flip;                    // dgrad: tap t of the walk uses weight tap taps - 1 - t
  int Ho, Wo, stride, pad;     // pixel p -> (n, ho, wo); base coordinates of im2col loads: (wo * stride - pad, ho * stride - pad, n)
  int epi;
  int stages, stage_bytes;     // ring of the streamed operands (A, or A and B)
  int b_resident;              // all K blocks of B are loaded once and stay in shared memory
  int b_block_bytes;           // bytes of one K block of B (mma_n * 128)
  int stat_bytes;              // shared-memory bytes of the statistics accumulators ([warp][2][BN] floats) or 0
  float* stats;                // EPI_STATS: [gridDim.x][2][N] partial sums
  const __nv_bfloat16* add;    // EPI_ADD: [M, N] row-major tensor added to the product
  float* workspace;            // EPI_SPLITK: [tile][slice][BM][mma_n] fp32
  __nv_bfloat16* out;          // store epilogue: [M, N] row-major result
  int* status;
};

__device__ __forceinline__ void fail(Shared* sh, const Problem& p, int where) {
  atomicExch(&sh->error, where);
  if (p.status) atomicCAS(p.status, 0, 2000 + where);
}

__device__ __forceinline__ bool item(const Problem& p, int it, int* m_blk, int* n_blk, int* slice) {
  const int t = blockIdx.x + it * gridDim.x;
  const int tiles = p.tiles_m * p.tiles_n;
  if (t >= tiles * p.slices) return false;
  if (p.slices == 1) {
    *slice = 0; *m_blk = t / p.tiles_n; *n_blk = t - *m_blk * p.tiles_n;     // the n tiles of a row block run side by side
  } else {
    *slice = t / tiles;
    const int r = t - *slice * tiles;
    *n_blk = r / p.tiles_m; *m_blk = r - *n_blk * p.tiles_m;                  // the tiles of a K slice run side by side
  }
  return true;
}

__device__ __forceinline__ void pixel_coords(const Problem& p, int pix, int* w, int* h, int* n) {
  const int per = p.Ho * p.Wo;
  *n = pix / per;
  const int r = pix - *n * per;
  const int ho = r / p.Wo;
  *w = (r - ho * p.Wo) * p.stride - p.pad;
  *h = ho * p.stride - p.pad;
}

__device__ __forceinline__ int b_chunks(const Problem& p, int n0) { return (min(p.mma_n, p.N - n0) + 63) / 64; }

// the loads of one K block of B into b_dst
__device__ __forceinline__ void load_b(const Problem& p, const CUtensorMap* mb, unsigned char* b_dst, int kb, int n0, int chunks,
                                       uint64_t* bar) {
  int tap = 0, cb = kb;
  if (p.taps > 1 && p.a_mode != A_MN) { tap = kb / p.cblocks; cb = kb - tap * p.cblocks; }
  if (p.b_mode == B_K) {
    sm100::tma_load_2d(b_dst, mb, tap * p.Cb + cb * BK, n0, bar);
  } else if (p.b_mode == B_MN) {                // [K, N] with N contiguous: the weight in dgrad, the activation in a 1x1 wgrad
    const int wtap = p.flip ? p.taps - 1 - tap : tap;
    const int row = (p.a_mode == A_MN ? kb : cb) * BK;
    for (int j = 0; j < chunks; ++j) sm100::tma_load_2d(b_dst + j * CHUNK_BYTES, mb, wtap * p.Cb + n0 + 64 * j, row, bar);
  } else {                                      // wgrad of a filter with taps or a stride: im2col boxes of 64 pixels
    int bw, bh, bn;
    pixel_coords(p, kb * BK, &bw, &bh, &bn);
    for (int j = 0; j < chunks; ++j) {
      const int nj = n0 + 64 * j;
      const int tj = nj / p.Cb, r = tj / p.S;
      sm100::tma_load_im2col_4d(b_dst + j * CHUNK_BYTES, mb, nj - tj * p.Cb, bw, bh, bn, (unsigned short)(tj - r * p.S),
                                (unsigned short)r, bar);
    }
  }
}

__device__ void producer(Shared* sh, unsigned char* tiles, unsigned char* b_res, const Problem& p, const CUtensorMap* ma,
                         const CUtensorMap* mb) {
  if (p.b_resident) {                           // one column tile: every K block of B, once
    const int chunks = b_chunks(p, 0);
    const uint32_t per = p.b_mode == B_K ? (uint32_t)p.b_block_bytes : (uint32_t)chunks * CHUNK_BYTES;
    sm100::mbar_expect_tx(&sh->b_full, per * (uint32_t)p.k_blocks_total);
    for (int kb = 0; kb < p.k_blocks_total; ++kb) load_b(p, mb, b_res + (size_t)kb * p.b_block_bytes, kb, 0, chunks, &sh->b_full);
  }
  int stage = 0;
  uint32_t phase = 0;
  int m_blk, n_blk, slice;
  for (int it = 0; item(p, it, &m_blk, &n_blk, &slice); ++it) {
    const int m0 = m_blk * BM, n0 = n_blk * BN;
    int aw = 0, ah = 0, an = 0;
    if (p.a_mode == A_IM2COL) pixel_coords(p, m0, &aw, &ah, &an);
    const int chunks = b_chunks(p, n0);
    const uint32_t tx = A_BYTES + (p.b_resident ? 0u : p.b_mode == B_K ? (uint32_t)p.b_block_bytes : (uint32_t)chunks * CHUNK_BYTES);
    const int kb0 = slice * p.k_per_slice, kb1 = min(kb0 + p.k_per_slice, p.k_blocks_total);
    for (int kb = kb0; kb < kb1; ++kb) {
      if (!sm100::mbar_wait(&sh->empty[stage], phase ^ 1, kWaitBudgetNs) || sh->error) { fail(sh, p, 2); return; }
      unsigned char* a_dst = tiles + (size_t)stage * p.stage_bytes;
      uint64_t* bar = &sh->full[stage];
      sm100::mbar_expect_tx(bar, tx);
      if (p.a_mode == A_TILED) {
        sm100::tma_load_2d(a_dst, ma, kb * BK, m0, bar);
      } else if (p.a_mode == A_IM2COL) {
        const int tap = kb / p.cblocks, r = tap / p.S;
        sm100::tma_load_im2col_4d(a_dst, ma, (kb - tap * p.cblocks) * BK, aw, ah, an, (unsigned short)(tap - r * p.S),
                                  (unsigned short)r, bar);
      } else {                                  // [K, M] with M contiguous: two boxes of 64 columns x 64 k-rows
        sm100::tma_load_2d(a_dst, ma, m0, kb * BK, bar);
        sm100::tma_load_2d(a_dst + CHUNK_BYTES, ma, m0 + 64, kb * BK, bar);
      }
      if (!p.b_resident) load_b(p, mb, a_dst + A_BYTES, kb, n0, chunks, bar);
      if (++stage == p.stages) { stage = 0; phase ^= 1; }
    }
  }
}

__device__ void mma_issuer(Shared* sh, unsigned char* tiles, unsigned char* b_res, const Problem& p) {
  const bool a_mn = p.a_mode == A_MN, b_mn = p.b_mode != B_K;
  const uint32_t idesc = sm100::make_idesc_f16(BM, p.mma_n, true, b_mn, a_mn);
  if (p.b_resident) {
    if (!sm100::mbar_wait(&sh->b_full, 0, kWaitBudgetNs) || sh->error) { fail(sh, p, 7); return; }
    sm100::tc_fence_after();
  }
  const uint32_t b_res_addr = sm100::smem_u32(b_res);
  int stage = 0;
  uint32_t phase = 0;
  int m_blk, n_blk, slice;
  for (int it = 0; item(p, it, &m_blk, &n_blk, &slice); ++it) {
    const int acc = it & 1;
    const uint32_t acc_phase = (it >> 1) & 1;
    if (!sm100::mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1, kWaitBudgetNs) || sh->error) { fail(sh, p, 3); return; }
    sm100::tc_fence_after();
    const uint32_t d_tmem = sh->tmem_base + (uint32_t)acc * BN;
    const int kb0 = slice * p.k_per_slice, kb1 = min(kb0 + p.k_per_slice, p.k_blocks_total);
    for (int kb = kb0; kb < kb1; ++kb) {
      if (!sm100::mbar_wait(&sh->full[stage], phase, kWaitBudgetNs) || sh->error) { fail(sh, p, 4); return; }
      sm100::tc_fence_after();
      const uint32_t a_addr = sm100::smem_u32(tiles + (size_t)stage * p.stage_bytes);
      const uint32_t b_addr = p.b_resident ? b_res_addr + (uint32_t)kb * (uint32_t)p.b_block_bytes : a_addr + A_BYTES;
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) {
        const uint64_t da = a_mn ? sm100::make_desc_sw128_mn(a_addr + k * UMMA_K * 128, CHUNK_BYTES, 1024)
                                 : sm100::make_desc_sw128(a_addr + k * UMMA_K * 2);
        const uint64_t db = b_mn ? sm100::make_desc_sw128_mn(b_addr + k * UMMA_K * 128, CHUNK_BYTES, 1024)
                                 : sm100::make_desc_sw128(b_addr + k * UMMA_K * 2);
        sm100::umma_f16(d_tmem, da, db, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
      }
      sm100::umma_commit(&sh->empty[stage]);
      if (++stage == p.stages) { stage = 0; phase ^= 1; }
    }
    sm100::umma_commit(&sh->acc_full[acc]);
  }
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) { f[2 * e] = __uint_as_float(w[e] << 16); f[2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u); }
}

// bf16 rows (+ statistics, + added tensor).  Every warp works on its own: it reads its 32 accumulator
// rows 64 columns at a time, converts them into its staging tile (32 rows x 128 bytes, swizzled so that
// both the row-wise writes and the line-wise reads are conflict free), reads the tile back line by line
// - eight lanes per 128-byte row, four rows per instruction - and stores full lines.  The same read
// feeds the column sums.  Group g (four warps, one per lane quarter) drains accumulator g, so two tiles
// are in the epilogue at any time and no barrier between warps sits in the loop.
template <bool do_stats, bool do_add>
__device__ void epilogue_store(Shared* sh, unsigned char* stg, float* stats_all, const Problem& p, int ew, int quarter, int lane) {
  const int group = ew >> 2;                      // ew: index of this warp among the epilogue warps
  const int chunk = lane & 7, rsub = lane >> 3;
  // Running column sums of this lane (packed fp32 pairs) for the 8 columns of its chunk in each of the four
  // 64-column slices of a tile.  The CTA always visits the same n_blk (the grid is a multiple of tiles_n), so
  // the columns stay the same over all its tiles and the sums live in registers until the kernel ends.
  unsigned long long cs2[4][4], cq2[4][4];
#pragma unroll
  for (int sl = 0; sl < 4; ++sl)
#pragma unroll
    for (int e = 0; e < 4; ++e) { cs2[sl][e] = 0ull; cq2[sl][e] = 0ull; }
  int m_blk, n_blk, slice;
  for (int it = group; item(p, it, &m_blk, &n_blk, &slice); it += 2) {
    const uint32_t acc_phase = (it >> 1) & 1;
    if (!sm100::mbar_wait(&sh->acc_full[group], acc_phase, kWaitBudgetNs) || sh->error) { fail(sh, p, 5); break; }
    sm100::tc_fence_after();
    const int row0 = m_blk * BM + quarter * 32;
    const uint32_t t_base = sh->tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)group * BN;
#pragma unroll
    for (int sl = 0; sl < BN / SLICE; ++sl) {
      const int c0 = sl * SLICE;
      const int col0 = n_blk * BN + c0;
      if (c0 < p.mma_n && col0 < p.N) {
        // the second gradient, read line by line like the store (the eight loads fly while the accumulator is converted)
        uint4 av[8];
        if (do_add) {
          const __nv_bfloat16* addp = p.add + (size_t)row0 * p.N + col0 + chunk * 8;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int rw = i * 4 + rsub;
            av[i] = row0 + rw < p.M ? __ldg(reinterpret_cast<const uint4*>(addp + (size_t)rw * p.N)) : make_uint4(0, 0, 0, 0);
          }
        }
        uint32_t r[2][32];
        sm100::tmem_ld_32x32(t_base + c0, r[0]);
        sm100::tmem_ld_32x32(t_base + c0 + 32, r[1]);
        sm100::tmem_ld_wait();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[h][j]), __uint_as_float(r[h][j + 1]));
            __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[h][j + 2]), __uint_as_float(r[h][j + 3]));
            __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[h][j + 4]), __uint_as_float(r[h][j + 5]));
            __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[h][j + 6]), __uint_as_float(r[h][j + 7]));
            uint4 u;
            u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
            u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
            const int ck = h * 4 + j / 8;
            *reinterpret_cast<uint4*>(stg + (size_t)lane * 128 + ((ck ^ (lane & 7)) << 4)) = u;
          }
        }
        __syncwarp();
        __nv_bfloat16* out = p.out + (size_t)row0 * p.N + col0 + chunk * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rw = i * 4 + rsub;
          uint4 u = *reinterpret_cast<const uint4*>(stg + (size_t)rw * 128 + ((chunk ^ (rw & 7)) << 4));
          if (row0 + rw < p.M) {
            if (do_add) {                       // bf16(product) + it, as a separate accumulation kernel would compute
              __nv_bfloat162* uu = reinterpret_cast<__nv_bfloat162*>(&u);
              const __nv_bfloat162* aa = reinterpret_cast<const __nv_bfloat162*>(&av[i]);
#pragma unroll
              for (int e = 0; e < 4; ++e) uu[e] = __hadd2(uu[e], aa[e]);
            }
            *reinterpret_cast<uint4*>(out + (size_t)rw * p.N) = u;
          }
          if (do_stats) {                       // rows past M hold zeros
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              unsigned long long f2;
              asm("mov.b64 %0, {%1, %2};" : "=l"(f2) : "r"(w[e] << 16), "r"(w[e] & 0xffff0000u));
              asm("add.rn.f32x2 %0, %0, %1;" : "+l"(cs2[sl][e]) : "l"(f2));
              asm("fma.rn.f32x2 %0, %1, %1, %0;" : "+l"(cq2[sl][e]) : "l"(f2));
            }
          }
        }
        __syncwarp();                           // the staging tile is rewritten by the next slice
      }
    }
    sm100::tc_fence_before();
    __syncwarp();
    if (lane == 0) sm100::mbar_arrive(&sh->acc_empty[group]);
  }
  if (do_stats) {
    // once per kernel: add the four row groups of the warp (lanes l, l + 8, l + 16, l + 24 hold the same
    // columns), park the warp's sums in shared memory, then add the eight warps in a fixed order
    float* mine = stats_all + (size_t)ew * 2 * BN;
#pragma unroll
    for (int sl = 0; sl < 4; ++sl)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        uint32_t lo, hi;
        float v[4];
        asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(cs2[sl][e]));
        v[0] = __uint_as_float(lo); v[1] = __uint_as_float(hi);
        asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(cq2[sl][e]));
        v[2] = __uint_as_float(lo); v[3] = __uint_as_float(hi);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[k] += __shfl_xor_sync(0xffffffffu, v[k], 8);
          v[k] += __shfl_xor_sync(0xffffffffu, v[k], 16);
        }
        if (rsub == 0) {
          const int c = sl * SLICE + chunk * 8 + 2 * e;
          mine[c] = v[0]; mine[c + 1] = v[1]; mine[BN + c] = v[2]; mine[BN + c + 1] = v[3];
        }
      }
    // the CTA's partial row: the sums over its column window, zeros elsewhere
    asm volatile("bar.sync 3, 256;" ::: "memory");     // all eight epilogue warps have parked their sums
    const int tid = ew * 32 + lane;
    const int win0 = (blockIdx.x % p.tiles_n) * BN;
    float* dst = p.stats + (size_t)blockIdx.x * 2 * p.N;
    for (int c = tid; c < 2 * p.N; c += 256) {
      const int which = c >= p.N, col = c - which * p.N - win0;
      float v = 0.f;
      if (col >= 0 && col < BN) {
#pragma unroll
        for (int w = 0; w < EPI_WARPS; ++w) v += stats_all[(w * 2 + which) * BN + col];
      }
      dst[c] = v;
    }
  }
}

// fp32 partial tiles of a K slice: workspace[tile][slice][row][mma_n]
__device__ void epilogue_splitk(Shared* sh, const Problem& p, int group, int quarter, int lane) {
  const int r_in_tile = quarter * 32 + lane;
  int m_blk, n_blk, slice;
  for (int it = group; item(p, it, &m_blk, &n_blk, &slice); it += 2) {
    const uint32_t acc_phase = (it >> 1) & 1;
    if (!sm100::mbar_wait(&sh->acc_full[group], acc_phase, kWaitBudgetNs) || sh->error) { fail(sh, p, 6); break; }
    sm100::tc_fence_after();
    const int tile = n_blk * p.tiles_m + m_blk;
    const int ncols = min(p.mma_n, p.N - n_blk * BN);
    const uint32_t t_base = sh->tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)group * BN;
    float* mine = p.workspace + (((size_t)tile * p.slices + slice) * BM + r_in_tile) * p.mma_n;
#pragma unroll 1
    for (int c0 = 0; c0 < ncols; c0 += 32) {
      uint32_t r[32];
      sm100::tmem_ld_32x32(t_base + c0, r);
      sm100::tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<uint4*>(mine + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
    }
    sm100::tc_fence_before();
    __syncwarp();
    if (lane == 0) sm100::mbar_arrive(&sh->acc_empty[group]);
  }
}

// EPI: the epilogue flags as a template parameter, so that each flavour carries only its own registers
template <int EPI>
__global__ void __launch_bounds__(THREADS, 1)
conv_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Problem p) {
  extern __shared__ unsigned char smem_raw[];
  const uintptr_t base = ((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023;
  unsigned char* tiles = (unsigned char*)base;
  unsigned char* b_res = tiles + (size_t)p.stages * p.stage_bytes;
  unsigned char* staging = b_res + (p.b_resident ? (size_t)p.k_blocks_total * p.b_block_bytes : 0);
  float* stats = (float*)(staging + STAGING_BYTES);
  Shared* sh = (Shared*)((unsigned char*)stats + p.stat_bytes);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(&map_a);
    sm100::tma_prefetch_desc(&map_b);
    for (int s = 0; s < p.stages; ++s) { sm100::mbar_init(&sh->full[s], 1); sm100::mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { sm100::mbar_init(&sh->acc_full[a], 1); sm100::mbar_init(&sh->acc_empty[a], 4); }
    sm100::mbar_init(&sh->b_full, 1);
    sh->error = 0;
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc(&sh->tmem_base, TMEM_COLS);
    sm100::tmem_relinquish();
  }
  if (p.epi & EPI_STATS)
    for (int i = threadIdx.x; i < EPI_WARPS * 2 * BN; i += THREADS) stats[i] = 0.f;
  sm100::tc_fence_before();
  __syncthreads();
  sm100::tc_fence_after();

  if (warp == 0) {
    if (sm100::elect_one()) producer(sh, tiles, b_res, p, &map_a, &map_b);
  } else if (warp == 1) {
    if (sm100::elect_one()) mma_issuer(sh, tiles, b_res, p);
  } else if constexpr ((EPI & EPI_SPLITK) != 0) {
    epilogue_splitk(sh, p, (warp - 2) >> 2, warp & 3, lane);
  } else {
    epilogue_store<(EPI & EPI_STATS) != 0, (EPI & EPI_ADD) != 0>(sh, staging + (size_t)(warp - 2) * WARP_STAGING_BYTES, stats, p,
                                                              warp - 2, warp & 3, lane);
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

// out[row, n0 + c] (+)= sum over slices of the partial tiles.  L lanes (a power of two up to 32) share one group of
// 8 columns: lane j adds slices j, j + L, ... and the L partial sums are combined by a fixed butterfly, so the
// result does not depend on timing.
__global__ void __launch_bounds__(256)
conv_splitk_reduce_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ out, int M, int N, int tiles_m, int tiles_n,
                          int slices, int mma_n, int accumulate, int L) {
  const int groups = N / 8;                                    // N is a multiple of 8
  const long long total = (long long)M * groups;
  const int sub = threadIdx.x & (L - 1);
  const long long per_block = blockDim.x / L;
  for (long long i0 = (long long)blockIdx.x * per_block; i0 < total; i0 += (long long)gridDim.x * per_block) {
    const long long i = i0 + threadIdx.x / L;
    const bool live = i < total;
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.f;
    int row = 0, col = 0;
    if (live) {
      row = (int)(i / groups); col = (int)(i - (long long)row * groups) * 8;
      const int m_blk = row / BM, n_blk = col / BN;
      const int tile = n_blk * tiles_m + m_blk;
      const float* src = ws + (((size_t)tile * slices) * BM + (row - m_blk * BM)) * mma_n + (col - n_blk * BN);
      int s = sub;
      for (; s + 3 * L < slices; s += 4 * L) {                 // four slices of loads in flight
        float4 x[4][2];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float4* q = reinterpret_cast<const float4*>(src + (size_t)(s + u * L) * BM * mma_n);
          x[u][0] = __ldcs(q); x[u][1] = __ldcs(q + 1);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          a[0] += x[u][0].x; a[1] += x[u][0].y; a[2] += x[u][0].z; a[3] += x[u][0].w;
          a[4] += x[u][1].x; a[5] += x[u][1].y; a[6] += x[u][1].z; a[7] += x[u][1].w;
        }
      }
      for (; s < slices; s += L) {
        const float4* q = reinterpret_cast<const float4*>(src + (size_t)s * BM * mma_n);
        const float4 x0 = __ldcs(q), x1 = __ldcs(q + 1);
        a[0] += x0.x; a[1] += x0.y; a[2] += x0.z; a[3] += x0.w; a[4] += x1.x; a[5] += x1.y; a[6] += x1.z; a[7] += x1.w;
      }
    }
    for (int d = 1; d < L; d <<= 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) a[e] += __shfl_xor_sync(0xffffffffu, a[e], d);
    }
    if (live && sub == 0) {
      __nv_bfloat16* dst = out + (size_t)row * N + col;
      if (accumulate) {
        float f[8];
        unpack8(*reinterpret_cast<const uint4*>(dst), f);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] += f[e];
      }
      __nv_bfloat162 h0 = __floats2bfloat162_rn(a[0], a[1]), h1 = __floats2bfloat162_rn(a[2], a[3]);
      __nv_bfloat162 h2 = __floats2bfloat162_rn(a[4], a[5]), h3 = __floats2bfloat162_rn(a[6], a[7]);
      uint4 u;
      u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
      u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
      *reinterpret_cast<uint4*>(dst) = u;
    }
  }
}

}  // namespace conv

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeIm2colFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const int*, const int*, cuuint32_t, cuuint32_t, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeIm2colFn encode_im2col_fn() {
  static EncodeIm2colFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeIm2colFn)p;
  });
  return fn;
}

// im2col-mode map of a channels-last [N, H, W, C] bf16 tensor for an R x S filter with the given padding and
// stride: boxes of 64 channels x `pixels` filter positions, 128-byte swizzle.
static int make_im2col_map(CUtensorMap* map, const void* base, int N, int H, int W, int C, int R, int S, int stride, int pad,
                           int pixels) {
  EncodeIm2colFn fn = encode_im2col_fn();
  if (!fn) return fail(TMPI_ERR_UNSUPPORTED, "cuTensorMapEncodeIm2col is not available");
  if (((uintptr_t)base & 15) || C % 8) return fail(TMPI_ERR_INVALID, "conv: activation must be 16-byte aligned with C a multiple of 8");
  cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
  cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)W * C * 2, (cuuint64_t)H * W * C * 2};
  int lower[2] = {-pad, -pad};
  int upper[2] = {pad - (S - 1), pad - (R - 1)};
  cuuint32_t estr[4] = {1, (cuuint32_t)stride, (cuuint32_t)stride, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, lower, upper,
                  (cuuint32_t)conv::BK, (cuuint32_t)pixels, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TMPI_ERR_CUDA, "cuTensorMapEncodeIm2col failed (CUresult %d)", (int)r);
  return TMPI_OK;
}

static int* conv_status_word(int** host_out = nullptr) {
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

// Plans the shared memory (stages, resident weight) and launches.
static int conv_launch(const CUtensorMap& ma, const CUtensorMap& mb, conv::Problem& p, int* grid_out, cudaStream_t s) {
  void (*kernel)(const CUtensorMap, const CUtensorMap, const conv::Problem) = nullptr;
  switch (p.epi) {
    case 0: kernel = conv::conv_gemm_kernel<0>; break;
    case conv::EPI_STATS: kernel = conv::conv_gemm_kernel<conv::EPI_STATS>; break;
    case conv::EPI_ADD: kernel = conv::conv_gemm_kernel<conv::EPI_ADD>; break;
    case conv::EPI_SPLITK: kernel = conv::conv_gemm_kernel<conv::EPI_SPLITK>; break;
    default: return fail(TMPI_ERR_INVALID, "conv: unsupported epilogue combination %d", p.epi);
  }
  cudaError_t ae = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)conv::SMEM_LIMIT);
  if (ae != cudaSuccess) return fail(TMPI_ERR_CUDA, "conv: shared memory attribute: %s", cudaGetErrorString(ae));
  p.status = conv_status_word();
  p.b_block_bytes = p.mma_n * conv::BK * 2;
  p.stat_bytes = (p.epi & conv::EPI_STATS) ? conv::EPI_WARPS * 2 * conv::BN * (int)sizeof(float) : 0;
  const long budget = (long)conv::SMEM_LIMIT - (long)conv::SMEM_FIXED - p.stat_bytes;
  const long b_all = (long)p.k_blocks_total * p.b_block_bytes;
  p.b_resident = 0;
  if (p.tiles_n == 1 && p.slices == 1 && b_all < (1 << 20) && (budget - b_all) / conv::A_BYTES >= 5) {
    p.b_resident = 1;
    p.stage_bytes = conv::A_BYTES;
    p.stages = (int)std::min<long>(conv::MAX_STAGES, (budget - b_all) / conv::A_BYTES);
  } else {
    p.stage_bytes = conv::A_BYTES + p.b_block_bytes;
    p.stages = (int)std::min<long>(conv::MAX_STAGES, budget / p.stage_bytes);
  }
  if (p.stages < 2) return fail(TMPI_ERR_UNSUPPORTED, "conv: shared memory plan leaves %d stages", p.stages);
  const size_t smem = conv::SMEM_FIXED + p.stat_bytes + (size_t)p.stages * p.stage_bytes + (p.b_resident ? (size_t)b_all : 0);
  const int items = p.tiles_m * p.tiles_n * p.slices;
  int grid = std::min(items, gemm_sm_count());
  // statistics: a CTA keeps sums for one window of 256 columns, so every tile it visits must have the same n_blk
  if ((p.epi & conv::EPI_STATS) && grid % p.tiles_n) grid -= grid % p.tiles_n;
  if (grid_out) *grid_out = grid;
  kernel<<<grid, conv::THREADS, smem, s>>>(ma, mb, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "conv launch: %s", cudaGetErrorString(e));
}

static int launch_splitk_reduce(const conv::Problem& p, const void* workspace, void* out, int accumulate, cudaStream_t s) {
  int L = 1;
  while (L < 32 && L < p.slices) L <<= 1;                       // lanes per group of 8 columns
  const long long groups = (long long)p.M * (p.N / 8);
  const long long per_block = 256 / L;
  const int grid = (int)std::min<long long>((groups + per_block - 1) / per_block, (long long)gemm_sm_count() * 8);
  conv::conv_splitk_reduce_kernel<<<grid, 256, 0, s>>>((const float*)workspace, (__nv_bfloat16*)out, p.M, p.N, p.tiles_m, p.tiles_n,
                                                     p.slices, p.mma_n, accumulate, L);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "split-K reduce launch: %s", cudaGetErrorString(e));
}

struct Geom { int N, H, W, Cin, Cout, R, S, stride, pad, Ho, Wo; };

static int check_geom(const Geom& g, const char* what) {
  if (g.N < 1 || g.H < 1 || g.W < 1 || g.R < 1 || g.S < 1 || g.stride < 1 || g.pad < 0)
    return fail(TMPI_ERR_INVALID, "%s: bad geometry", what);
  if (g.Cin % 64 || g.Cout % 64) return fail(TMPI_ERR_UNSUPPORTED, "%s: channel counts must be multiples of 64 (got %d -> %d)", what, g.Cin, g.Cout);
  if (g.R != g.S) return fail(TMPI_ERR_UNSUPPORTED, "%s: square filters only", what);
  if (g.pad > g.R - 1 || g.R > 16) return fail(TMPI_ERR_UNSUPPORTED, "%s: padding beyond the filter or filter too large", what);
  if ((int64_t)g.N * g.Ho * g.Wo >= (int64_t)1 << 31 || (int64_t)g.N * g.H * g.W >= (int64_t)1 << 31)
    return fail(TMPI_ERR_UNSUPPORTED, "%s: more than 2^31 pixels", what);
  return TMPI_OK;
}

static Geom geom(int N, int H, int W, int Cin, int Cout, int R, int S, int stride, int pad) {
  Geom g{N, H, W, Cin, Cout, R, S, stride, pad, 0, 0};
  g.Ho = (H + 2 * pad - R) / stride + 1;
  g.Wo = (W + 2 * pad - S) / stride + 1;
  return g;
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

// Largest number of CTAs a convolution launches: rows of the statistics buffer.
int tmpi_conv_max_ctas(void) { return gemm_sm_count(); }

// y[N, Ho, Wo, Cout] = conv(x[N, H, W, Cin], w[Cout, R, S, Cin]); all bf16, channels-last, dense.
// stats (nullable): [tmpi_conv_max_ctas()][2][Cout] floats; rows 0 .. *stat_rows - 1 receive per-CTA partial
// sums and sums of squares of y per channel (the layout tmpi_bn_relu_fwd_partials reads).
int tmpi_conv_fwd(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int R, int S, int stride,
                  int pad, float* stats, int* stat_rows, void* stream) {
  const Geom g = geom(N, H, W, Cin, Cout, R, S, stride, pad);
  int st = check_geom(g, "conv forward");
  if (st) return st;
  const int64_t M = (int64_t)N * g.Ho * g.Wo;
  const bool plain = R == 1 && S == 1 && stride == 1 && pad == 0;
  CUtensorMap ma, mb;
  if (plain) st = make_tmap_bf16(&ma, x, (uint64_t)M, (uint64_t)Cin, (uint64_t)Cin, conv::BM);
  else st = make_im2col_map(&ma, x, N, H, W, Cin, R, S, stride, pad, conv::BM);
  if (st) return st;
  conv::Problem p{};
  p.M = (int)M; p.N = Cout;
  p.mma_n = std::min(conv::BN, (Cout + 15) / 16 * 16);
  if ((st = make_tmap_bf16(&mb, w, (uint64_t)Cout, (uint64_t)R * S * Cin, (uint64_t)R * S * Cin, (uint32_t)p.mma_n))) return st;
  if ((uintptr_t)y & 15) return fail(TMPI_ERR_INVALID, "conv: output must be 16-byte aligned");
  p.out = (__nv_bfloat16*)y;
  p.tiles_m = (int)((M + conv::BM - 1) / conv::BM);
  p.tiles_n = (Cout + conv::BN - 1) / conv::BN;
  p.taps = R * S; p.S = S; p.cblocks = Cin / conv::BK; p.Cb = Cin;
  p.k_blocks_total = p.taps * p.cblocks; p.k_per_slice = p.k_blocks_total; p.slices = 1;
  p.a_mode = plain ? conv::A_TILED : conv::A_IM2COL; p.b_mode = conv::B_K;
  p.Ho = g.Ho; p.Wo = g.Wo; p.stride = stride; p.pad = pad;
  p.epi = stats ? conv::EPI_STATS : 0;
  p.stats = stats;
  return conv_launch(ma, mb, p, stat_rows, (cudaStream_t)stream);
}

// dx[N, H, W, Cin] = gradient of the stride-1 convolution above with respect to x, given dy[N, Ho, Wo, Cout];
// add (nullable): a tensor shaped like dx that is added to the result (a second gradient into the same activation).
int tmpi_conv_dgrad(const void* dy, const void* w, void* dx, const void* add, int N, int H, int W, int Cin, int Cout, int R,
                    int S, int stride, int pad, void* stream) {
  const Geom g = geom(N, H, W, Cin, Cout, R, S, stride, pad);
  int st = check_geom(g, "conv dgrad");
  if (st) return st;
  if (stride != 1) return fail(TMPI_ERR_UNSUPPORTED, "conv dgrad: stride 1 only");
  const int64_t M = (int64_t)N * H * W;
  const bool plain = R == 1 && S == 1 && pad == 0;
  const int bpad = R - 1 - pad;                      // padding of the transposed convolution over dy
  CUtensorMap ma, mb;
  if (plain) st = make_tmap_bf16(&ma, dy, (uint64_t)M, (uint64_t)Cout, (uint64_t)Cout, conv::BM);
  else st = make_im2col_map(&ma, dy, N, g.Ho, g.Wo, Cout, R, S, 1, bpad, conv::BM);
  if (st) return st;
  conv::Problem p{};
  p.M = (int)M; p.N = Cin;
  p.mma_n = std::min(conv::BN, Cin);
  if ((st = make_tmap_bf16(&mb, w, (uint64_t)Cout, (uint64_t)R * S * Cin, (uint64_t)R * S * Cin, 64))) return st;
  if (((uintptr_t)dx | (uintptr_t)add) & 15) return fail(TMPI_ERR_INVALID, "conv: gradients must be 16-byte aligned");
  p.out = (__nv_bfloat16*)dx;
  p.tiles_m = (int)((M + conv::BM - 1) / conv::BM);
  p.tiles_n = (Cin + conv::BN - 1) / conv::BN;
  p.taps = R * S; p.S = S; p.cblocks = Cout / conv::BK; p.Cb = Cin; p.flip = 1;
  p.k_blocks_total = p.taps * p.cblocks; p.k_per_slice = p.k_blocks_total; p.slices = 1;
  p.a_mode = plain ? conv::A_TILED : conv::A_IM2COL; p.b_mode = conv::B_MN;
  p.Ho = H; p.Wo = W; p.stride = 1; p.pad = bpad;    // the walk is over the pixels of dx
  p.epi = add ? conv::EPI_ADD : 0;
  p.add = (const __nv_bfloat16*)add;
  return conv_launch(ma, mb, p, nullptr, (cudaStream_t)stream);
}

// Split of the K dimension (the pixels, for a weight gradient) of a [Mrows, Ncols] product over P rows of K.
static void splitk_plan(int Mrows, int Ncols, int64_t P, int* tiles_m, int* tiles_n, int* mma_n, int* kb_total, int* per, int* slices);
static void wgrad_split(const Geom& g, int* tiles_m, int* tiles_n, int* mma_n, int* kb_total, int* per, int* slices) {
  splitk_plan(g.Cout, g.R * g.S * g.Cin, (int64_t)g.N * g.Ho * g.Wo, tiles_m, tiles_n, mma_n, kb_total, per, slices);
}
static void splitk_plan(int Mrows, int Ncols, int64_t P, int* tiles_m, int* tiles_n, int* mma_n, int* kb_total, int* per, int* slices) {
  *tiles_m = (Mrows + conv::BM - 1) / conv::BM;
  *mma_n = std::min(conv::BN, (Ncols + 63) / 64 * 64);
  *tiles_n = (Ncols + conv::BN - 1) / conv::BN;
  *kb_total = (int)((P + conv::BK - 1) / conv::BK);
  const int tiles = *tiles_m * *tiles_n;
  int want = std::max(1, gemm_sm_count() / tiles);                       // one wave of work items
  want = std::min(want, std::max(1, *kb_total / 4));                     // at least four K blocks per slice
  *per = (*kb_total + want - 1) / want;
  *slices = (*kb_total + *per - 1) / *per;
}

// Bytes of workspace (fp32 partial tiles) tmpi_conv_wgrad needs for this geometry.
size_t tmpi_conv_wgrad_workspace_bytes(int N, int H, int W, int Cin, int Cout, int R, int S, int stride, int pad) {
  const Geom g = geom(N, H, W, Cin, Cout, R, S, stride, pad);
  int tm, tn, mn, kbt, per, sl;
  wgrad_split(g, &tm, &tn, &mn, &kbt, &per, &sl);
  return (size_t)tm * tn * sl * conv::BM * mn * sizeof(float);
}

// dw[Cout, R, S, Cin] (+)= gradient with respect to the weight: a split-K product into the workspace, then the sum
// over the slices (a second kernel).  `accumulate` adds to dw instead of overwriting it.  Launches that share a
// workspace must not overlap.
int tmpi_conv_wgrad(const void* dy, const void* x, void* dw, int N, int H, int W, int Cin, int Cout, int R, int S,
                    int stride, int pad, void* workspace, size_t workspace_bytes, int accumulate, void* stream) {
  const Geom g = geom(N, H, W, Cin, Cout, R, S, stride, pad);
  int st = check_geom(g, "conv wgrad");
  if (st) return st;
  const int64_t P = (int64_t)N * g.Ho * g.Wo;
  const bool plain = R == 1 && S == 1 && stride == 1 && pad == 0;
  conv::Problem p{};
  wgrad_split(g, &p.tiles_m, &p.tiles_n, &p.mma_n, &p.k_blocks_total, &p.k_per_slice, &p.slices);
  const size_t need = (size_t)p.tiles_m * p.tiles_n * p.slices * conv::BM * p.mma_n * sizeof(float);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15))
    return fail(TMPI_ERR_INVALID, "conv wgrad: workspace of %zu bytes (16-byte aligned) needed, got %zu", need, workspace_bytes);
  if ((uintptr_t)dw & 15) return fail(TMPI_ERR_INVALID, "conv wgrad: dw must be 16-byte aligned");
  CUtensorMap ma, mb;
  if ((st = make_tmap_bf16(&ma, dy, (uint64_t)P, (uint64_t)Cout, (uint64_t)Cout, 64))) return st;
  if (plain) st = make_tmap_bf16(&mb, x, (uint64_t)P, (uint64_t)Cin, (uint64_t)Cin, 64);
  else st = make_im2col_map(&mb, x, N, H, W, Cin, R, S, stride, pad, 64);
  if (st) return st;
  p.M = Cout; p.N = R * S * Cin;
  p.taps = R * S; p.S = S; p.cblocks = 1; p.Cb = Cin;
  p.a_mode = conv::A_MN; p.b_mode = plain ? conv::B_MN : conv::B_MN_IM2COL;
  p.Ho = g.Ho; p.Wo = g.Wo; p.stride = stride; p.pad = pad;
  p.epi = conv::EPI_SPLITK;
  p.workspace = (float*)workspace;
  if ((st = conv_launch(ma, mb, p, nullptr, (cudaStream_t)stream))) return st;
  return launch_splitk_reduce(p, workspace, dw, accumulate, (cudaStream_t)stream);
}

// C[M, N] (+)= A^T B for row-major A [K, M] and B [K, N] (both read as they lie) with a long K and a small
// output: K is split over the SMs, fp32 partial tiles go to the workspace and a second kernel adds them in
// slice order.  M, N multiples of 8; lda / ldb / ldc: row pitches in elements (0: dense).
size_t tmpi_gemm_tn_splitk_workspace_bytes(int M, int N, int64_t K) {
  int tm, tn, mn, kbt, per, sl;
  splitk_plan(M, N, K, &tm, &tn, &mn, &kbt, &per, &sl);
  return (size_t)tm * tn * sl * conv::BM * mn * sizeof(float);
}

int tmpi_gemm_bf16_tn_splitk(const void* A, const void* B, void* C, int M, int N, int64_t K, int64_t lda, int64_t ldb,
                             void* workspace, size_t workspace_bytes, int accumulate, void* stream) {
  if (M < 1 || N < 1 || K < 1 || M % 8 || N % 8) return fail(TMPI_ERR_INVALID, "gemm_tn_splitk: M and N must be positive multiples of 8");
  if (!lda) lda = M;
  if (!ldb) ldb = N;
  conv::Problem p{};
  splitk_plan(M, N, K, &p.tiles_m, &p.tiles_n, &p.mma_n, &p.k_blocks_total, &p.k_per_slice, &p.slices);
  const size_t need = (size_t)p.tiles_m * p.tiles_n * p.slices * conv::BM * p.mma_n * sizeof(float);
  if (!workspace || workspace_bytes < need || ((uintptr_t)workspace & 15) || ((uintptr_t)C & 15))
    return fail(TMPI_ERR_INVALID, "gemm_tn_splitk: workspace of %zu bytes needed (got %zu); buffers 16-byte aligned", need, workspace_bytes);
  CUtensorMap ma, mb;
  int st;
  if ((st = make_tmap_bf16(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 64))) return st;
  if ((st = make_tmap_bf16(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 64))) return st;
  p.M = M; p.N = N;
  p.taps = 1; p.S = 1; p.cblocks = 1; p.Cb = N;
  p.a_mode = conv::A_MN; p.b_mode = conv::B_MN;
  p.Ho = p.Wo = 1; p.stride = 1;
  p.epi = conv::EPI_SPLITK;
  p.workspace = (float*)workspace;
  if ((st = conv_launch(ma, mb, p, nullptr, (cudaStream_t)stream))) return st;
  return launch_splitk_reduce(p, workspace, C, accumulate, (cudaStream_t)stream);
}

// Non-zero after a convolution CTA gave up on a bounded wait (2000 + the point where it happened); clears it.
int tmpi_conv_status(void) {
  int* host = nullptr;
  conv_status_word(&host);
  if (!host) return 0;
  int v = *(volatile int*)host;
  if (v) *(volatile int*)host = 0;
  return v;
}

}  // extern "C"
