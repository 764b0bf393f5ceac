// Building blocks of the bf16 tcgen05 GEMM: C[M,N] = act(A[M,K] * B[N,K]^T + bias).
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer - one elected thread streams 128x64 A tiles and 256x64 B tiles
//               (128-byte swizzle) into a 4-stage shared-memory ring, completion on mbarriers;
//   warp 1      MMA issuer - owns the tensor memory (512 columns = two 128x256 fp32 accumulators);
//               one thread issues four tcgen05.mma (K = 16 each) per stage and commits the stage
//               back to the producer, then commits the accumulator to the epilogue;
//   warps 2-5   epilogue - tcgen05.ld the accumulator (lane quarter = warp % 4), add bias, apply
//               GELU, convert to bf16 and store, while the issuer already fills the other accumulator.
// Every mbarrier wait is bounded; on expiry the CTA records an error, stops issuing work, drains
// what is in flight within a second budget, frees its tensor memory and returns.
//
// The roles take three hooks so that the fused kernels (all-gather -> GEMM, GEMM -> reduce-scatter)
// reuse them: a tile order, a "rows of A are ready" wait in the producer, and the row -> destination
// mapping of the epilogue.
#pragma once
#include <cuda_bf16.h>
#include "sm100_ptx.cuh"

namespace tmpi {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int EPI_STAGING_BYTES = 2 * BM * 64 * 2;           // two 128 x 64 bf16 staging tiles for TMA stores
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + EPI_STAGING_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr unsigned long long kWaitBudgetNs = 4000000000ull;   // 4 s: far beyond any legitimate wait

enum { EPI_NONE = 0, EPI_BIAS = 1, EPI_GELU = 2, EPI_BIAS_GELU = 3,
       B_IS_KN = 4, A_IS_KM = 8 /* operand layout flags in the same word */ };

struct Shared {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int error;
};

struct Problem {
  int M, N, K;
  int tiles_m, tiles_n, k_blocks;
  int epilogue;
  const __nv_bfloat16* bias;   // [N] or nullptr
  int tma_store;               // epilogue writes through TMA (needs 16-byte aligned rows of C)
  int b_mn;                    // B is given as [K, N] with N contiguous (CTA-pair kernels only)
  int a_mn;                    // A is given as [K, M] with M contiguous (plain CTA-pair GEMM only)
  int mma_n;                   // single-CTA kernel, narrow outputs: rows of B staged per tile and N of the MMA
                               // (a multiple of 16 below BN); 0 = BN
  int* status;                 // global error word (nullptr: none)
};

__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.f + erff(x * 0.70710678118654752f)); }

__device__ __forceinline__ void setup(Shared* sh, unsigned char* tiles, int warp, const CUtensorMap* ma, const CUtensorMap* mb) {
  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(ma);
    sm100::tma_prefetch_desc(mb);
    for (int s = 0; s < STAGES; ++s) { sm100::mbar_init(&sh->full[s], 1); sm100::mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { sm100::mbar_init(&sh->acc_full[a], 1); sm100::mbar_init(&sh->acc_empty[a], 4); }
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
}

template <typename Sh>
__device__ __forceinline__ void fail(Sh* sh, const Problem& p, int where) {
  atomicExch(&sh->error, where);
  if (p.status) atomicCAS(p.status, 0, 1000 + where);
}

// ---- producer: TileOrder(tile_iter, &m_blk, &n_blk) -> bool;
// ASource(m_blk, &map, &row0) -> bool picks the tensor map and first row of the A tile (and may wait,
// bounded, until those rows are ready)
template <typename TileOrder, typename ASource>
__device__ __forceinline__ void producer(Shared* sh, unsigned char* tiles, const Problem& p, const CUtensorMap* ma,
                                         const CUtensorMap* mb, TileOrder order, ASource a_source) {
  int stage = 0;
  uint32_t phase = 0;
  int m_blk, n_blk;
  for (int it = 0; order(it, &m_blk, &n_blk); ++it) {
    const CUtensorMap* a_map = ma;
    int a_row0 = m_blk * BM;
    if (!a_source(m_blk, &a_map, &a_row0)) { fail(sh, p, 1); return; }
    for (int kb = 0; kb < p.k_blocks; ++kb) {
      if (!sm100::mbar_wait(&sh->empty[stage], phase ^ 1, kWaitBudgetNs) || sh->error) { fail(sh, p, 2); return; }
      unsigned char* a_dst = tiles + (size_t)stage * STAGE_BYTES;
      sm100::mbar_expect_tx(&sh->full[stage], A_BYTES + (p.mma_n ? p.mma_n : BN) * BK * 2);
      sm100::tma_load_2d(a_dst, a_map, kb * BK, a_row0, &sh->full[stage]);
      sm100::tma_load_2d(a_dst + A_BYTES, mb, kb * BK, n_blk * BN, &sh->full[stage]);
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  }
}

template <typename TileOrder>
__device__ __forceinline__ void mma_issuer(Shared* sh, unsigned char* tiles, const Problem& p, TileOrder order) {
  const uint32_t idesc = sm100::make_idesc_f16(BM, p.mma_n ? p.mma_n : BN, true);
  int stage = 0;
  uint32_t phase = 0;
  int m_blk, n_blk;
  for (int it = 0; order(it, &m_blk, &n_blk); ++it) {
    const int acc = it & 1;
    const uint32_t acc_phase = (it >> 1) & 1;
    if (!sm100::mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1, kWaitBudgetNs) || sh->error) { fail(sh, p, 3); return; }
    sm100::tc_fence_after();
    const uint32_t d_tmem = sh->tmem_base + (uint32_t)acc * BN;
    for (int kb = 0; kb < p.k_blocks; ++kb) {
      if (!sm100::mbar_wait(&sh->full[stage], phase, kWaitBudgetNs) || sh->error) { fail(sh, p, 4); return; }
      sm100::tc_fence_after();
      const uint32_t a_addr = sm100::smem_u32(tiles + (size_t)stage * STAGE_BYTES);
      const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) {
        const uint64_t da = sm100::make_desc_sw128(a_addr + k * UMMA_K * 2);
        const uint64_t db = sm100::make_desc_sw128(b_addr + k * UMMA_K * 2);
        sm100::umma_f16(d_tmem, da, db, idesc, (kb | k) != 0);
      }
      sm100::umma_commit(&sh->empty[stage]);          // stage reusable once these MMAs have read it
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    sm100::umma_commit(&sh->acc_full[acc]);           // accumulator complete
  }
}

// ---- epilogue: Dest(m_blk, row_in_tile, &ptr_to_row_start_of_C_in_columns_space) gives, for a global
// row, the address of element (row, 0) of the destination matrix with leading dimension N; nullptr
// skips the row.  quarter = warp % 4 selects the 32 accumulator lanes this warp may read.
template <typename TileOrder, typename Dest>
__device__ __forceinline__ void epilogue(Shared* sh, const Problem& p, int quarter, int lane, TileOrder order, Dest dest) {
  int m_blk, n_blk;
  for (int it = 0; order(it, &m_blk, &n_blk); ++it) {
    const int acc = it & 1;
    const uint32_t acc_phase = (it >> 1) & 1;
    if (!sm100::mbar_wait(&sh->acc_full[acc], acc_phase, kWaitBudgetNs) || sh->error) { fail(sh, p, 5); return; }
    sm100::tc_fence_after();
    const int row = m_blk * BM + quarter * 32 + lane;
    __nv_bfloat16* crow = row < p.M ? dest(m_blk, row) : nullptr;
    const uint32_t t_base = sh->tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * BN;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
      uint32_t r[32];
      sm100::tmem_ld_32x32(t_base + c0, r);
      sm100::tmem_ld_wait();
      const int col0 = n_blk * BN + c0;
      if (crow && col0 < p.N) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (p.epilogue & EPI_BIAS) {
#pragma unroll
          for (int j = 0; j < 32; ++j) if (col0 + j < p.N) v[j] += __bfloat162float(p.bias[col0 + j]);
        }
        if (p.epilogue & EPI_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
        }
        __nv_bfloat16* dst = crow + col0;
        if (col0 + 32 <= p.N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
            __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
            uint4 u;
            u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
            u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(dst + j) = u;
          }
        } else {
          for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = __float2bfloat16_rn(v[j]);
        }
      }
    }
    sm100::tc_fence_before();
    __syncwarp();
    if (lane == 0) sm100::mbar_arrive(&sh->acc_empty[acc]);   // four warps arrive: accumulator drained
  }
}

// ---- epilogue with TMA stores.  The four epilogue warps convert 64-column slices of the accumulator
// to bf16 into a 128-byte-swizzled staging tile (two of them, 16 KB each) and one thread hands each
// slice to the TMA engine, which writes full 128-byte rows - to local memory or straight into a
// peer's memory - while the warps already convert the next slice.  Direct stores from the
// accumulator layout would issue 32 separate 16-byte writes per warp instruction.
// DestMap(m_blk, &map, &row0) picks the destination tensor map (box 64 columns x 128 rows) and the
// first row inside it.  Rows and columns beyond the tensor are clipped by the TMA unit.
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(sm100::smem_u32(smem_src)), "r"(c0), "r"(c1) : "memory");
}

// Release(acc) is called by one lane of each of the four warps once the accumulator is drained.
template <typename Sh, typename TileOrder, typename DestMap, typename Release>
__device__ __forceinline__ void epilogue_tma_impl(Sh* sh, unsigned char* staging, const Problem& p, int quarter, int lane,
                                                  TileOrder order, DestMap dest, Release release) {
  constexpr int SLICE = 64, SLICE_BYTES = BM * SLICE * 2;
  const int r_in_tile = quarter * 32 + lane;
  const bool leader = quarter == 2 && lane == 0;      // warp 2 of the CTA holds quarter 2
  int m_blk, n_blk;
  int slice_no = 0;
  for (int it = 0; order(it, &m_blk, &n_blk); ++it) {
    const int acc = it & 1;
    const uint32_t acc_phase = (it >> 1) & 1;
    // the 128 epilogue threads meet at named barriers below, so they must agree on going on:
    // vote (every thread gets here, its wait being bounded) and leave together on a failure
    const uint32_t ok = sm100::mbar_wait(&sh->acc_full[acc], acc_phase, kWaitBudgetNs) && !sh->error;
    uint32_t all_ok;
    asm volatile("{\n .reg .pred p, q;\n setp.ne.b32 p, %1, 0;\n barrier.cta.red.and.pred q, 1, 128, p;\n selp.u32 %0, 1, 0, q;\n}\n"
                 : "=r"(all_ok) : "r"(ok) : "memory");
    if (!all_ok) { fail(sh, p, 5); break; }
    sm100::tc_fence_after();
    const CUtensorMap* cmap = nullptr;
    int row0 = 0;
    dest(m_blk, &cmap, &row0);
    const uint32_t t_base = sh->tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)acc * BN;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += SLICE, ++slice_no) {
      const int col0 = n_blk * BN + c0;
      if (col0 >= p.N) break;            // uniform over the 128 threads: the rest of the tile lies outside C
      unsigned char* stg = staging + (size_t)(slice_no & 1) * SLICE_BYTES;
      uint32_t r[2][32];
      sm100::tmem_ld_32x32(t_base + c0, r[0]);
      sm100::tmem_ld_32x32(t_base + c0 + 32, r[1]);
      sm100::tmem_ld_wait();
      // the store that used this staging buffer two slices ago must have read it
      if (leader) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      epi_bar_sync();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[h][j]);
        if (p.epilogue & EPI_BIAS) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int c = col0 + h * 32 + j;
            if (c < p.N) v[j] += __bfloat162float(p.bias[c]);
          }
        }
        if (p.epilogue & EPI_GELU) {
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = gelu_erf(v[j]);
        }
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
          __nv_bfloat162 h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
          uint4 u;
          u.x = *reinterpret_cast<uint32_t*>(&h0); u.y = *reinterpret_cast<uint32_t*>(&h1);
          u.z = *reinterpret_cast<uint32_t*>(&h2); u.w = *reinterpret_cast<uint32_t*>(&h3);
          const int chunk = h * 4 + j / 8;                               // 16-byte chunk inside the 128-byte row
          *reinterpret_cast<uint4*>(stg + (size_t)r_in_tile * 128 + ((chunk ^ (r_in_tile & 7)) << 4)) = u;
        }
      }
      sm100::fence_proxy_async();        // generic-proxy writes to shared memory -> visible to the TMA unit
      epi_bar_sync();
      if (leader && cmap) {
        tma_store_2d(cmap, stg, col0, row0);
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    sm100::tc_fence_before();
    __syncwarp();
    if (lane == 0) release(acc);                                // four warps arrive: accumulator drained
  }
  if (leader) {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");   // all stores complete before exit
    sm100::fence_proxy_async();
  }
}

template <typename TileOrder, typename DestMap>
__device__ __forceinline__ void epilogue_tma(Shared* sh, unsigned char* staging, const Problem& p, int quarter, int lane,
                                             TileOrder order, DestMap dest) {
  epilogue_tma_impl(sh, staging, p, quarter, lane, order, dest, [sh](int acc) { sm100::mbar_arrive(&sh->acc_empty[acc]); });
}

// Frees the tensor memory after every role is done (all threads call).  When an error was raised
// the CTA first waits, bounded, for its outstanding TMA copies (the full barriers) so that no copy
// lands in shared memory after exit.
__device__ __forceinline__ void teardown(Shared* sh, int warp) {
  sm100::tc_fence_before();
  __syncthreads();
  if (sh->error && warp == 0 && sm100::elect_one()) {
    const unsigned long long t0 = sm100::now_ns();
    while (sm100::now_ns() - t0 < 200000000ull) { __nanosleep(1000); }   // copies in flight complete within microseconds
  }
  __syncthreads();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc(sh->tmem_base, TMEM_COLS);
  }
}

// Carves the dynamic shared memory: 1024-byte aligned tile ring, the epilogue staging tiles, the barrier block.
__device__ __forceinline__ void carve(unsigned char* raw, unsigned char** tiles, Shared** sh, unsigned char** staging = nullptr) {
  uintptr_t base = ((uintptr_t)raw + 1023) & ~(uintptr_t)1023;
  *tiles = (unsigned char*)base;
  if (staging) *staging = (unsigned char*)(base + (size_t)STAGES * STAGE_BYTES);
  *sh = (Shared*)(base + (size_t)STAGES * STAGE_BYTES + EPI_STAGING_BYTES);
}

}  // namespace gemm
}  // namespace tmpi
