// The bf16 tcgen05 GEMM on CTA pairs (cta_group::2): two CTAs of a cluster, on the two SMs of a
// TPC, compute one 256 x 256 output tile.
//
// Each CTA stages 128 rows of A and 128 rows of B (its half of the 256 columns of the tile) per
// 64-wide K block, so a stage is 32 KB and six stages fit beside the epilogue staging.  One thread
// of the even CTA issues tcgen05.mma.cta_group::2 with M = 256, N = 256: both tensor cores read
// their own A half and both B halves, which halves the shared-memory traffic per FLOP against a
// 128 x 256 tile on one CTA.  Each CTA keeps the 128 accumulator rows of its A half in its own
// tensor memory (two 256-column accumulators) and runs its own epilogue.
//
// Synchronisation (all waits bounded, as in gemm_core.cuh):
//   full[s]   lives in the even CTA; both producers' TMA loads count their bytes there
//   empty[s]  one per CTA; the issuer commits to both after the MMAs of the stage
//   acc_full  one per CTA; the issuer commits to both after the last K block of a tile
//   acc_empty lives in the even CTA; the eight epilogue warps of the pair arrive there
// The roles take the same hooks as the single-CTA ones; m_blk counts 128-row blocks, so the hooks of
// the fused kernels (rows-ready wait, destination map) apply per CTA.
#pragma once
#include "gemm_core.cuh"

namespace tmpi {
namespace gemm2 {

using gemm::Problem;
constexpr int BM = 128;               // rows per CTA; the pair covers 2 * BM
constexpr int BN = 256;               // columns of the pair's tile; each CTA stages BN / 2 rows of B
constexpr int BK = 64, STAGES = 6, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = (BN / 2) * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + gemm::EPI_STAGING_BYTES + 1024 + 256;
constexpr unsigned long long kWaitBudgetNs = gemm::kWaitBudgetNs;
static_assert(BN == gemm::BN && BM == gemm::BM, "the epilogue is shared with the single-CTA kernel");
static_assert(SMEM_BYTES <= 232448, "shared memory of one CTA");

struct Shared {
  uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int error;
};

__device__ __forceinline__ void carve(unsigned char* raw, unsigned char** tiles, Shared** sh, unsigned char** staging) {
  uintptr_t base = ((uintptr_t)raw + 1023) & ~(uintptr_t)1023;
  *tiles = (unsigned char*)base;
  *staging = (unsigned char*)(base + (size_t)STAGES * STAGE_BYTES);
  *sh = (Shared*)(base + (size_t)STAGES * STAGE_BYTES + gemm::EPI_STAGING_BYTES);
}

// All threads of both CTAs.  The dynamic shared memory has the same layout in both CTAs, so an
// offset taken in one is valid in the other.
__device__ __forceinline__ void setup(Shared* sh, int warp, const CUtensorMap* ma, const CUtensorMap* mb) {
  if (warp == 0 && sm100::elect_one()) {
    sm100::tma_prefetch_desc(ma);
    sm100::tma_prefetch_desc(mb);
    for (int s = 0; s < STAGES; ++s) { sm100::mbar_init(&sh->full[s], 1); sm100::mbar_init(&sh->empty[s], 1); }
    for (int a = 0; a < 2; ++a) { sm100::mbar_init(&sh->acc_full[a], 1); sm100::mbar_init(&sh->acc_empty[a], 8); }
    sh->error = 0;
    sm100::fence_barrier_init();
  }
  if (warp == 1) {
    sm100::tmem_alloc_pair(&sh->tmem_base, TMEM_COLS);
    sm100::tmem_relinquish_pair();
  }
  sm100::tc_fence_before();
  __syncthreads();
  sm100::cluster_sync();          // the other CTA's barriers exist before anything signals them
  sm100::tc_fence_after();
}

// One thread in EACH CTA.  order(it, &m_blk, &n_blk): m_blk is this CTA's 128-row block.
template <typename TileOrder, typename ASource>
__device__ __forceinline__ void producer(Shared* sh, unsigned char* tiles, const Problem& p, const CUtensorMap* ma,
                                         const CUtensorMap* mb, uint32_t rank, TileOrder order, ASource a_source) {
  int stage = 0;
  uint32_t phase = 0;
  int m_blk, n_blk;
  for (int it = 0; order(it, &m_blk, &n_blk); ++it) {
    const CUtensorMap* a_map = ma;
    int a_row0 = m_blk * BM;
    if (!a_source(m_blk, &a_map, &a_row0)) { gemm::fail(sh, p, 11); return; }
    const int b_row0 = n_blk * BN + (int)rank * (BN / 2);
    for (int kb = 0; kb < p.k_blocks; ++kb) {
      if (!sm100::mbar_wait(&sh->empty[stage], phase ^ 1, kWaitBudgetNs) || sh->error) { gemm::fail(sh, p, 12); return; }
      unsigned char* a_dst = tiles + (size_t)stage * STAGE_BYTES;
      const uint32_t full0 = sm100::map_to_cta(&sh->full[stage], 0);
      if (rank == 0) sm100::mbar_expect_tx(&sh->full[stage], 2 * STAGE_BYTES);   // both CTAs' bytes
      if (!p.a_mn) {
        sm100::tma_load_2d_pair(a_dst, a_map, kb * BK, a_row0, full0);
      } else {   // A is [K, M]: two boxes of 64 rows of the product x 64 k-rows
        sm100::tma_load_2d_pair(a_dst, a_map, a_row0, kb * BK, full0);
        sm100::tma_load_2d_pair(a_dst + A_BYTES / 2, a_map, a_row0 + 64, kb * BK, full0);
      }
      if (!p.b_mn) {
        sm100::tma_load_2d_pair(a_dst + A_BYTES, mb, kb * BK, b_row0, full0);
      } else {   // B is [K, N]: two boxes of 64 columns x 64 k-rows, each a column of eight swizzle atoms
        sm100::tma_load_2d_pair(a_dst + A_BYTES, mb, b_row0, kb * BK, full0);
        sm100::tma_load_2d_pair(a_dst + A_BYTES + B_BYTES / 2, mb, b_row0 + 64, kb * BK, full0);
      }
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
  }
}

// One thread of the EVEN CTA only.
template <typename TileOrder>
__device__ __forceinline__ void mma_issuer(Shared* sh, unsigned char* tiles, const Problem& p, TileOrder order) {
  const uint32_t idesc = sm100::make_idesc_f16(2 * BM, BN, true, p.b_mn != 0, p.a_mn != 0);
  int stage = 0;
  uint32_t phase = 0;
  int m_blk, n_blk;
  for (int it = 0; order(it, &m_blk, &n_blk); ++it) {
    const int acc = it & 1;
    const uint32_t acc_phase = (it >> 1) & 1;
    if (!sm100::mbar_wait(&sh->acc_empty[acc], acc_phase ^ 1, kWaitBudgetNs) || sh->error) { gemm::fail(sh, p, 13); return; }
    sm100::tc_fence_after();
    const uint32_t d_tmem = sh->tmem_base + (uint32_t)acc * BN;
    for (int kb = 0; kb < p.k_blocks; ++kb) {
      if (!sm100::mbar_wait(&sh->full[stage], phase, kWaitBudgetNs) || sh->error) { gemm::fail(sh, p, 14); return; }
      sm100::tc_fence_after();
      const uint32_t a_addr = sm100::smem_u32(tiles + (size_t)stage * STAGE_BYTES);
      const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
      for (int k = 0; k < BK / UMMA_K; ++k) {
        const uint64_t da = p.a_mn ? sm100::make_desc_sw128_mn(a_addr + k * UMMA_K * 128, A_BYTES / 2, 1024)
                                   : sm100::make_desc_sw128(a_addr + k * UMMA_K * 2);
        const uint64_t db = p.b_mn ? sm100::make_desc_sw128_mn(b_addr + k * UMMA_K * 128, B_BYTES / 2, 1024)
                                   : sm100::make_desc_sw128(b_addr + k * UMMA_K * 2);
        sm100::umma_f16_pair(d_tmem, da, db, idesc, (kb | k) != 0);
      }
      sm100::umma_commit_pair(sm100::map_to_cta(&sh->empty[stage], 0));   // both producers may refill the stage
      sm100::umma_commit_pair(sm100::map_to_cta(&sh->empty[stage], 1));
      if (++stage == STAGES) { stage = 0; phase ^= 1; }
    }
    sm100::umma_commit_pair(sm100::map_to_cta(&sh->acc_full[acc], 0));    // both epilogues may read
    sm100::umma_commit_pair(sm100::map_to_cta(&sh->acc_full[acc], 1));
  }
}

// The four epilogue warps of EACH CTA (see gemm::epilogue_tma_impl for DestMap; leaving the map
// null skips the stores of a row block).
template <typename TileOrder, typename DestMap>
__device__ __forceinline__ void epilogue(Shared* sh, unsigned char* staging, const Problem& p, int quarter, int lane,
                                         TileOrder order, DestMap dest) {
  gemm::epilogue_tma_impl(sh, staging, p, quarter, lane, order, dest, [sh](int acc) {
    sm100::mbar_arrive_cluster(sm100::map_to_cta(&sh->acc_empty[acc], 0));
  });
}

// All threads of both CTAs.  Neither CTA frees its tensor memory or exits while the other may still
// signal its barriers or have the pair's MMAs read its shared memory.
__device__ __forceinline__ void teardown(Shared* sh, int warp) {
  sm100::tc_fence_before();
  __syncthreads();
  if (sh->error && warp == 0 && sm100::elect_one()) {
    const unsigned long long t0 = sm100::now_ns();
    while (sm100::now_ns() - t0 < 200000000ull) { __nanosleep(1000); }   // copies in flight complete within microseconds
  }
  __syncthreads();
  sm100::cluster_sync();
  if (warp == 1) {
    sm100::tc_fence_after();
    sm100::tmem_dealloc_pair(sh->tmem_base, TMEM_COLS);
  }
}

}  // namespace gemm2
}  // namespace tmpi
