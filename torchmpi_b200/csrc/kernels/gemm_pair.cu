// bf16 GEMM on CTA pairs: C[M,N] = act(A[M,K] * B[N,K]^T + bias) with 256 x 256 tiles computed by
// two CTAs of a cluster (gemm_pair.cuh).  One cluster per TPC, persistent; tiles are visited in
// bands of 8 tile-rows so that the clusters running at one time share B panels in L2.
#include "gemm_pair.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include <algorithm>
#include <cstring>
#include <mutex>

namespace tmpi {

int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
int gemm_sm_count();

namespace gemm2 {

constexpr int BAND = 8;   // 256-row tiles per band

__device__ __forceinline__ void band_order(int t, int tiles_m, int tiles_n, int* m_tile, int* n_blk) {
  const int per_band = BAND * tiles_n;
  const int band = t / per_band;
  const int rows = min(BAND, tiles_m - band * BAND);
  const int r = t - band * per_band;
  *m_tile = band * BAND + r % rows;
  *n_blk = r / rows;
}

// p.tiles_m counts 256-row tiles here.
__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                      const __grid_constant__ CUtensorMap map_c, const Problem p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *tiles, *staging;
  Shared* sh;
  carve(smem_raw, &tiles, &sh, &staging);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = sm100::cluster_ctarank();
  setup(sh, warp, &map_a, &map_b);

  const int total = p.tiles_m * p.tiles_n;
  const int cluster = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  auto order = [&](int it, int* m_blk, int* n_blk) -> bool {
    const int t = cluster + it * nclusters;
    if (t >= total) return false;
    int m_tile;
    band_order(t, p.tiles_m, p.tiles_n, &m_tile, n_blk);
    *m_blk = m_tile * 2 + (int)rank;
    return true;
  };
  if (warp == 0) {
    if (sm100::elect_one()) producer(sh, tiles, p, &map_a, &map_b, rank, order, [](int, const CUtensorMap**, int*) { return true; });
  } else if (warp == 1) {
    if (rank == 0 && sm100::elect_one()) mma_issuer(sh, tiles, p, order);
  } else {
    epilogue(sh, staging, p, warp & 3, lane, order, [&](int m_blk, const CUtensorMap** m, int* row0) {
      *row0 = m_blk * BM;
      *m = *row0 < p.M ? &map_c : nullptr;
    });
  }
  __syncwarp();
  teardown(sh, warp);
}

// Largest number of co-resident clusters of two CTAs (falls back to one per two SMs).
static int max_clusters() {
  static int n = 0;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaFuncSetAttribute(gemm_bf16_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.gridDim = dim3(2 * (gemm_sm_count() / 2)); cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = SMEM_BYTES; cfg.attrs = at; cfg.numAttrs = 1;
    int c = 0;
    if (cudaOccupancyMaxActiveClusters(&c, (void*)gemm_bf16_pair_kernel, &cfg) == cudaSuccess && c > 0) n = c;
    else { cudaGetLastError(); n = gemm_sm_count() / 2; }
  });
  return n;
}

}  // namespace gemm2

// Shapes the pair kernel takes: TMA-storable C and at least one full pair tile each way.
bool gemm_pair_applicable(const void* C, int M, int N, int K, int flags) {
  const bool a_km = (flags & gemm::A_IS_KM) != 0, b_kn = (flags & gemm::B_IS_KN) != 0;
  if (M < 2 * gemm2::BM || N < gemm2::BN || N % 8 || ((uintptr_t)C & 15)) return false;
  if ((a_km ? M : K) % 8) return false;          // 16-byte rows of A as stored
  if (!b_kn && K % 8) return false;              // 16-byte rows of B as stored ([K, N] rows are covered by N % 8)
  return true;
}

// lda / ldb / ldc: row pitch of A, B, C as stored, in elements (0: dense).  With explicit pitches the
// extents themselves need not be multiples of 8 (a [T, 50257] matrix held in rows of 50264).
int launch_gemm_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int epilogue,
                     int* status_word, cudaStream_t stream, int64_t lda, int64_t ldb, int64_t ldc) {
  CUtensorMap ma, mb, mc;
  int st;
  const bool a_km = (epilogue & gemm::A_IS_KM) != 0;       // A given as [K, M], M contiguous
  if (!lda) lda = a_km ? M : K;
  if (a_km) st = make_tmap_bf16(&ma, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, gemm2::BK);
  else st = make_tmap_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, gemm2::BM);
  if (st) return st;
  const bool b_kn = (epilogue & gemm::B_IS_KN) != 0;       // B given as [K, N], N contiguous
  if (!ldb) ldb = b_kn ? N : K;
  if (b_kn) st = make_tmap_bf16(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, gemm2::BK);
  else st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)ldb, gemm2::BN / 2);
  if (st) return st;
  if (!ldc) ldc = N;
  if ((st = make_tmap_bf16(&mc, C, (uint64_t)M, (uint64_t)N, (uint64_t)ldc, gemm2::BM))) return st;
  gemm::Problem p{};
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + 2 * gemm2::BM - 1) / (2 * gemm2::BM);
  p.tiles_n = (N + gemm2::BN - 1) / gemm2::BN;
  p.k_blocks = (K + gemm2::BK - 1) / gemm2::BK;
  p.epilogue = epilogue & 3;
  p.b_mn = b_kn ? 1 : 0;
  p.a_mn = a_km ? 1 : 0;
  p.bias = (const __nv_bfloat16*)bias;
  p.tma_store = 1;
  p.status = status_word;
  const int nclusters = std::min(p.tiles_m * p.tiles_n, gemm2::max_clusters());
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * nclusters); cfg.blockDim = dim3(gemm2::THREADS);
  cfg.dynamicSmemBytes = gemm2::SMEM_BYTES; cfg.stream = stream; cfg.attrs = at; cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm2::gemm_bf16_pair_kernel, ma, mb, mc, p);
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "pair gemm launch: %s", cudaGetErrorString(e));
}

}  // namespace tmpi
