// Tensor-parallel GEMMs fused with their collectives over NVLink peer memory.
//
//   ag_gemm  (all-gather -> GEMM):   C[M, N] = act(gather_rows(A_shard)[M, K] * B[N, K]^T + bias)
//   gemm_rs  (GEMM -> reduce-scatter): out[M/R, N] = sum over ranks of (A[M, K] * B[N, K]^T)[my rows]
//
// Both are ONE persistent kernel per rank in which a few CTAs move data between GPUs while the rest
// run the tcgen05 pipeline of gemm_core.cuh, tile by tile:
//
// ag_gemm: the first `n_comm` CTAs are copy engines.  One thread per CTA streams each peer's shard
//   (contiguous rows) through shared memory with bulk asynchronous copies - peer memory -> shared
//   memory -> the local full-A buffer, six 32 KB copies in flight per CTA - and publishes a flag per
//   128-row tile.  The GEMM CTAs visit M-tiles in the order the shards arrive (own shard first) and
//   their TMA producer waits for the tile's flag, so the math on shard j overlaps the transfer of
//   shard j+1 and every remote byte crosses NVLink exactly once.  No load uses cluster multicast, and
//   no TMA load of the GEMM touches peer memory: it reads the local copy.
// gemm_rs: the epilogue stores each output tile straight into a per-source slot in the memory of the
//   rank that owns those rows (remote tiles first, own tiles last); after a grid-wide and a
//   cross-rank barrier every CTA sums the slots of its rows locally in rank order (deterministic).
//
// These replace what the reference's model-parallel example does with two library calls and a full
// allreduce (examples/mnist/mnist_modelparallel.lua:30-60).  All waits are bounded.
#include "gemm_fused.cuh"
#include "gemm_pair.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include "../runtime/cuda_state.h"
#include <cstring>
#include <mutex>

namespace tmpi {

int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
int gemm_sm_count();

namespace gemm {

__global__ void __launch_bounds__(THREADS, 1)
ag_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_own,
               const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
               __nv_bfloat16* __restrict__ C, const Problem p, const __grid_constant__ FusedArgs g) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  unsigned char *tiles, *staging;
  Shared* sh;
  carve(smem_raw, &tiles, &sh, &staging);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_abort = 0;
  if ((int)blockIdx.x < g.n_comm) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < STAGES; ++s) { sm100::mbar_init(&sh->full[s], 1); sm100::mbar_init(&sh->empty[s], 1); }
      sh->error = 0;
      sm100::fence_barrier_init();
    }
    __syncthreads();
    ag_comm(g, p, tiles, sh, &s_abort);
    return;
  }
  setup(sh, tiles, warp, &map_a, &map_b);
  const int workers = gridDim.x - g.n_comm, wid = blockIdx.x - g.n_comm;
  const int total = p.tiles_m * p.tiles_n;
  const int tiles_per_rank = g.rows_per_rank / BM;
  const int rot = g.P.me * tiles_per_rank;
  // bands of one shard each, visited in arrival order; inside a band walk down the rows first
  auto order = [&](int it, int* m_blk, int* n_blk) -> bool {
    const int t = wid + it * workers;
    if (t >= total) return false;
    const int per_band = tiles_per_rank * p.tiles_n;
    const int band = t / per_band, r = t - band * per_band;
    *m_blk = (rot + band * tiles_per_rank + r % tiles_per_rank) % p.tiles_m;
    *n_blk = r / tiles_per_rank;
    return true;
  };
  if (warp == 0) {
    if (sm100::elect_one()) {
      producer(sh, tiles, p, &map_a, &map_b, order, [&](int m_blk, const CUtensorMap** amap, int* row0) {
        if (m_blk >= rot && m_blk < rot + tiles_per_rank) {      // my own rows: read the shard where it lies
          *amap = &map_own;
          *row0 = (m_blk - rot) * BM;
          return true;
        }
        const unsigned long long t0 = sm100::now_ns();
        while (ld_acquire_gpu(&g.ready[m_blk]) != g.ready_value) {
          __nanosleep(200);
          if (sm100::now_ns() - t0 > kWaitBudgetNs) return false;
        }
        sm100::fence_proxy_async();
        return true;
      });
    }
  } else if (warp == 1) {
    if (sm100::elect_one()) mma_issuer(sh, tiles, p, order);
  } else {
    epilogue_tma(sh, staging, p, warp & 3, lane, order,
                 [&](int m_blk, const CUtensorMap** m, int* row0) { *m = &map_c; *row0 = m_blk * BM; });
  }
  teardown(sh, warp);
}

// ------------------------------------------------------------------ GEMM -> reduce-scatter
struct SlotMaps { CUtensorMap m[8]; };   // destination slot (mine) inside every owner's memory

__global__ void __launch_bounds__(THREADS, 1)
gemm_rs_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ SlotMaps slot_maps, const Problem p, const __grid_constant__ FusedArgs g) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  unsigned char *tiles, *staging;
  Shared* sh;
  carve(smem_raw, &tiles, &sh, &staging);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_abort = 0;
  setup(sh, tiles, warp, &map_a, &map_b);
  const Peers& P = g.P;
  const int R = P.n;
  const int total = p.tiles_m * p.tiles_n;
  const int tiles_per_rank = g.rows_per_rank / BM;
  const int rot = ((P.me + 1) % R) * tiles_per_rank;      // the next rank's rows first, my own rows last
  auto order = [&](int it, int* m_blk, int* n_blk) -> bool {
    const int t = blockIdx.x + it * gridDim.x;
    if (t >= total) return false;
    const int per_band = tiles_per_rank * p.tiles_n;
    const int band = t / per_band, r = t - band * per_band;
    *m_blk = (rot + band * tiles_per_rank + r % tiles_per_rank) % p.tiles_m;
    *n_blk = r / tiles_per_rank;
    return true;
  };
  const size_t slot_elems = (size_t)g.rows_per_rank * p.N;
  if (warp == 0) {
    if (sm100::elect_one()) producer(sh, tiles, p, &map_a, &map_b, order, [](int, const CUtensorMap**, int*) { return true; });
  } else if (warp == 1) {
    if (sm100::elect_one()) mma_issuer(sh, tiles, p, order);
  } else {
    // the tile goes straight into my slot inside the owner's memory (TMA store over NVLink for peers)
    epilogue_tma(sh, staging, p, warp & 3, lane, order, [&](int m_blk, const CUtensorMap** m, int* row0) {
      const int owner = m_blk / tiles_per_rank;
      *m = &slot_maps.m[owner];
      *row0 = (m_blk - owner * tiles_per_rank) * BM;
    });
  }
  // all tiles of this CTA are stored; make them visible system-wide, then meet the rest of the grid
  __threadfence_system();
  sm100::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(g.grid_counter, 1u);
    const unsigned long long t0 = sm100::now_ns();
    while ((int)(*(volatile unsigned int*)g.grid_counter - g.grid_target) < 0) {
      __nanosleep(200);
      if (sm100::now_ns() - t0 > kWaitBudgetNs) { fail(sh, p, 20); s_abort = 1; break; }
    }
    __threadfence();
  }
  __syncthreads();
  if (peer_barrier(P, 1, 210, &s_abort) && !sh->error) {
    // every rank's partial rows for me are in my slots: sum them in rank order
    const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(P.base[P.me] + g.sym_off);
    gemm::slot_sum(slots, slot_elems, R, g.local, (size_t)blockIdx.x * THREADS + threadIdx.x, (size_t)gridDim.x * THREADS);
    peer_barrier(P, 2, 211, &s_abort);      // slots may be overwritten by the next call only after everyone has summed
  }
  teardown(sh, warp);
}

}  // namespace gemm

// ------------------------------------------------------------------ the same two kernels on CTA pairs
// 256 x 256 tiles computed by two CTAs (gemm_pair.cuh).  The grid is made of clusters of two; the
// copy engines of ag_gemm occupy whole clusters (n_comm is even) and never use the cluster barrier.
// Row blocks stay 128 rows, so the flags of the all-gather and the slot maps of the reduce-scatter
// are the same as in the single-CTA kernels; rows per rank must be a multiple of 256.
namespace gemm2 {

using gemm::FusedArgs;
using gemm::SlotMaps;

__global__ void __launch_bounds__(THREADS, 1)
ag_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_own,
                    const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                    const Problem p, const __grid_constant__ FusedArgs g) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  unsigned char *tiles, *staging;
  Shared* sh;
  carve(smem_raw, &tiles, &sh, &staging);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_abort = 0;
  if ((int)blockIdx.x < g.n_comm) {
    if (threadIdx.x == 0) {
      for (int s = 0; s < STAGES; ++s) { sm100::mbar_init(&sh->full[s], 1); sm100::mbar_init(&sh->empty[s], 1); }
      sh->error = 0;
      sm100::fence_barrier_init();
    }
    __syncthreads();
    gemm::ag_comm(g, p, tiles, sh, &s_abort);
    return;
  }
  const uint32_t rank = sm100::cluster_ctarank();
  setup(sh, warp, &map_a, &map_b);
  const int workers = ((int)gridDim.x - g.n_comm) >> 1, wid = ((int)blockIdx.x - g.n_comm) >> 1;
  const int total = p.tiles_m * p.tiles_n;                   // p.tiles_m counts 256-row tiles
  const int tiles_per_rank = g.rows_per_rank / (2 * BM);     // 256-row tiles of one shard
  const int blocks_per_rank = g.rows_per_rank / BM;          // 128-row blocks of one shard
  const int rot = g.P.me * tiles_per_rank, rot_blk = g.P.me * blocks_per_rank;
  // bands of one shard each, visited in arrival order; inside a band walk down the rows first
  auto order = [&](int it, int* m_blk, int* n_blk) -> bool {
    const int t = wid + it * workers;
    if (t >= total) return false;
    const int per_band = tiles_per_rank * p.tiles_n;
    const int band = t / per_band, r = t - band * per_band;
    const int m_tile = (rot + band * tiles_per_rank + r % tiles_per_rank) % p.tiles_m;
    *m_blk = m_tile * 2 + (int)rank;
    *n_blk = r / tiles_per_rank;
    return true;
  };
  if (warp == 0) {
    if (sm100::elect_one()) {
      producer(sh, tiles, p, &map_a, &map_b, rank, order, [&](int m_blk, const CUtensorMap** amap, int* row0) {
        if (m_blk >= rot_blk && m_blk < rot_blk + blocks_per_rank) {   // my own rows: read the shard where it lies
          *amap = &map_own;
          *row0 = (m_blk - rot_blk) * BM;
          return true;
        }
        const unsigned long long t0 = sm100::now_ns();
        while (gemm::ld_acquire_gpu(&g.ready[m_blk]) != g.ready_value) {
          __nanosleep(200);
          if (sm100::now_ns() - t0 > kWaitBudgetNs) return false;
        }
        sm100::fence_proxy_async();
        return true;
      });
    }
  } else if (warp == 1) {
    if (rank == 0 && sm100::elect_one()) mma_issuer(sh, tiles, p, order);
  } else {
    epilogue(sh, staging, p, warp & 3, lane, order,
             [&](int m_blk, const CUtensorMap** m, int* row0) { *m = &map_c; *row0 = m_blk * BM; });
  }
  __syncwarp();
  teardown(sh, warp);
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_rs_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    const __grid_constant__ SlotMaps slot_maps, const Problem p, const __grid_constant__ FusedArgs g) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ int s_abort;
  unsigned char *tiles, *staging;
  Shared* sh;
  carve(smem_raw, &tiles, &sh, &staging);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) s_abort = 0;
  const uint32_t rank = sm100::cluster_ctarank();
  setup(sh, warp, &map_a, &map_b);
  const Peers& P = g.P;
  const int R = P.n;
  const int total = p.tiles_m * p.tiles_n;
  const int tiles_per_rank = g.rows_per_rank / (2 * BM), blocks_per_rank = g.rows_per_rank / BM;
  const int rot = ((P.me + 1) % R) * tiles_per_rank;      // the next rank's rows first, my own rows last
  const int cluster = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  auto order = [&](int it, int* m_blk, int* n_blk) -> bool {
    const int t = cluster + it * nclusters;
    if (t >= total) return false;
    const int per_band = tiles_per_rank * p.tiles_n;
    const int band = t / per_band, r = t - band * per_band;
    const int m_tile = (rot + band * tiles_per_rank + r % tiles_per_rank) % p.tiles_m;
    *m_blk = m_tile * 2 + (int)rank;
    *n_blk = r / tiles_per_rank;
    return true;
  };
  const size_t slot_elems = (size_t)g.rows_per_rank * p.N;
  if (warp == 0) {
    if (sm100::elect_one()) producer(sh, tiles, p, &map_a, &map_b, rank, order, [](int, const CUtensorMap**, int*) { return true; });
  } else if (warp == 1) {
    if (rank == 0 && sm100::elect_one()) mma_issuer(sh, tiles, p, order);
  } else {
    // the row block goes straight into my slot inside the owner's memory (TMA store over NVLink for peers)
    epilogue(sh, staging, p, warp & 3, lane, order, [&](int m_blk, const CUtensorMap** m, int* row0) {
      const int owner = m_blk / blocks_per_rank;
      *m = &slot_maps.m[owner];
      *row0 = (m_blk - owner * blocks_per_rank) * BM;
    });
  }
  // all tiles of this CTA are stored; make them visible system-wide, then meet the rest of the grid
  __threadfence_system();
  sm100::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(g.grid_counter, 1u);
    const unsigned long long t0 = sm100::now_ns();
    while ((int)(*(volatile unsigned int*)g.grid_counter - g.grid_target) < 0) {
      __nanosleep(200);
      if (sm100::now_ns() - t0 > kWaitBudgetNs) { gemm::fail(sh, p, 20); s_abort = 1; break; }
    }
    __threadfence();
  }
  __syncthreads();
  if (peer_barrier(P, 1, 210, &s_abort) && !sh->error) {
    // every rank's partial rows for me are in my slots: sum them in rank order
    const __nv_bfloat16* slots = reinterpret_cast<const __nv_bfloat16*>(P.base[P.me] + g.sym_off);
    gemm::slot_sum(slots, slot_elems, R, g.local, (size_t)blockIdx.x * THREADS + threadIdx.x, (size_t)gridDim.x * THREADS);
    peer_barrier(P, 2, 211, &s_abort);      // slots may be overwritten by the next call only after everyone has summed
  }
  __syncwarp();
  teardown(sh, warp);
}

}  // namespace gemm2
}  // namespace tmpi

// ------------------------------------------------------------------ host entry points
namespace tmpi {
namespace {

struct FusedWorkspace {
  uint32_t* ready = nullptr;          // kMaxTilesM flags
  unsigned int* grid_counter = nullptr;
  uint32_t ready_value = 0;
  unsigned int grid_total = 0;
  int* status = nullptr;              // host-mapped error word
};
constexpr int kMaxTilesM = 8192;
FusedWorkspace g_ws;
std::mutex g_ws_mu;

int workspace(FusedWorkspace** out) {
  if (!g_ws.ready) {
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, (kMaxTilesM + 64) * sizeof(uint32_t));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc(fused GEMM workspace)");
    e = cudaMemset(p, 0, (kMaxTilesM + 64) * sizeof(uint32_t));
    if (e != cudaSuccess) return cuda_fail(e, "cudaMemset(fused GEMM workspace)");
    g_ws.ready = (uint32_t*)p;
    g_ws.grid_counter = (unsigned int*)p + kMaxTilesM;
    int* host = nullptr;
    if (cudaHostAlloc((void**)&host, sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
      *host = 0;
      cudaHostGetDevicePointer((void**)&g_ws.status, host, 0);
    }
  }
  *out = &g_ws;
  return TMPI_OK;
}

int check_fused_shapes(int M, int N, int K, int R) {
  if (M < 1 || N < 1 || K < 1 || M % R) return fail(TMPI_ERR_INVALID, "fused gemm: M=%d must split evenly over %d ranks", M, R);
  if ((M / R) % gemm::BM) return fail(TMPI_ERR_INVALID, "fused gemm: rows per rank (%d) must be a multiple of %d", M / R, gemm::BM);
  if (K % 128) return fail(TMPI_ERR_INVALID, "fused gemm: K=%d must be a multiple of 128", K);
  if (N % 8) return fail(TMPI_ERR_INVALID, "fused gemm: N=%d must be a multiple of 8", N);
  if (M / gemm::BM > kMaxTilesM) return fail(TMPI_ERR_INVALID, "fused gemm: too many row tiles");
  return TMPI_OK;
}

// Co-resident clusters of two CTAs of a pair kernel (its shared-memory attribute is set here too).
template <typename Kernel>
int pair_clusters(Kernel kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm2::SMEM_BYTES);
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(2 * (gemm_sm_count() / 2)); cfg.blockDim = dim3(gemm2::THREADS);
  cfg.dynamicSmemBytes = gemm2::SMEM_BYTES; cfg.attrs = at; cfg.numAttrs = 1;
  int c = 0;
  if (cudaOccupancyMaxActiveClusters(&c, (void*)kernel, &cfg) == cudaSuccess && c > 0) return c;
  cudaGetLastError();
  return gemm_sm_count() / 2;
}

template <typename Kernel, typename... Args>
cudaError_t launch_pairs(Kernel kernel, int ctas, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
  cfg.gridDim = dim3(ctas); cfg.blockDim = dim3(gemm2::THREADS);
  cfg.dynamicSmemBytes = gemm2::SMEM_BYTES; cfg.stream = stream; cfg.attrs = at; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

bool use_pairs(int M, int R) { return tunable("gemm_pair") != 0 && (M / R) % (2 * gemm2::BM) == 0; }

}  // namespace
}  // namespace tmpi

using namespace tmpi;

extern "C" {

// C[M, N] = act(A_full[M, K] * B[N, K]^T + bias) where A_full is the row-wise concatenation of every
// member's shard.  a_shard_off: heap offset of the [M/R, K] shard (same on every rank);
// a_full_off: heap offset of this rank's [M, K] gather buffer (filled by the kernel, reusable by backward).
int tmpi_cuda_ag_gemm(size_t a_shard_off, size_t a_full_off, const void* B, void* C, const void* bias, int M, int N,
                      int K, int epilogue, int n_comm, const tmpi_group_t* grp, void* stream) {
  CudaHeap& h = heap();
  if (!h.live || h.emulated) return fail(TMPI_ERR_STATE, "ag_gemm needs a real CUDA heap");
  const int R = grp->nmembers;
  int st = check_fused_shapes(M, N, K, R);
  if (st) return st;
  std::lock_guard<std::mutex> lk(g_ws_mu);
  FusedWorkspace* ws;
  if ((st = workspace(&ws))) return st;
  gemm::Problem p{};
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / gemm::BM; p.tiles_n = (N + gemm::BN - 1) / gemm::BN; p.k_blocks = K / gemm::BK;
  p.epilogue = epilogue & 3; p.bias = (const __nv_bfloat16*)bias; p.status = ws->status;
  const bool b_kn = (epilogue & gemm::B_IS_KN) != 0;
  if (b_kn && !use_pairs(M, R)) return fail(TMPI_ERR_UNSUPPORTED, "ag_gemm: B as [K, N] needs the CTA-pair kernel (rows per rank %% 256 == 0)");
  gemm::FusedArgs fa{};
  {
    std::lock_guard<std::mutex> hk(h.mu);
    if ((st = fill_peers(&fa.P, grp->members, R, grp->me, grp->lane))) return st;
  }
  char* a_full = h.base[h.rank] + a_full_off;
  CUtensorMap ma, mb;
  if ((st = make_tmap_bf16(&ma, a_full, (uint64_t)M, (uint64_t)K, (uint64_t)K, gemm::BM))) return st;
  if (!b_kn && (st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, gemm::BN))) return st;
  CUtensorMap mc;
  if ((st = make_tmap_bf16(&mc, C, (uint64_t)M, (uint64_t)N, (uint64_t)N, gemm::BM))) return st;
  CUtensorMap mown;
  if ((st = make_tmap_bf16(&mown, h.base[h.rank] + a_shard_off, (uint64_t)(M / R), (uint64_t)K, (uint64_t)K, gemm::BM))) return st;
  if (use_pairs(M, R)) {
    static int clusters = 0;
    if (!clusters) clusters = pair_clusters(gemm2::ag_gemm_pair_kernel);
    p.tiles_m = M / (2 * gemm2::BM);
    p.b_mn = b_kn ? 1 : 0;
    if (b_kn) st = make_tmap_bf16(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)N, gemm2::BK);
    else st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, gemm2::BN / 2);
    if (st) return st;
    const int tiles = p.tiles_m * p.tiles_n;
    int comm = n_comm > 0 ? (n_comm + 1) / 2 : 0;             // in clusters
    if (comm <= 0) {
      // as many copy clusters as the tile count leaves idle anyway (not below 4, i.e. 8 copy CTAs)
      const int waves = (tiles + clusters - 4 - 1) / (clusters - 4);
      comm = 4;
      while (comm + 1 <= clusters / 4 && (tiles + clusters - comm - 2) / (clusters - comm - 1) == waves) ++comm;
    }
    comm = std::min(comm, clusters / 4);
    fa.sym_off = a_shard_off; fa.local = (__nv_bfloat16*)a_full; fa.ready = ws->ready;
    fa.ready_value = ++ws->ready_value; fa.rows_per_rank = M / R; fa.n_comm = 2 * comm;
    cudaError_t e = launch_pairs(gemm2::ag_gemm_pair_kernel, 2 * clusters, (cudaStream_t)stream, ma, mown, mb, mc, p, fa);
    if (e != cudaSuccess) return cuda_fail(e, "ag_gemm (pairs) launch");
    std::lock_guard<std::mutex> hk(h.mu);
    advance_epochs(grp->members, R, grp->me, grp->lane, R > 1 ? 2 : 0);
    return TMPI_OK;
  }
  int sms = gemm_sm_count();
  if (n_comm <= 0) {
    // as many copy CTAs as the tile count leaves idle anyway: the largest count that does not add
    // a wave of output tiles over what 8 copy CTAs would give
    const int tiles = p.tiles_m * p.tiles_n;
    const int waves = (tiles + sms - 8 - 1) / (sms - 8);
    n_comm = 8;
    while (n_comm + 1 <= sms / 4 && (tiles + sms - n_comm - 2) / (sms - n_comm - 1) == waves) ++n_comm;
  }
  if (n_comm > sms / 4) n_comm = sms / 4;
  fa.sym_off = a_shard_off; fa.local = (__nv_bfloat16*)a_full; fa.ready = ws->ready;
  fa.ready_value = ++ws->ready_value; fa.rows_per_rank = M / R; fa.n_comm = n_comm;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaFuncSetAttribute(gemm::ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm::SMEM_BYTES);
  });
  gemm::ag_gemm_kernel<<<sms, gemm::THREADS, gemm::SMEM_BYTES, (cudaStream_t)stream>>>(ma, mown, mb, mc, (__nv_bfloat16*)C, p, fa);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "ag_gemm launch");
  std::lock_guard<std::mutex> hk(h.mu);
  advance_epochs(grp->members, R, grp->me, grp->lane, R > 1 ? 2 : 0);
  return TMPI_OK;
}

// out[M/R, N] = sum over members of (A[M, K] * B[N, K]^T)[rows of this member].
// slots_off: heap offset of a [R, M/R, N] bf16 scratch array (same on every rank).
// flags: 4 = B is given as [K, N] with N contiguous (CTA-pair kernel only).
int tmpi_cuda_gemm_rs(const void* A, const void* B, size_t slots_off, void* out, int M, int N, int K, int flags,
                      const tmpi_group_t* grp, void* stream) {
  CudaHeap& h = heap();
  if (!h.live || h.emulated) return fail(TMPI_ERR_STATE, "gemm_rs needs a real CUDA heap");
  const int R = grp->nmembers;
  int st = check_fused_shapes(M, N, K, R);
  if (st) return st;
  if ((size_t)(M / R) * N % 8) return fail(TMPI_ERR_INVALID, "gemm_rs: slot size must be a multiple of 8 elements");
  std::lock_guard<std::mutex> lk(g_ws_mu);
  FusedWorkspace* ws;
  if ((st = workspace(&ws))) return st;
  gemm::Problem p{};
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = M / gemm::BM; p.tiles_n = (N + gemm::BN - 1) / gemm::BN; p.k_blocks = K / gemm::BK;
  p.epilogue = 0; p.bias = nullptr; p.status = ws->status;
  const bool b_kn = (flags & gemm::B_IS_KN) != 0;
  if (b_kn && !use_pairs(M, R)) return fail(TMPI_ERR_UNSUPPORTED, "gemm_rs: B as [K, N] needs the CTA-pair kernel (rows per rank %% 256 == 0)");
  gemm::FusedArgs fa{};
  {
    std::lock_guard<std::mutex> hk(h.mu);
    if ((st = fill_peers(&fa.P, grp->members, R, grp->me, grp->lane))) return st;
  }
  CUtensorMap ma, mb;
  if ((st = make_tmap_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, gemm::BM))) return st;
  if (!b_kn && (st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, gemm::BN))) return st;
  if (R > 8) return fail(TMPI_ERR_UNSUPPORTED, "gemm_rs supports at most 8 ranks");
  gemm::SlotMaps sm;
  memset(&sm, 0, sizeof(sm));
  const size_t slot_bytes = (size_t)(M / R) * N * 2;
  for (int o = 0; o < R; ++o) {
    char* slot = fa.P.base[o] + slots_off + (size_t)grp->me * slot_bytes;
    if ((st = make_tmap_bf16(&sm.m[o], slot, (uint64_t)(M / R), (uint64_t)N, (uint64_t)N, gemm::BM))) return st;
  }
  fa.sym_off = slots_off; fa.local = (__nv_bfloat16*)out; fa.rows_per_rank = M / R;
  if (use_pairs(M, R)) {
    static int clusters = 0;
    if (!clusters) clusters = pair_clusters(gemm2::gemm_rs_pair_kernel);
    p.tiles_m = M / (2 * gemm2::BM);
    p.b_mn = b_kn ? 1 : 0;
    if (b_kn) st = make_tmap_bf16(&mb, B, (uint64_t)K, (uint64_t)N, (uint64_t)N, gemm2::BK);
    else st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, gemm2::BN / 2);
    if (st) return st;
    const int ctas = 2 * std::min(clusters, p.tiles_m * p.tiles_n);   // all co-resident: the grid meets at a barrier
    fa.grid_counter = ws->grid_counter;
    ws->grid_total += (unsigned)ctas;
    fa.grid_target = ws->grid_total;
    cudaError_t e = launch_pairs(gemm2::gemm_rs_pair_kernel, ctas, (cudaStream_t)stream, ma, mb, sm, p, fa);
    if (e != cudaSuccess) return cuda_fail(e, "gemm_rs (pairs) launch");
    std::lock_guard<std::mutex> hk(h.mu);
    advance_epochs(grp->members, R, grp->me, grp->lane, R > 1 ? 2 : 0);
    return TMPI_OK;
  }
  int grid = std::min(gemm_sm_count(), p.tiles_m * p.tiles_n);
  fa.grid_counter = ws->grid_counter;
  ws->grid_total += (unsigned)grid;
  fa.grid_target = ws->grid_total;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaFuncSetAttribute(gemm::gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm::SMEM_BYTES);
  });
  gemm::gemm_rs_kernel<<<grid, gemm::THREADS, gemm::SMEM_BYTES, (cudaStream_t)stream>>>(ma, mb, sm, p, fa);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return cuda_fail(e, "gemm_rs launch");
  std::lock_guard<std::mutex> hk(h.mu);
  advance_epochs(grp->members, R, grp->me, grp->lane, R > 1 ? 2 : 0);
  return TMPI_OK;
}

int tmpi_cuda_fused_gemm_status(void) {
  std::lock_guard<std::mutex> lk(g_ws_mu);
  if (!g_ws.status) return 0;
  cudaPointerAttributes at;
  if (cudaPointerGetAttributes(&at, g_ws.status) != cudaSuccess || !at.hostPointer) return 0;
  volatile int* host = (volatile int*)at.hostPointer;
  int v = *host;
  if (v) *host = 0;
  return v;
}

}  // extern "C"
