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
#include "gemm_core.cuh"
#include "flags.cuh"
#include "vec.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include "../runtime/cuda_state.h"
#include <cstring>
#include <mutex>

namespace tmpi {

int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows);
int gemm_sm_count();

namespace gemm {

struct FusedArgs {
  Peers P;
  size_t sym_off;              // ag: offset of every rank's A shard; rs: offset of the slot array [R][rows][N]
  __nv_bfloat16* local;        // ag: local full-A buffer; rs: local output [rows_per_rank, N]
  uint32_t* ready;             // ag: one flag per M-tile (local memory)
  uint32_t ready_value;
  unsigned int* grid_counter;  // rs: monotonically growing arrival counter (local memory)
  unsigned int grid_target;
  int rows_per_rank;
  int n_comm;
};

constexpr int COPY_BYTES = 32768, COPY_STAGES = 6;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(sm100::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(sm100::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(sm100::smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ------------------------------------------------------------------ all-gather -> GEMM
// Copy-engine body of one comm CTA (all threads enter; one thread drives the copies).
//
// The CTA's tiles (128 rows = tile_bytes contiguous bytes each, own shard first, then the peers in
// ring order) are cut into 32 KB pieces numbered q = 0, 1, ...; piece q uses ring stage q % 6 and
// mbarrier parity (q / 6) & 1.  Steady state of iteration k: piece k has landed -> start its store
// -> wait until all stores but the newest are complete -> publish the tiles they finish ->
// start the load of piece k + 4 (its stage was last used by piece k - 2, whose store is complete).
// Four loads (128 KB) and up to two stores are in flight per CTA.
__device__ void ag_comm(const FusedArgs& g, const Problem& p, unsigned char* tiles, Shared* sh, int* s_abort) {
  const Peers& P = g.P;
  const int R = P.n;
  const int tiles_per_rank = g.rows_per_rank / BM;
  const size_t tile_bytes = (size_t)BM * p.K * 2;
  const int ppt = (int)(tile_bytes / COPY_BYTES);               // pieces per tile (K % 128 == 0 on the host side)
  const int b = blockIdx.x;
  const int cnt = b < tiles_per_rank ? (tiles_per_rank - b + g.n_comm - 1) / g.n_comm : 0;   // my tiles per shard
  const int total = cnt * R * ppt;
  if (!peer_barrier(P, 1, 200, s_abort)) return;                // every rank's shard is ready to be read
  if (threadIdx.x == 0 && total > 0) {
    uint64_t* bars = sh->full;                                   // full[0..3], empty[0..1]: six contiguous barriers
    auto src_of = [&](int q, const char** sp, char** dp, int* m_tile) {
      const int u = q / ppt, pi = q % ppt;
      // peers in ring order first; my own shard last (the GEMM reads it in place, the copy only completes A_full)
      const int src = (P.me + 1 + u / cnt) % R, c = b + (u % cnt) * g.n_comm;
      *m_tile = src * tiles_per_rank + c;
      *sp = P.base[src] + g.sym_off + (size_t)c * tile_bytes + (size_t)pi * COPY_BYTES;
      *dp = (char*)g.local + (size_t)(*m_tile) * tile_bytes + (size_t)pi * COPY_BYTES;
    };
    auto load = [&](int q) {
      const char* sp; char* dp; int mt;
      src_of(q, &sp, &dp, &mt);
      const int st = q % COPY_STAGES;
      sm100::mbar_expect_tx(&bars[st], COPY_BYTES);
      bulk_load(tiles + (size_t)st * COPY_BYTES, sp, COPY_BYTES, &bars[st]);
    };
    auto publish = [&](int q) {                                  // piece q is complete in local memory
      if (q % ppt != ppt - 1) return;
      const char* sp; char* dp; int mt;
      src_of(q, &sp, &dp, &mt);
      sm100::fence_proxy_async();
      __threadfence();
      st_release_gpu(&g.ready[mt], g.ready_value);
    };
    bool ok = true;
    for (int q = 0; q < 4 && q < total; ++q) load(q);
    for (int k = 0; k < total; ++k) {
      const int st = k % COPY_STAGES;
      if (!sm100::mbar_wait(&bars[st], (uint32_t)((k / COPY_STAGES) & 1), kWaitBudgetNs)) { ok = false; break; }
      const char* sp; char* dp; int mt;
      src_of(k, &sp, &dp, &mt);
      bulk_store(dp, tiles + (size_t)st * COPY_BYTES, COPY_BYTES);
      bulk_commit();
      asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); // stores of pieces <= k - 1 are complete
      if (k >= 1) publish(k - 1);
      if (k + 4 < total) load(k + 4);                           // its stage was last used by piece k - 2
    }
    bulk_wait_all();
    if (ok) {
      publish(total - 1);
    } else {
      fail(sh, p, 10);
      atomicExch(s_abort, 1);
    }
  }
  peer_barrier(P, 2, 201, s_abort);                              // nobody still reads my shard
}

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
    const size_t nv = slot_elems / 8;
    for (size_t i = (size_t)blockIdx.x * THREADS + threadIdx.x; i < nv; i += (size_t)gridDim.x * THREADS) {
      Acc<__nv_bfloat16, 8> acc;
      for (int r = 0; r < R; ++r) {
        Pack<__nv_bfloat16, 8> x = ld_pack_peer<__nv_bfloat16, 8>(slots + (size_t)r * slot_elems + i * 8);
        if (r == 0) acc.set(x); else acc.add(x);
      }
      st_pack<__nv_bfloat16, 8>(g.local + i * 8, acc.pack(1.0f));
    }
    peer_barrier(P, 2, 211, &s_abort);      // slots may be overwritten by the next call only after everyone has summed
  }
  teardown(sh, warp);
}

}  // namespace gemm
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
  p.epilogue = epilogue; p.bias = (const __nv_bfloat16*)bias; p.status = ws->status;
  gemm::FusedArgs fa{};
  {
    std::lock_guard<std::mutex> hk(h.mu);
    if ((st = fill_peers(&fa.P, grp->members, R, grp->me, grp->lane))) return st;
  }
  char* a_full = h.base[h.rank] + a_full_off;
  CUtensorMap ma, mb;
  if ((st = make_tmap_bf16(&ma, a_full, (uint64_t)M, (uint64_t)K, (uint64_t)K, gemm::BM))) return st;
  if ((st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, gemm::BN))) return st;
  CUtensorMap mc;
  if ((st = make_tmap_bf16(&mc, C, (uint64_t)M, (uint64_t)N, (uint64_t)N, gemm::BM))) return st;
  CUtensorMap mown;
  if ((st = make_tmap_bf16(&mown, h.base[h.rank] + a_shard_off, (uint64_t)(M / R), (uint64_t)K, (uint64_t)K, gemm::BM))) return st;
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
int tmpi_cuda_gemm_rs(const void* A, const void* B, size_t slots_off, void* out, int M, int N, int K,
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
  gemm::FusedArgs fa{};
  {
    std::lock_guard<std::mutex> hk(h.mu);
    if ((st = fill_peers(&fa.P, grp->members, R, grp->me, grp->lane))) return st;
  }
  CUtensorMap ma, mb;
  if ((st = make_tmap_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, gemm::BM))) return st;
  if ((st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, gemm::BN))) return st;
  if (R > 8) return fail(TMPI_ERR_UNSUPPORTED, "gemm_rs supports at most 8 ranks");
  gemm::SlotMaps sm;
  memset(&sm, 0, sizeof(sm));
  const size_t slot_bytes = (size_t)(M / R) * N * 2;
  for (int o = 0; o < R; ++o) {
    char* slot = fa.P.base[o] + slots_off + (size_t)grp->me * slot_bytes;
    if ((st = make_tmap_bf16(&sm.m[o], slot, (uint64_t)(M / R), (uint64_t)N, (uint64_t)N, gemm::BM))) return st;
  }
  int grid = std::min(gemm_sm_count(), p.tiles_m * p.tiles_n);
  fa.sym_off = slots_off; fa.local = (__nv_bfloat16*)out; fa.rows_per_rank = M / R;
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
