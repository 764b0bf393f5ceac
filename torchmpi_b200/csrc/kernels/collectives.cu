// Kernel wrappers and host-side dispatch of the peer-memory collectives.
//
// Every op has two entry kernels around the same device body: the real one (one
// rank per GPU, arguments by value) and an emulation one in which gridDim.y
// enumerates all ranks of a single-GPU heap; the latter is launched
// cooperatively so that the blocks that wait on one another are co-resident.
#include "collectives.cuh"
#include "../include/tmpi_c_api.h"

namespace tmpi {

template <int OP, typename T, int V>
__device__ __forceinline__ void run_body(const CollArgs& a, int* s_abort) {
  if constexpr (OP == OP_AR_ONESHOT) body_ar_oneshot<T, V>(a, s_abort);
  else if constexpr (OP == OP_AR_TWOSHOT) body_ar_twoshot<T, V>(a, s_abort);
  else if constexpr (OP == OP_AR_TWOSHOT_ANY) body_ar_twoshot_any<T, V>(a, s_abort);
  else if constexpr (OP == OP_AR_NVLS) body_ar_nvls<T, V>(a, s_abort);
  else if constexpr (OP == OP_AR_RING) body_ar_ring<T, V>(a, s_abort);
  else if constexpr (OP == OP_BCAST_PULL) body_bcast_pull<T, V>(a, s_abort);
  else if constexpr (OP == OP_BCAST_CHUNKED) body_bcast_chunked<T, V>(a, s_abort);
  else if constexpr (OP == OP_BCAST_MC) body_bcast_mc<T, V>(a, s_abort);
  else if constexpr (OP == OP_BCAST_ANY) body_bcast_any<T, V>(a, s_abort);
  else if constexpr (OP == OP_BCAST_SCATTER_MC) body_bcast_scatter_mc<T, V>(a, s_abort);
  else if constexpr (OP == OP_BCAST_SCATTER_PUSH) body_bcast_scatter_push<T, V>(a, s_abort);
  else if constexpr (OP == OP_REDUCE) body_reduce<T, V>(a, s_abort);
  else if constexpr (OP == OP_ALLGATHER) body_allgather<T, V>(a, s_abort);
  else if constexpr (OP == OP_REDUCE_SCATTER) body_reduce_scatter<T, V>(a, s_abort);
  else body_barrier<T, V>(a, s_abort);
}

template <int OP, typename T, int V>
__global__ void __launch_bounds__(1024) coll_kernel(const __grid_constant__ CollArgs a) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  // local tensors of ops that take ordinary pointers: generous windows (the strict check is on the heaps)
  TMPI_DBG_ENTER(a.P, a.in, a.n * sizeof(T) * kMaxPeers, a.out, a.n * sizeof(T) * kMaxPeers);
  __syncthreads();
  run_body<OP, T, V>(a, &s_abort);
}

template <int OP, typename T, int V>
__global__ void __launch_bounds__(1024) coll_kernel_emu(const __grid_constant__ CollArgsPack pack) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  TMPI_DBG_ENTER(pack.r[blockIdx.y].P, pack.r[blockIdx.y].in, pack.r[blockIdx.y].n * sizeof(T) * kMaxPeers,
                 pack.r[blockIdx.y].out, pack.r[blockIdx.y].n * sizeof(T) * kMaxPeers);
  __syncthreads();
  run_body<OP, T, V>(pack.r[blockIdx.y], &s_abort);
}

int barriers_used(int op, int n) {
  if (n <= 1) return 0;
  switch (op) {
    case OP_AR_ONESHOT: return 1;
    case OP_AR_RING: return 1 + 2 * (n - 1);
    case OP_BCAST_CHUNKED: return 3;
    case OP_AR_TWOSHOT_ANY: return 3;
    case OP_BARRIER: return 1;
    default: return 2;
  }
}

template <int OP, typename T, int V>
cudaError_t launch_typed(const CollArgs* args, int nranks, int grid, int threads, cudaStream_t s) {
  if (nranks == 1) {
    coll_kernel<OP, T, V><<<grid, threads, 0, s>>>(args[0]);
    return cudaGetLastError();
  }
  CollArgsPack pack;
  for (int r = 0; r < nranks && r < 8; ++r) pack.r[r] = args[r];
  void* params[] = {&pack};
  return cudaLaunchCooperativeKernel((void*)coll_kernel_emu<OP, T, V>, dim3(grid, nranks), dim3(threads),
                                     params, 0, s);
}

template <int OP, typename T>
cudaError_t launch_vec(const CollArgs* args, int nranks, int vec, int grid, int threads, cudaStream_t s) {
  if (vec) return launch_typed<OP, T, 16 / sizeof(T)>(args, nranks, grid, threads, s);
  return launch_typed<OP, T, 1>(args, nranks, grid, threads, s);
}

// reductions depend on the element type
template <int OP>
cudaError_t launch_reduction(int dtype, const CollArgs* a, int nr, int vec, int g, int t, cudaStream_t s) {
  switch (dtype) {
    case TMPI_U8: return launch_vec<OP, uint8_t>(a, nr, vec, g, t, s);
    case TMPI_I8: return launch_vec<OP, int8_t>(a, nr, vec, g, t, s);
    case TMPI_I16: return launch_vec<OP, int16_t>(a, nr, vec, g, t, s);
    case TMPI_I32: return launch_vec<OP, int32_t>(a, nr, vec, g, t, s);
    case TMPI_I64: return launch_vec<OP, long long>(a, nr, vec, g, t, s);
    case TMPI_F16: return launch_vec<OP, __half>(a, nr, vec, g, t, s);
    case TMPI_BF16: return launch_vec<OP, __nv_bfloat16>(a, nr, vec, g, t, s);
    case TMPI_F32: return launch_vec<OP, float>(a, nr, vec, g, t, s);
    case TMPI_F64: return launch_vec<OP, double>(a, nr, vec, g, t, s);
  }
  return cudaErrorInvalidValue;
}

template <int OP>
cudaError_t launch_float_only(int dtype, const CollArgs* a, int nr, int g, int t, cudaStream_t s) {
  switch (dtype) {
    case TMPI_F16: return launch_typed<OP, __half, 8>(a, nr, g, t, s);
    case TMPI_BF16: return launch_typed<OP, __nv_bfloat16, 8>(a, nr, g, t, s);
    case TMPI_F32: return launch_typed<OP, float, 4>(a, nr, g, t, s);
  }
  return cudaErrorInvalidValue;
}

// copies only move bytes: n is re-expressed in bytes by the caller
template <int OP>
cudaError_t launch_bytes(const CollArgs* a, int nr, int vec, int g, int t, cudaStream_t s) {
  return launch_vec<OP, uint8_t>(a, nr, vec, g, t, s);
}

cudaError_t launch_collective(int op, int dtype, const CollArgs* args, int nranks, int vec,
                              int grid, int threads, cudaStream_t s) {
  if (grid < 1) grid = 1;
  if (grid > kMaxBlocks) grid = kMaxBlocks;
  switch (op) {
    case OP_AR_ONESHOT: return launch_reduction<OP_AR_ONESHOT>(dtype, args, nranks, vec, grid, threads, s);
    case OP_AR_TWOSHOT: return launch_reduction<OP_AR_TWOSHOT>(dtype, args, nranks, vec, grid, threads, s);
    case OP_AR_RING: return launch_reduction<OP_AR_RING>(dtype, args, nranks, vec, grid, threads, s);
    case OP_AR_TWOSHOT_ANY: return launch_reduction<OP_AR_TWOSHOT_ANY>(dtype, args, nranks, vec, grid, threads, s);
    case OP_REDUCE: return launch_reduction<OP_REDUCE>(dtype, args, nranks, vec, grid, threads, s);
    case OP_REDUCE_SCATTER: return launch_reduction<OP_REDUCE_SCATTER>(dtype, args, nranks, vec, grid, threads, s);
    case OP_AR_NVLS: return launch_float_only<OP_AR_NVLS>(dtype, args, nranks, grid, threads, s);
    case OP_BCAST_PULL: return launch_bytes<OP_BCAST_PULL>(args, nranks, vec, grid, threads, s);
    case OP_BCAST_CHUNKED: return launch_bytes<OP_BCAST_CHUNKED>(args, nranks, vec, grid, threads, s);
    case OP_BCAST_MC: return launch_typed<OP_BCAST_MC, uint8_t, 16>(args, nranks, grid, threads, s);
    case OP_BCAST_SCATTER_MC: return launch_typed<OP_BCAST_SCATTER_MC, uint8_t, 16>(args, nranks, grid, threads, s);
    case OP_BCAST_SCATTER_PUSH: return launch_bytes<OP_BCAST_SCATTER_PUSH>(args, nranks, vec, grid, threads, s);
    case OP_ALLGATHER: return launch_bytes<OP_ALLGATHER>(args, nranks, vec, grid, threads, s);
    case OP_BCAST_ANY: return launch_bytes<OP_BCAST_ANY>(args, nranks, vec, grid, threads, s);
    case OP_BARRIER: return launch_typed<OP_BARRIER, uint8_t, 1>(args, nranks, grid, threads, s);
  }
  return cudaErrorInvalidValue;
}

// A wait on a flag that nobody sets: exercises the bounded-wait path (tests).
__global__ void wait_probe_kernel(const __grid_constant__ Peers P) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    // lane kMaxLanes-1, block kMaxBlocks-1 is reserved for this probe and never signalled
    uint32_t* f = flag_ptr(P.base[P.me], kMaxLanes - 1, kMaxBlocks - 1, 0);
    uint32_t want = ld_acquire_sys(f) + 1;
    if (!wait_flag(f, want, P.budget_ns)) report(P, ST_TIMEOUT, 99, -1, want);
  }
}

cudaError_t launch_wait_probe(const Peers& P, cudaStream_t s) {
  wait_probe_kernel<<<1, 32, 0, s>>>(P);
  return cudaGetLastError();
}

}  // namespace tmpi
