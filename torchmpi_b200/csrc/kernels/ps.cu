// One-sided parameter-server kernels: shards stay resident in GPU memory.
//
// The tensor of n elements is split into contiguous shards (floor(n/size) each,
// the first n mod size ranks one more - lib/parameterserver.cpp:282-294); shard
// i lives in the symmetric heap of member i at `shard_off`.  A push applies the
// client's slice to every owner's shard directly over NVLink - plain stores for
// `zero` and `copy`, atomic adds for `add`, which are exact under concurrency -
// and a pull loads every shard into the client's tensor.  No server thread, no
// host staging (the reference stages GPU tensors through pinned host memory and
// MPI messages, torchmpi/parameterserver/init.lua:129-135,189-211).
#include "collectives.cuh"
#include "../include/tmpi_c_api.h"

namespace tmpi {

__device__ __forceinline__ void shard_range(size_t n, int size, int i, size_t* b, size_t* e) {
  size_t q = n / size, r = n % size;
  *b = (size_t)i * q + ((size_t)i < r ? (size_t)i : r);
  *e = *b + q + ((size_t)i < r ? 1 : 0);
}

template <typename T> __device__ __forceinline__ void atomic_add_elem(T* p, T v) { atomicAdd(p, v); }
template <> __device__ __forceinline__ void atomic_add_elem<long long>(long long* p, long long v) {
  atomicAdd(reinterpret_cast<unsigned long long*>(p), (unsigned long long)v);
}

template <typename T>
__global__ void __launch_bounds__(512) ps_kernel(const __grid_constant__ PsArgs a) {
  const Peers& P = a.P;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  T* data = reinterpret_cast<T*>(a.data);
  for (int j = 0; j < P.n; ++j) {
    const int m = (P.me + j) % P.n;          // start at my own shard: clients spread over owners
    size_t b, e;
    shard_range(a.n, P.n, m, &b, &e);
    T* shard = at<T>(P.base[m], a.shard_off);
    const size_t len = e - b;
    if (a.rule < 0) {
      for (size_t i = t0; i < len; i += stride) data[b + i] = ld_pack_peer<T, 1>(shard + i).v[0];
    } else if (a.rule == 0) {
      for (size_t i = t0; i < len; i += stride) shard[i] = from_acc<T>((typename AccOf<T>::type)0);
    } else if (a.rule == 1) {
      for (size_t i = t0; i < len; i += stride) shard[i] = data[b + i];
    } else {
      for (size_t i = t0; i < len; i += stride) atomic_add_elem<T>(shard + i, data[b + i]);
    }
  }
  __threadfence_system();
}

cudaError_t launch_ps(int dtype, const PsArgs* args, int grid, int threads, cudaStream_t s) {
  if (threads > 512) threads = 512;
  switch (dtype) {
    case TMPI_F32: ps_kernel<float><<<grid, threads, 0, s>>>(*args); break;
    case TMPI_F64: ps_kernel<double><<<grid, threads, 0, s>>>(*args); break;
    case TMPI_BF16: ps_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(*args); break;
    case TMPI_F16: ps_kernel<__half><<<grid, threads, 0, s>>>(*args); break;
    case TMPI_I32: ps_kernel<int><<<grid, threads, 0, s>>>(*args); break;
    case TMPI_I64: ps_kernel<long long><<<grid, threads, 0, s>>>(*args); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

}  // namespace tmpi
