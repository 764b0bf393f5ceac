// One-sided parameter-server kernels: shards stay resident in GPU memory.
//
// The tensor of n elements is split into contiguous shards (floor(n/size) each, the first
// n mod size ranks one more - lib/parameterserver.cpp:282-294); shard i lives in the symmetric heap
// of member i at `shard_off`.  A push applies the client's slice to every owner's shard directly
// over NVLink - plain stores for `zero` and `copy`, atomic adds (`red`) for `add`, which are exact
// under concurrency - and a pull loads every shard into the client's tensor.  No server thread, no
// host staging (the reference stages GPU tensors through pinned host memory and MPI messages,
// torchmpi/parameterserver/init.lua:129-135,189-211).  Slices whose client-side address is
// 16-byte aligned move as 16-byte packs (vector `red` for fp32 adds); the rest element by element.
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

// 16 bytes of additions in one reduction message where the type allows it
template <typename T, int V>
__device__ __forceinline__ void red_add_pack(T* p, const Pack<T, V>& x) {
#pragma unroll
  for (int k = 0; k < V; ++k) atomic_add_elem<T>(p + k, x.v[k]);
}
template <>
__device__ __forceinline__ void red_add_pack<float, 4>(float* p, const Pack<float, 4>& x) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "f"(x.v[0]), "f"(x.v[1]), "f"(x.v[2]), "f"(x.v[3]) : "memory");
}
template <>
__device__ __forceinline__ void red_add_pack<__nv_bfloat16, 8>(__nv_bfloat16* p, const Pack<__nv_bfloat16, 8>& x) {
  const uint4 u = *reinterpret_cast<const uint4*>(&x);
  asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
}
template <>
__device__ __forceinline__ void red_add_pack<__half, 8>(__half* p, const Pack<__half, 8>& x) {
  const uint4 u = *reinterpret_cast<const uint4*>(&x);
  asm volatile("red.relaxed.sys.global.add.noftz.v4.f16x2 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
}

template <typename T, int V>
__device__ __forceinline__ void ps_range(T* shard, T* data, size_t len, int rule, size_t t0, size_t stride) {
  const size_t nv = len / V;
  if (rule < 0) {
    // pulls are remote loads: keep eight of them in flight per thread
    constexpr int U = 8;
    size_t i = t0;
    for (; i + (U - 1) * stride < nv; i += U * stride) {
      Pack<T, V> x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = ld_pack_peer<T, V>(shard + (i + u * stride) * V);
#pragma unroll
      for (int u = 0; u < U; ++u) st_pack<T, V>(data + (i + u * stride) * V, x[u]);
    }
    for (; i < nv; i += stride) st_pack<T, V>(data + i * V, ld_pack_peer<T, V>(shard + i * V));
  } else if (rule == 0) {
    Pack<T, V> z;
#pragma unroll
    for (int k = 0; k < V; ++k) z.v[k] = from_acc<T>((typename AccOf<T>::type)0);
    for (size_t i = t0; i < nv; i += stride) st_pack_peer<T, V>(shard + i * V, z);
  } else if (rule == 1) {
    for (size_t i = t0; i < nv; i += stride) st_pack_peer<T, V>(shard + i * V, ld_pack<T, V>(data + i * V));
  } else {
    for (size_t i = t0; i < nv; i += stride) red_add_pack<T, V>(shard + i * V, ld_pack<T, V>(data + i * V));
  }
}

// All owners inside the inner loop: a thread applies vector i of EVERY shard before it moves on, so that
// loads from (or reductions into) all peers are in flight at once, as the two-shot allreduce does, instead of
// the whole grid visiting one owner at a time.  NP owners, known at compile time; every shard's slice of the
// client's tensor starts on 16 bytes.  U rounds per iteration keep about eight 16-byte transfers in flight.
template <typename T, int V, int NP>
__device__ __forceinline__ void ps_all_owners(const PsArgs& a, T* data, size_t t0, size_t stride) {
  const Peers& P = a.P;
  T* shard[NP];
  T* mine[NP];
  size_t nv[NP], maxnv = 0;
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int m = (P.me + j) % NP;            // rotate: clients start at different owners
    size_t b, e;
    shard_range(a.n, NP, m, &b, &e);
    shard[j] = at<T>(P.base[m], a.shard_off);
    mine[j] = data + b;
    nv[j] = (e - b) / V;
    maxnv = nv[j] > maxnv ? nv[j] : maxnv;
  }
  constexpr int U = NP >= 8 ? 1 : 8 / NP;
  const int rule = a.rule;
  Pack<T, V> z;
#pragma unroll
  for (int k = 0; k < V; ++k) z.v[k] = from_acc<T>((typename AccOf<T>::type)0);
  for (size_t i = t0; i < maxnv; i += U * stride) {
    Pack<T, V> x[U][NP];
    if (rule < 0) {                           // pull: all loads first
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < NP; ++j)
          if (i + u * stride < nv[j]) x[u][j] = ld_pack_peer<T, V>(shard[j] + (i + u * stride) * V);
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < NP; ++j)
          if (i + u * stride < nv[j]) st_pack<T, V>(mine[j] + (i + u * stride) * V, x[u][j]);
    } else {
      if (rule != 0) {
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
          for (int j = 0; j < NP; ++j)
            if (i + u * stride < nv[j]) x[u][j] = ld_pack<T, V>(mine[j] + (i + u * stride) * V);
      }
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int j = 0; j < NP; ++j)
          if (i + u * stride < nv[j]) {
            T* dst = shard[j] + (i + u * stride) * V;
            if (rule == 0) st_pack_peer<T, V>(dst, z);
            else if (rule == 1) st_pack_peer<T, V>(dst, x[u][j]);
            else red_add_pack<T, V>(dst, x[u][j]);
          }
    }
  }
  // the elements of each shard beyond its last full pack
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const int m = (P.me + j) % NP;
    size_t b, e;
    shard_range(a.n, NP, m, &b, &e);
    const size_t body = nv[j] * V;
    ps_range<T, 1>(shard[j] + body, mine[j] + body, (e - b) - body, rule, t0, stride);
  }
}

// true when the slice of every owner starts on a 16-byte boundary of the client's tensor
template <typename T>
__device__ __forceinline__ bool ps_slices_aligned(const PsArgs& a, const T* data) {
  for (int m = 0; m < a.P.n; ++m) {
    size_t b, e;
    shard_range(a.n, a.P.n, m, &b, &e);
    if ((uintptr_t)(data + b) & 15) return false;
  }
  return true;
}

template <typename T>
__global__ void __launch_bounds__(512) ps_kernel(const __grid_constant__ PsArgs a) {
  const Peers& P = a.P;
  constexpr int V = 16 / sizeof(T);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  T* data = reinterpret_cast<T*>(a.data);
  TMPI_DBG_ENTER(P, nullptr, 0, nullptr, 0);
#ifdef TMPI_DEBUG_BOUNDS
  __syncthreads();
#endif
  if ((P.n == 2 || P.n == 4 || P.n == 8) && ps_slices_aligned<T>(a, data)) {
    if (P.n == 2) ps_all_owners<T, V, 2>(a, data, t0, stride);
    else if (P.n == 4) ps_all_owners<T, V, 4>(a, data, t0, stride);
    else ps_all_owners<T, V, 8>(a, data, t0, stride);
    __threadfence_system();
    return;
  }
  for (int j = 0; j < P.n; ++j) {
    const int m = (P.me + j) % P.n;          // start at my own shard: clients spread over owners
    size_t b, e;
    shard_range(a.n, P.n, m, &b, &e);
    T* shard = at<T>(P.base[m], a.shard_off);   // 256-byte aligned
    const size_t len = e - b;
    if (((uintptr_t)(data + b) & 15) == 0) {
      const size_t body = len / V * V;
      ps_range<T, V>(shard, data + b, body, a.rule, t0, stride);
      ps_range<T, 1>(shard + body, data + b + body, len - body, a.rule, t0, stride);
    } else {
      ps_range<T, 1>(shard, data + b, len, a.rule, t0, stride);
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
