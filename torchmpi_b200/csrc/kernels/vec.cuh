// 16-byte packs of elements and their accumulators.
//
// Collective and optimizer kernels move data as 16-byte vectors (V = 16 /
// sizeof(T) elements) and, for buffers whose address or length is not 16-byte
// aligned, as single elements (V = 1).  Low-precision floats accumulate in
// fp32, double in double, integers in their own type - the in-register sum that
// replaces the reference's separate `out += in` kernel
// (lib/detail/reduce_kernel.cu:23-136).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tmpi {

template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<__nv_bfloat16> { using type = float; };
template <> struct AccOf<__half> { using type = float; };

template <typename T> __device__ __forceinline__ typename AccOf<T>::type to_acc(T v) { return v; }
template <> __device__ __forceinline__ float to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_acc<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_acc(typename AccOf<T>::type v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_acc<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_acc<__half>(float v) { return __float2half_rn(v); }

template <int BYTES> struct RawOf;
template <> struct RawOf<1> { using type = uint8_t; };
template <> struct RawOf<2> { using type = uint16_t; };
template <> struct RawOf<4> { using type = uint32_t; };
template <> struct RawOf<8> { using type = uint64_t; };

template <typename T, int V>
struct alignas(sizeof(T) * V) Pack {
  T v[V];
};

template <typename T, int V>
__device__ __forceinline__ Pack<T, V> ld_pack(const T* p) {
  return *reinterpret_cast<const Pack<T, V>*>(p);
}
template <typename T, int V>
__device__ __forceinline__ void st_pack(T* p, const Pack<T, V>& x) {
  *reinterpret_cast<Pack<T, V>*>(p) = x;
}

// ---------------------------------------------------------------- debug build: recording bounds checks
// With -DTMPI_DEBUG_BOUNDS every peer load and store first checks that its address lies inside one of the
// mapped heaps (or one of the launch's two local tensors).  An access outside is NOT made: the first one is
// recorded in the lane's status word (code 7, the checked line's block and the address bits) and the kernel
// goes on, so that a wrong offset shows up as a Python error instead of a memory fault.  compute-sanitizer
// is not available where this library is developed; this build stands in for it on the multi-rank kernels.
#ifdef TMPI_DEBUG_BOUNDS
struct DbgBounds {
  const char* lo[20];      // heap bases of the members, the multicast mapping, two local tensors
  size_t len[20];
  int n;
  int* status;             // host-mapped status word of the lane
};
static __device__ DbgBounds g_dbg;   // one copy per translation unit, filled at kernel entry
__device__ __forceinline__ bool dbg_ok(const void* p, size_t bytes) {
  const char* c = reinterpret_cast<const char*>(p);
  for (int i = 0; i < g_dbg.n; ++i)
    if (g_dbg.lo[i] && c >= g_dbg.lo[i] && c + bytes <= g_dbg.lo[i] + g_dbg.len[i]) return true;
  if (g_dbg.status && atomicCAS(g_dbg.status, 0, 7) == 0) {
    g_dbg.status[1] = (int)blockIdx.x;
    g_dbg.status[2] = (int)threadIdx.x;
    g_dbg.status[3] = (int)(((uintptr_t)c >> 4) & 0x7fffffff);
    __threadfence_system();
  }
  return false;
}
#define TMPI_DBG_CHECK(p, bytes) dbg_ok((p), (bytes))
#else
#define TMPI_DBG_CHECK(p, bytes) true
#endif

// peer / streaming variants: bypass L1 (peer lines must not be cached there)
template <typename T, int V>
__device__ __forceinline__ Pack<T, V> ld_pack_peer(const T* p) {
  Pack<T, V> r;
  if (!TMPI_DBG_CHECK(p, sizeof(T) * V)) {
    memset(&r, 0, sizeof(r));
    return r;
  }
  if constexpr (sizeof(T) * V == 16) {
    uint4 u;
    asm volatile("ld.global.relaxed.sys.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(u.x), "=r"(u.y), "=r"(u.z), "=r"(u.w) : "l"(p) : "memory");
    r = *reinterpret_cast<Pack<T, V>*>(&u);
  } else {
    using R = typename RawOf<sizeof(T)>::type;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      R u = *reinterpret_cast<const volatile R*>(p + i);
      r.v[i] = *reinterpret_cast<T*>(&u);
    }
  }
  return r;
}
template <typename T, int V>
__device__ __forceinline__ void st_pack_peer(T* p, const Pack<T, V>& x) {
  if (!TMPI_DBG_CHECK(p, sizeof(T) * V)) return;
  if constexpr (sizeof(T) * V == 16) {
    const uint4 u = *reinterpret_cast<const uint4*>(&x);
    asm volatile("st.global.relaxed.sys.v4.u32 [%0], {%1,%2,%3,%4};"
                 ::"l"(p), "r"(u.x), "r"(u.y), "r"(u.z), "r"(u.w) : "memory");
  } else {
    *reinterpret_cast<Pack<T, V>*>(p) = x;
  }
}

template <typename T, int V>
struct Acc {
  typename AccOf<T>::type a[V];
  __device__ __forceinline__ void set(const Pack<T, V>& x) {
#pragma unroll
    for (int i = 0; i < V; ++i) a[i] = to_acc<T>(x.v[i]);
  }
  __device__ __forceinline__ void add(const Pack<T, V>& x) {
#pragma unroll
    for (int i = 0; i < V; ++i) a[i] += to_acc<T>(x.v[i]);
  }
  __device__ __forceinline__ Pack<T, V> pack(float scale) const {
    Pack<T, V> r;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      auto v = a[i];
      if (scale != 1.0f) v = (typename AccOf<T>::type)(v * scale);
      r.v[i] = from_acc<T>(v);
    }
    return r;
  }
};

}  // namespace tmpi
