// Device bodies of the peer-memory collectives (sm_100a, NVLink 5 / NVSwitch).
//
// NVSwitch gives every GPU full bandwidth to every peer, so nothing here is a
// ring by necessity: a rank reads (or writes) all peers directly.  One launch
// per collective; the host takes no part between its steps.  These kernels
// replace the reference's copy-engine ring with a 2-block reduce kernel and a
// host barrier per step (lib/detail/collectives_cuda.cpp:202-388), its IPC tree
// / pipeline broadcast (:43-159) and its NCCL call sites
// (lib/collectives_cuda.cpp:887-892,960-967,1046-1052).
//
// Bit-identical results on all ranks: every element is summed in member order
// by exactly one rank (two-shot, NVLS, ring, reduce-scatter) or by every rank in
// the same member order (one-shot).
#pragma once
#include "flags.cuh"
#include "launch.h"
#include "vec.cuh"

namespace tmpi {

template <typename T> __device__ __forceinline__ T* at(char* base, size_t off) {
  return reinterpret_cast<T*>(base + off);
}

__device__ __forceinline__ size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// ------------------------------------------------------------------ one-shot (push)
// Slot of writer w (a heap rank) with parity q inside a heap: in_off + (q * world + w) * aux, where the
// host passes the heap's world size in a.root; a lane's region is 2 * world slots (layout_heap).
template <typename T, int V>
__device__ void body_ar_oneshot(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const size_t nv = a.n / V;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t start = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const T* in = reinterpret_cast<const T*>(a.in);
  T* out = reinterpret_cast<T*>(a.out);
  const int my_rank = P.rank_of[P.me];
  for (size_t i = start; i < nv; i += stride) {
    Pack<T, V> x = ld_pack<T, V>(in + i * V);
    for (int m = 0; m < P.n; ++m) {
      if (m == P.me) continue;
      size_t slot = a.in_off + ((size_t)(P.epoch[m] & 1) * (size_t)a.root + my_rank) * a.aux;
      st_pack_peer<T, V>(at<T>(P.base[m], slot) + i * V, x);
    }
  }
  if (!peer_barrier(P, 1, 10, s_abort)) return;
  for (size_t i = start; i < nv; i += stride) {
    Acc<T, V> acc;
    for (int m = 0; m < P.n; ++m) {
      Pack<T, V> x;
      if (m == P.me) {
        x = ld_pack<T, V>(in + i * V);
      } else {
        size_t slot = a.in_off + ((size_t)(P.epoch[m] & 1) * (size_t)a.root + P.rank_of[m]) * a.aux;
        x = ld_pack_peer<T, V>(at<T>(P.base[P.me], slot) + i * V);
      }
      if (m == 0) acc.set(x); else acc.add(x);
    }
    st_pack<T, V>(out + i * V, acc.pack(a.scale));
  }
}

// ------------------------------------------------------------------ two-shot
// NP = number of members known at compile time (0: runtime loop).  Each thread keeps about eight
// 16-byte peer loads in flight (U vectors x NP peers): NVLink round trips take microseconds, so the
// bytes in flight per thread, not the thread count, decide the bandwidth.
template <typename T, int V, int NP>
__device__ __forceinline__ void twoshot_range(const CollArgs& a, size_t lo, size_t hi) {
  const Peers& P = a.P;
  const int n = NP ? NP : P.n;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if constexpr (NP != 0) {
    constexpr int U = NP >= 8 ? 1 : 8 / NP;
    for (; i + (U - 1) * stride < hi; i += U * stride) {
      Pack<T, V> x[U][NP];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int m = 0; m < NP; ++m) x[u][m] = ld_pack_peer<T, V>(at<T>(P.base[m], a.in_off) + (i + u * stride) * V);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        Acc<T, V> acc;
        acc.set(x[u][0]);
#pragma unroll
        for (int m = 1; m < NP; ++m) acc.add(x[u][m]);
        Pack<T, V> r = acc.pack(a.scale);
#pragma unroll
        for (int m = 0; m < NP; ++m) st_pack_peer<T, V>(at<T>(P.base[m], a.out_off) + (i + u * stride) * V, r);
      }
    }
  }
  for (; i < hi; i += stride) {
    Acc<T, V> acc;
    for (int m = 0; m < n; ++m) {
      Pack<T, V> x = ld_pack_peer<T, V>(at<T>(P.base[m], a.in_off) + i * V);
      if (m == 0) acc.set(x); else acc.add(x);
    }
    Pack<T, V> r = acc.pack(a.scale);
    for (int m = 0; m < n; ++m) st_pack_peer<T, V>(at<T>(P.base[m], a.out_off) + i * V, r);
  }
}

template <typename T, int V>
__device__ void body_ar_twoshot(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const size_t nv = a.n / V;
  const size_t per = ceil_div(nv, P.n);
  size_t lo = per * P.me, hi = lo + per;
  if (lo > nv) lo = nv;
  if (hi > nv) hi = nv;
  if (!peer_barrier(P, 1, 20, s_abort)) return;
  switch (P.n) {
    case 2: twoshot_range<T, V, 2>(a, lo, hi); break;
    case 4: twoshot_range<T, V, 4>(a, lo, hi); break;
    case 8: twoshot_range<T, V, 8>(a, lo, hi); break;
    default: twoshot_range<T, V, 0>(a, lo, hi); break;
  }
  peer_barrier(P, 2, 21, s_abort);
}

// ------------------------------------------------------------------ two-shot for tensors outside the heap
// `in` and `out` are ordinary local tensors; the heap only provides scratch.  Phase A scatters: the
// slice that member m owns is pushed from my input into slot [me] of m's scratch (in_off, R slots of
// `per` vectors).  Phase B: every rank sums the R slots of its own slice into its result region
// (out_off).  Phase C gathers: each rank pulls every owner's result straight into its output.  The
// same NVLink bytes as the symmetric two-shot, and no separate copy kernels around the collective.
// grid-strided copy of `len` packs with U loads in flight per thread; either side may be peer memory
template <typename T, int V, int U>
__device__ __forceinline__ void copy_packs(T* dst, const T* src, size_t len, size_t t0, size_t stride) {
  size_t i = t0;
  for (; i + (U - 1) * stride < len; i += U * stride) {
    Pack<T, V> x[U];
#pragma unroll
    for (int u = 0; u < U; ++u) x[u] = ld_pack_peer<T, V>(src + (i + u * stride) * V);
#pragma unroll
    for (int u = 0; u < U; ++u) st_pack_peer<T, V>(dst + (i + u * stride) * V, x[u]);
  }
  for (; i < len; i += stride) st_pack_peer<T, V>(dst + i * V, ld_pack_peer<T, V>(src + i * V));
}

// out[i] = scale * sum over members (in member order) of the pack at element offset `first` + i * V of
// the symmetric buffer at in_off; U vectors per thread and iteration, so U loads per peer are in flight
template <typename T, int V>
__device__ __forceinline__ void sum_from_peers(const Peers& P, size_t in_off, size_t first, T* out, size_t nv, float scale,
                                               size_t t0, size_t stride) {
  constexpr int U = V * sizeof(T) == 16 ? 4 : 2;
  size_t i = t0;
  for (; i + (U - 1) * stride < nv; i += U * stride) {
    Acc<T, V> acc[U];
    for (int m = 0; m < P.n; ++m) {
      const T* src = at<T>(P.base[m], in_off) + first;
      Pack<T, V> x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = ld_pack_peer<T, V>(src + (i + u * stride) * V);
#pragma unroll
      for (int u = 0; u < U; ++u) { if (m == 0) acc[u].set(x[u]); else acc[u].add(x[u]); }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) st_pack<T, V>(out + (i + u * stride) * V, acc[u].pack(scale));
  }
  for (; i < nv; i += stride) {
    Acc<T, V> acc;
    for (int m = 0; m < P.n; ++m) {
      Pack<T, V> x = ld_pack_peer<T, V>(at<T>(P.base[m], in_off) + first + i * V);
      if (m == 0) acc.set(x); else acc.add(x);
    }
    st_pack<T, V>(out + i * V, acc.pack(scale));
  }
}

template <typename T, int V>
__device__ void body_ar_twoshot_any(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const int R = P.n;
  const size_t nv = a.n / V;
  const size_t per = ceil_div(nv, R);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const T* in = reinterpret_cast<const T*>(a.in);
  T* out = reinterpret_cast<T*>(a.out);
  constexpr int U = V * sizeof(T) == 16 ? 8 : 4;
  if (!peer_barrier(P, 1, 25, s_abort)) return;           // everybody is done with the previous use of the scratch
  for (int j = 1; j < R; ++j) {                           // my own slice stays where it is
    const int m = (P.me + j) % R;
    const size_t lo = per * m, len = lo < nv ? (nv - lo < per ? nv - lo : per) : 0;
    copy_packs<T, V, U>(at<T>(P.base[m], a.in_off) + (size_t)P.me * per * V, in + lo * V, len, t0, stride);
  }
  if (!peer_barrier(P, 2, 26, s_abort)) return;
  const size_t mylo = per * P.me, mylen = mylo < nv ? (nv - mylo < per ? nv - mylo : per) : 0;
  {
    const T* slots = at<T>(P.base[P.me], a.in_off);
    T* res = at<T>(P.base[P.me], a.out_off);
    constexpr int UB = 2;
    size_t i = t0;
    for (; i + (UB - 1) * stride < mylen; i += UB * stride) {
      Acc<T, V> acc[UB];
#pragma unroll
      for (int u = 0; u < UB; ++u) acc[u].set(ld_pack<T, V>(in + (mylo + i + u * stride) * V));
      for (int w = 0; w < R; ++w) {
        if (w == P.me) continue;
        Pack<T, V> x[UB];
#pragma unroll
        for (int u = 0; u < UB; ++u) x[u] = ld_pack_peer<T, V>(slots + ((size_t)w * per + i + u * stride) * V);
#pragma unroll
        for (int u = 0; u < UB; ++u) acc[u].add(x[u]);
      }
#pragma unroll
      for (int u = 0; u < UB; ++u) {
        Pack<T, V> r = acc[u].pack(a.scale);
        st_pack<T, V>(res + (i + u * stride) * V, r);       // for the peers
        st_pack<T, V>(out + (mylo + i + u * stride) * V, r); // and my own output
      }
    }
    for (; i < mylen; i += stride) {
      Acc<T, V> acc;
      acc.set(ld_pack<T, V>(in + (mylo + i) * V));
      for (int w = 0; w < R; ++w)
        if (w != P.me) acc.add(ld_pack_peer<T, V>(slots + ((size_t)w * per + i) * V));
      Pack<T, V> r = acc.pack(a.scale);
      st_pack<T, V>(res + i * V, r);
      st_pack<T, V>(out + (mylo + i) * V, r);
    }
  }
  if (!peer_barrier(P, 3, 27, s_abort)) return;
  for (int j = 1; j < R; ++j) {
    const int m = (P.me + j) % R;
    const size_t lo = per * m, len = lo < nv ? (nv - lo < per ? nv - lo : per) : 0;
    copy_packs<T, V, U>(out + lo * V, at<T>(P.base[m], a.out_off), len, t0, stride);
  }
}

// ------------------------------------------------------------------ NVLS (multimem)
template <typename T> struct Multimem {
  static constexpr bool ok = false;
  __device__ static uint4 ld_reduce(const void*) { return uint4{}; }
};
template <> struct Multimem<float> {
  static constexpr bool ok = true;
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct Multimem<__nv_bfloat16> {
  static constexpr bool ok = true;
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
template <> struct Multimem<__half> {
  static constexpr bool ok = true;
  __device__ static uint4 ld_reduce(const void* p) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
  }
};
__device__ __forceinline__ void multimem_st(void* p, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T, int V>
__device__ void body_ar_nvls(const CollArgs& a, int* s_abort) {
  if constexpr (Multimem<T>::ok && V * sizeof(T) == 16) {
    const Peers& P = a.P;
    const size_t nv = a.n / V;
    const size_t per = ceil_div(nv, P.n);
    size_t lo = per * P.me, hi = lo + per;
    if (lo > nv) lo = nv;
    if (hi > nv) hi = nv;
    if (!peer_barrier(P, 1, 30, s_abort)) return;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    auto finish = [&](uint4 u, size_t at_i) {
      if (a.scale != 1.0f) {
        Pack<T, V> x = *reinterpret_cast<Pack<T, V>*>(&u);
        Acc<T, V> acc; acc.set(x);
        x = acc.pack(a.scale);
        u = *reinterpret_cast<uint4*>(&x);
      }
      multimem_st(at<T>(P.mc_base, a.out_off) + at_i * V, u);
    };
    constexpr int U = 8;                      // eight switch reductions in flight per thread
    for (; i + (U - 1) * stride < hi; i += U * stride) {
      uint4 u[U];
#pragma unroll
      for (int k = 0; k < U; ++k) u[k] = Multimem<T>::ld_reduce(at<T>(P.mc_base, a.in_off) + (i + k * stride) * V);
#pragma unroll
      for (int k = 0; k < U; ++k) finish(u[k], i + k * stride);
    }
    for (; i < hi; i += stride) finish(Multimem<T>::ld_reduce(at<T>(P.mc_base, a.in_off) + i * V), i);
    peer_barrier(P, 2, 31, s_abort);
  }
}

// ------------------------------------------------------------------ ring (comparison variant)
// In place on the buffer at out_off.  Chunk schedule of tmpi_ring_{send,recv}_chunk.
template <typename T, int V>
__device__ void body_ar_ring(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const int N = P.n;
  const size_t nv = a.n / V;
  const size_t per = ceil_div(nv, N);
  const int prev = (P.me + N - 1) % N;
  T* mine = at<T>(P.base[P.me], a.out_off);
  const T* theirs = at<T>(P.base[prev], a.out_off);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  uint32_t k = 1;
  if (!peer_barrier(P, k++, 40, s_abort)) return;
  for (int s = 0; s < N - 1; ++s) {
    int c = ((P.me - s - 1) % N + N) % N;
    size_t lo = per * c, hi = lo + per;
    if (lo > nv) lo = nv;
    if (hi > nv) hi = nv;
    const bool last = s == N - 2;
    for (size_t i = lo + t0; i < hi; i += stride) {
      Acc<T, V> acc;
      // fixed order: what arrives from the ring first, then my own contribution
      acc.set(ld_pack_peer<T, V>(theirs + i * V));
      acc.add(ld_pack<T, V>(mine + i * V));
      st_pack<T, V>(mine + i * V, acc.pack(last ? a.scale : 1.0f));
    }
    if (!peer_barrier(P, k++, 41, s_abort)) return;
  }
  for (int s = 0; s < N - 1; ++s) {
    int c = ((P.me - s) % N + N) % N;
    size_t lo = per * c, hi = lo + per;
    if (lo > nv) lo = nv;
    if (hi > nv) hi = nv;
    for (size_t i = lo + t0; i < hi; i += stride)
      st_pack<T, V>(mine + i * V, ld_pack_peer<T, V>(theirs + i * V));
    if (!peer_barrier(P, k++, 42, s_abort)) return;
  }
}

// ------------------------------------------------------------------ broadcast
template <typename T, int V>
__device__ void body_bcast_pull(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const size_t nv = a.n / V;
  if (!peer_barrier(P, 1, 50, s_abort)) return;
  if (P.me != a.root) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    T* dst = at<T>(P.base[P.me], a.out_off);
    const T* src = at<T>(P.base[a.root], a.out_off);
    copy_packs<T, V, 8>(dst, src, nv, (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride);
  }
  peer_barrier(P, 2, 51, s_abort);
}

// Large messages: member m first pulls chunk m from the root (the root sends each byte once),
// then everybody pulls the other chunks from their holders.
template <typename T, int V>
__device__ void body_bcast_chunked(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const int N = P.n;
  const size_t nv = a.n / V;
  const size_t per = ceil_div(nv, N);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  T* dst = at<T>(P.base[P.me], a.out_off);
  auto pull = [&](int chunk, int from) {
    size_t lo = per * chunk, hi = lo + per;
    if (lo > nv) lo = nv;
    if (hi > nv) hi = nv;
    const T* src = at<T>(P.base[from], a.out_off);
    for (size_t i = lo + t0; i < hi; i += stride) st_pack<T, V>(dst + i * V, ld_pack_peer<T, V>(src + i * V));
  };
  if (!peer_barrier(P, 1, 52, s_abort)) return;
  if (P.me != a.root) pull(P.me, a.root);
  if (!peer_barrier(P, 2, 53, s_abort)) return;
  if (P.me != a.root)
    for (int j = 1; j < N; ++j) {
      int m = (P.me + j) % N;          // start at my neighbour so that holders are hit evenly
      pull(m, m);                      // chunk m lives at member m (the root holds everything)
    }
  peer_barrier(P, 3, 54, s_abort);
}

template <typename T, int V>
__device__ void body_bcast_mc(const CollArgs& a, int* s_abort) {
  if constexpr (V * sizeof(T) == 16) {
    const Peers& P = a.P;
    const size_t nv = a.n / V;
    if (!peer_barrier(P, 1, 55, s_abort)) return;
    if (P.me == a.root) {
      const size_t stride = (size_t)gridDim.x * blockDim.x;
      const T* src = at<T>(P.base[P.me], a.out_off);
      constexpr int U = 8;             // bytes in flight per thread: the loads are local, the stores are posted
      size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
      for (; i + (U - 1) * stride < nv; i += U * stride) {
        Pack<T, V> x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) x[u] = ld_pack<T, V>(src + (i + u * stride) * V);
#pragma unroll
        for (int u = 0; u < U; ++u)
          multimem_st(at<T>(P.mc_base, a.out_off) + (i + u * stride) * V, *reinterpret_cast<uint4*>(&x[u]));
      }
      for (; i < nv; i += stride) {
        Pack<T, V> x = ld_pack<T, V>(src + i * V);
        multimem_st(at<T>(P.mc_base, a.out_off) + i * V, *reinterpret_cast<uint4*>(&x));
      }
    }
    peer_barrier(P, 2, 56, s_abort);
  }
}

// Scatter through peer loads, all-gather through the switch, in one pass: member m reads chunk m out of the root's
// buffer and stores it through the multicast mapping, which delivers it to every member (the root included, where it
// rewrites the same values).  The root sends each byte once - 1/N of them as multicast stores of its own chunk - and
// every member's multicast stream carries only 1/N of the message, so no single multicast writer is the limit.
template <typename T, int V>
__device__ void body_bcast_scatter_mc(const CollArgs& a, int* s_abort) {
  if constexpr (V * sizeof(T) == 16) {
    const Peers& P = a.P;
    const size_t nv = a.n / V;
    const size_t per = ceil_div(nv, P.n);
    size_t lo = per * P.me, hi = lo + per;
    if (lo > nv) lo = nv;
    if (hi > nv) hi = nv;
    if (!peer_barrier(P, 1, 59, s_abort)) return;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const T* src = at<T>(P.base[a.root], a.out_off);
    T* mc = at<T>(P.mc_base, a.out_off);
    constexpr int U = 8;
    size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (U - 1) * stride < hi; i += U * stride) {
      Pack<T, V> x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = ld_pack_peer<T, V>(src + (i + u * stride) * V);
#pragma unroll
      for (int u = 0; u < U; ++u) multimem_st(mc + (i + u * stride) * V, *reinterpret_cast<uint4*>(&x[u]));
    }
    for (; i < hi; i += stride) {
      Pack<T, V> x = ld_pack_peer<T, V>(src + i * V);
      multimem_st(mc + i * V, *reinterpret_cast<uint4*>(&x));
    }
    peer_barrier(P, 2, 49, s_abort);
  }
}

// Scatter and all-gather in one pass over plain peer pointers: the message is cut into one chunk per non-root
// member; a member reads its chunk out of the root's buffer and stores every pack it gets into its own buffer and
// into the other non-root members'.  The root sends each byte once and no link carries more than the message
// (a multicast store also returns to its sender and to the root, which costs the receivers a quarter of their
// ingress on four GPUs).  Works on any heap backend: no multicast mapping is needed.
template <typename T, int V>
__device__ void body_bcast_scatter_push(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const int N = P.n;
  const size_t nv = a.n / V;
  if (!peer_barrier(P, 1, 47, s_abort)) return;
  if (P.me != a.root) {
    const int my = P.me < a.root ? P.me : P.me - 1;      // my index among the N - 1 non-root members
    const size_t per = ceil_div(nv, (size_t)(N - 1));
    size_t lo = per * my, hi = lo + per;
    if (lo > nv) lo = nv;
    if (hi > nv) hi = nv;
    const T* src = at<T>(P.base[a.root], a.out_off);
    T* mine = at<T>(P.base[P.me], a.out_off);
    T* dst[kMaxPeers];                                    // the other non-root members, my neighbour first
    int nd = 0;
    for (int j = 1; j < N; ++j) {
      const int m = (P.me + j) % N;
      if (m != a.root) dst[nd++] = at<T>(P.base[m], a.out_off);
    }
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    constexpr int U = 4;
    size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (U - 1) * stride < hi; i += U * stride) {
      Pack<T, V> x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) x[u] = ld_pack_peer<T, V>(src + (i + u * stride) * V);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        st_pack<T, V>(mine + (i + u * stride) * V, x[u]);
        for (int d = 0; d < nd; ++d) st_pack_peer<T, V>(dst[d] + (i + u * stride) * V, x[u]);
      }
    }
    for (; i < hi; i += stride) {
      Pack<T, V> x = ld_pack_peer<T, V>(src + i * V);
      st_pack<T, V>(mine + i * V, x);
      for (int d = 0; d < nd; ++d) st_pack_peer<T, V>(dst[d] + i * V, x);
    }
  }
  peer_barrier(P, 2, 46, s_abort);
}

// Broadcast of a tensor that lives outside the heap: the root pushes its buffer into every peer's
// scratch (one multicast store through the switch when the heap has a multicast mapping, else one
// store per peer), and after the barrier every other rank copies its scratch into its own tensor.
template <typename T, int V>
__device__ void body_bcast_any(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const size_t nv = a.n / V;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  T* buf = reinterpret_cast<T*>(a.out);
  if (!peer_barrier(P, 1, 57, s_abort)) return;            // the scratch is free on every rank
  if (P.me == a.root) {
    const bool mc = a.aux != 0 && V * sizeof(T) == 16;
    if (mc) {
      if constexpr (V * sizeof(T) == 16) {
        constexpr int U = 4;
        size_t i = t0;
        for (; i + (U - 1) * stride < nv; i += U * stride) {
          Pack<T, V> x[U];
#pragma unroll
          for (int u = 0; u < U; ++u) x[u] = ld_pack<T, V>(buf + (i + u * stride) * V);
#pragma unroll
          for (int u = 0; u < U; ++u)
            multimem_st(at<T>(P.mc_base, a.in_off) + (i + u * stride) * V, *reinterpret_cast<uint4*>(&x[u]));
        }
        for (; i < nv; i += stride) {
          Pack<T, V> x = ld_pack<T, V>(buf + i * V);
          multimem_st(at<T>(P.mc_base, a.in_off) + i * V, *reinterpret_cast<uint4*>(&x));
        }
      }
    } else {
      for (int j = 1; j < P.n; ++j)
        copy_packs<T, V, 8>(at<T>(P.base[(P.me + j) % P.n], a.in_off), buf, nv, t0, stride);
    }
  }
  if (!peer_barrier(P, 2, 58, s_abort)) return;
  if (P.me != a.root) {
    const T* src = at<T>(P.base[P.me], a.in_off);
    copy_packs<T, V, 8>(buf, src, nv, t0, stride);
  }
}

// ------------------------------------------------------------------ reduce to root
template <typename T, int V>
__device__ void body_reduce(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const size_t nv = a.n / V;
  if (!peer_barrier(P, 1, 60, s_abort)) return;
  if (P.me == a.root) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    T* out = reinterpret_cast<T*>(a.out);
    bool done = false;
    if constexpr (Multimem<T>::ok && V * sizeof(T) == 16) {
      if (a.aux) {
        // the switch adds the members' vectors on the way: the root receives S bytes instead of (n - 1) S
        constexpr int U = 8;
        const T* mc = at<T>(P.mc_base, a.in_off);
        auto finish = [&](uint4 u, size_t i) {
          Pack<T, V> x = *reinterpret_cast<Pack<T, V>*>(&u);
          if (a.scale != 1.0f) { Acc<T, V> acc; acc.set(x); x = acc.pack(a.scale); }
          st_pack<T, V>(out + i * V, x);
        };
        size_t i = t0;
        for (; i + (U - 1) * stride < nv; i += U * stride) {
          uint4 u[U];
#pragma unroll
          for (int k = 0; k < U; ++k) u[k] = Multimem<T>::ld_reduce(mc + (i + k * stride) * V);
#pragma unroll
          for (int k = 0; k < U; ++k) finish(u[k], i + k * stride);
        }
        for (; i < nv; i += stride) finish(Multimem<T>::ld_reduce(mc + i * V), i);
        done = true;
      }
    }
    if (!done) sum_from_peers<T, V>(P, a.in_off, 0, out, nv, a.scale, t0, stride);
  }
  peer_barrier(P, 2, 61, s_abort);
}

// ------------------------------------------------------------------ all-gather (variable counts)
template <typename T, int V>
__device__ void body_allgather(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  if (!peer_barrier(P, 1, 70, s_abort)) return;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  T* out = reinterpret_cast<T*>(a.out);
  size_t off = 0;
  for (int j = 0; j < P.n; ++j) {
    int m = (P.me + j) % P.n;
    size_t o = 0;
    for (int q = 0; q < m; ++q) o += a.cnt[q];
    const T* src = at<T>(P.base[m], a.in_off);
    const size_t nv = a.cnt[m] / V;
    copy_packs<T, V, 8>(out + o, src, nv, t0, stride);
  }
  (void)off;
  peer_barrier(P, 2, 71, s_abort);
}

// ------------------------------------------------------------------ reduce-scatter
template <typename T, int V>
__device__ void body_reduce_scatter(const CollArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const size_t nv = a.n / V;   // n = elements of the output slice
  if (!peer_barrier(P, 1, 80, s_abort)) return;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  T* out = reinterpret_cast<T*>(a.out);
  sum_from_peers<T, V>(P, a.in_off, (size_t)P.me * a.n, out, nv, a.scale, (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride);
  peer_barrier(P, 2, 81, s_abort);
}

template <typename T, int V>
__device__ void body_barrier(const CollArgs& a, int* s_abort) {
  peer_barrier(a.P, 1, 90, s_abort);
}

}  // namespace tmpi
