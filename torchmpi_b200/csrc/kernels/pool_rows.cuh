// Shared-memory gather for the backward of a 3x3 / stride-2 / pad-1 max-pool with a one-byte window
// index (pool.cu, bn_relu.cu).  A block works on the input rows 2k and 2k + 1 of one image; the
// windows that cover them lie in the output rows k and k + 1.
#pragma once
#include "vec.cuh"

namespace tmpi {

constexpr int kBpThreads = 256;
struct BpDims { int N, H, W, C, OH, OW; };

// The two output rows go to shared memory (gradient and index) with one extra zero column and a zero
// row where the image ends.
template <typename T, int V>
__device__ __forceinline__ void stage_pool_rows(const T* __restrict__ dy, const unsigned char* __restrict__ idx, const BpDims& d,
                                                int n, int k, T* s_dy, unsigned char* s_ix) {
  const int cvn = d.C / V, pw = d.OW + 1;
  constexpr int U = 4;
  const int items = 2 * pw * cvn;
  for (int t0 = threadIdx.x; t0 < items; t0 += U * kBpThreads) {
    Pack<T, V> g[U];
    Pack<unsigned char, V> iv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u * kBpThreads;
      const int pos = t / cvn, cvv = t - pos * cvn;
      const int row = pos / pw, ow = pos - row * pw;
      const int oh = k + row;
#pragma unroll
      for (int c = 0; c < V; ++c) { g[u].v[c] = from_acc<T>((typename AccOf<T>::type)0.f); iv[u].v[c] = 255; }
      if (t < items && oh < d.OH && ow < d.OW) {
        const size_t o = ((((size_t)n * d.OH + oh) * d.OW + ow) * cvn + cvv) * V;
        g[u] = ld_pack<T, V>(dy + o);
        iv[u] = ld_pack<unsigned char, V>(idx + o);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u * kBpThreads;
      if (t >= items) break;
      st_pack<T, V>(s_dy + (size_t)t * V, g[u]);
      st_pack<unsigned char, V>(s_ix + (size_t)t * V, iv[u]);
    }
  }
}

// gradient routed by the pool to input position (ih, iw), channel group cv, from the staged rows
template <typename T, int V>
__device__ __forceinline__ void pooled_grad(const T* s_dy, const unsigned char* s_ix, const BpDims& d, int k, int ih, int iw,
                                            int cv, float (&g)[V]) {
  const int cvn = d.C / V, pw = d.OW + 1;
#pragma unroll
  for (int c = 0; c < V; ++c) g[c] = 0.f;
  // windows [2o - 1, 2o + 1] containing a coordinate i: o = i >> 1 and, for odd i, o + 1
  const int ow_lo = iw >> 1;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const int dr = q >> 1, dc = q & 1;
    if ((dr && !(ih & 1)) || (dc && !(iw & 1))) continue;
    const int oh = (ih >> 1) + dr, ow = ow_lo + dc;             // ow <= OW (the zero column), oh - k in {0, 1}
    const size_t o = ((size_t)((oh - k) * pw + ow) * cvn + cv) * V;
    Pack<unsigned char, V> iv = ld_pack<unsigned char, V>(s_ix + o);
    Pack<T, V> gv = ld_pack<T, V>(s_dy + o);
    const unsigned char w = (unsigned char)((ih - (oh * 2 - 1)) * 3 + (iw - (ow * 2 - 1)));
#pragma unroll
    for (int c = 0; c < V; ++c)
      if (iv.v[c] == w) g[c] += (float)to_acc<T>(gv.v[c]);
  }
}

}  // namespace tmpi
