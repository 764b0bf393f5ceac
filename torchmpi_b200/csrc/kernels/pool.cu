// Max pooling for channels-last activations, forward (with window index) and backward.
//
// Forward: one thread per output position and group of V channels (one 16-byte pack); it scans
// the k x k window, keeps the first maximum (strictly-greater comparison, NaN propagates) and stores
// the value and the position inside the window as one byte per element.  Backward: one thread per
// input position and channel group gathers from the (at most ceil(k/s)^2) outputs whose window
// covers it and whose stored index points at it - no atomics, every byte of dx written once.
// Traffic is one read of the input and one write of output + index forward, and a read of
// dy + index and one write of dx backward.
#include "vec.cuh"
#include "pool_rows.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include <algorithm>

namespace tmpi {

struct PoolDims { int N, H, W, C, OH, OW, k, s, p; };

// One block per (image, output row) forward and per (image, input row) backward: the row index comes
// from blockIdx and the position inside the row from 32-bit arithmetic (a flat 64-bit index with
// three run-time divisions per element cost more than the memory traffic).
// K3: the window is 3 x 3 (all nine loads are issued before the first comparison).
template <typename T, int V, bool K3>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                          unsigned char* __restrict__ idx, PoolDims d) {
  const int cvn = d.C / V;
  const int n = blockIdx.x / d.OH, oh = blockIdx.x % d.OH;
  const int ih0 = oh * d.s - d.p;
  const T* xin = x + (size_t)n * d.H * d.W * d.C;
  const size_t orow = ((size_t)n * d.OH + oh) * d.OW * d.C;
  for (int t = threadIdx.x; t < d.OW * cvn; t += blockDim.x) {
    const int ow = t / cvn, cv = t - ow * cvn;
    const int iw0 = ow * d.s - d.p;
    float best[V];
    unsigned char bi[V];
    bool first = true;
    if constexpr (K3) {
      Pack<T, V> win[9];
      bool ok[9];
#pragma unroll
      for (int q = 0; q < 9; ++q) {
        const int ih = ih0 + q / 3, iw = iw0 + q % 3;
        ok[q] = ih >= 0 && ih < d.H && iw >= 0 && iw < d.W;
        if (ok[q]) win[q] = ld_pack<T, V>(xin + ((size_t)ih * d.W + iw) * d.C + cv * V);
      }
#pragma unroll
      for (int q = 0; q < 9; ++q) {
        if (!ok[q]) continue;
#pragma unroll
        for (int c = 0; c < V; ++c) {
          const float f = (float)to_acc<T>(win[q].v[c]);
          if (first || f > best[c] || f != f) { best[c] = f; bi[c] = (unsigned char)q; }
        }
        first = false;
      }
    } else
    for (int kh = 0; kh < d.k; ++kh) {
      const int ih = ih0 + kh;
      if (ih < 0 || ih >= d.H) continue;
      for (int kw = 0; kw < d.k; ++kw) {
        const int iw = iw0 + kw;
        if (iw < 0 || iw >= d.W) continue;
        Pack<T, V> v = ld_pack<T, V>(xin + ((size_t)ih * d.W + iw) * d.C + cv * V);
#pragma unroll
        for (int c = 0; c < V; ++c) {
          const float f = (float)to_acc<T>(v.v[c]);
          if (first || f > best[c] || f != f) { best[c] = f; bi[c] = (unsigned char)(kh * d.k + kw); }
        }
        first = false;
      }
    }
    Pack<T, V> out;
    Pack<unsigned char, V> oi;
#pragma unroll
    for (int c = 0; c < V; ++c) { out.v[c] = from_acc<T>((typename AccOf<T>::type)best[c]); oi.v[c] = bi[c]; }
    st_pack<T, V>(y + orow + (size_t)t * V, out);
    st_pack<unsigned char, V>(idx + orow + (size_t)t * V, oi);
  }
}

// C2: at most two outputs per axis cover an input (k <= 2 s): their loads are issued together.
template <typename T, int V, bool C2>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const T* __restrict__ dy, const unsigned char* __restrict__ idx,
                                                          T* __restrict__ dx, PoolDims d) {
  const int cvn = d.C / V;
  const int n = blockIdx.x / d.H, ih = blockIdx.x % d.H;
  // outputs whose window [o*s - p, o*s - p + k) contains the input coordinate
  int oh_lo = ih + d.p - d.k + 1; oh_lo = oh_lo <= 0 ? 0 : (oh_lo + d.s - 1) / d.s;
  const int oh_hi = min((ih + d.p) / d.s, d.OH - 1);
  const size_t obase = (size_t)n * d.OH * d.OW * d.C;
  const size_t irow = ((size_t)n * d.H + ih) * d.W * d.C;
  for (int t = threadIdx.x; t < d.W * cvn; t += blockDim.x) {
    const int iw = t / cvn, cv = t - iw * cvn;
    int ow_lo = iw + d.p - d.k + 1; ow_lo = ow_lo <= 0 ? 0 : (ow_lo + d.s - 1) / d.s;
    const int ow_hi = min((iw + d.p) / d.s, d.OW - 1);
    float acc[V];
#pragma unroll
    for (int c = 0; c < V; ++c) acc[c] = 0.f;
    if constexpr (C2) {
      Pack<unsigned char, V> iv[4];
      Pack<T, V> gv[4];
      bool ok[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int oh = oh_lo + (q >> 1), ow = ow_lo + (q & 1);
        ok[q] = oh <= oh_hi && ow <= ow_hi;
        if (ok[q]) {
          const size_t o = obase + ((size_t)(oh * d.OW + ow) * cvn + cv) * V;
          iv[q] = ld_pack<unsigned char, V>(idx + o);
          gv[q] = ld_pack<T, V>(dy + o);
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (!ok[q]) continue;
        const int oh = oh_lo + (q >> 1), ow = ow_lo + (q & 1);
        const unsigned char w = (unsigned char)((ih - (oh * d.s - d.p)) * d.k + (iw - (ow * d.s - d.p)));
#pragma unroll
        for (int c = 0; c < V; ++c)
          if (iv[q].v[c] == w) acc[c] += (float)to_acc<T>(gv[q].v[c]);
      }
    } else
    for (int oh = oh_lo; oh <= oh_hi; ++oh)
      for (int ow = ow_lo; ow <= ow_hi; ++ow) {
        const unsigned char w = (unsigned char)((ih - (oh * d.s - d.p)) * d.k + (iw - (ow * d.s - d.p)));
        const size_t o = obase + ((size_t)(oh * d.OW + ow) * cvn + cv) * V;
        Pack<unsigned char, V> iv = ld_pack<unsigned char, V>(idx + o);
        Pack<T, V> gv = ld_pack<T, V>(dy + o);
#pragma unroll
        for (int c = 0; c < V; ++c)
          if (iv.v[c] == w) acc[c] += (float)to_acc<T>(gv.v[c]);
      }
    Pack<T, V> out;
#pragma unroll
    for (int c = 0; c < V; ++c) out.v[c] = from_acc<T>((typename AccOf<T>::type)acc[c]);
    st_pack<T, V>(dx + irow + (size_t)t * V, out);
  }
}

// 3x3 / stride 2 / pad 1: one block per pair of input rows, gathering from the two output rows that
// cover them after staging those in shared memory (each pooled gradient is otherwise fetched from L2
// by every input position of its window, and the kernel is bound by L2 bandwidth).
template <typename T, int V>
__global__ void __launch_bounds__(kBpThreads) maxpool_bwd_rows_kernel(const T* __restrict__ dy, const unsigned char* __restrict__ idx,
                                                                      T* __restrict__ dx, BpDims d) {
  extern __shared__ __align__(16) unsigned char s_raw[];
  const int cvn = d.C / V;
  T* s_dy = reinterpret_cast<T*>(s_raw);
  unsigned char* s_ix = s_raw + (size_t)2 * (d.OW + 1) * d.C * sizeof(T);
  const int hp = (d.H + 1) / 2;
  const int n = blockIdx.x / hp, k = blockIdx.x - n * hp;
  const int cv = threadIdx.x % cvn;                  // kBpThreads is a multiple of cvn
  stage_pool_rows<T, V>(dy, idx, d, n, k, s_dy, s_ix);
  __syncthreads();
  const int rows_here = min(2, d.H - 2 * k);
  const size_t irow = ((size_t)n * d.H + 2 * k) * d.W * d.C;
  for (int t = threadIdx.x; t < rows_here * d.W * cvn; t += kBpThreads) {
    const int pos = t / cvn;
    const int r = pos / d.W, iw = pos - r * d.W;
    float g[V];
    pooled_grad<T, V>(s_dy, s_ix, d, k, 2 * k + r, iw, cv, g);
    Pack<T, V> out;
#pragma unroll
    for (int c = 0; c < V; ++c) out.v[c] = from_acc<T>((typename AccOf<T>::type)g[c]);
    st_pack<T, V>(dx + irow + (size_t)t * V, out);
  }
}

template <typename T>
static int pool_launch(bool fwd, const void* a, void* b, void* idx, PoolDims d, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  if (d.C % V) return fail(TMPI_ERR_INVALID, "maxpool: C=%d must be a multiple of %d", d.C, V);
  if (d.k * d.k > 255) return fail(TMPI_ERR_INVALID, "maxpool: window too large");
  const long long rows = (long long)d.N * (fwd ? d.OH : d.H);
  if (rows < 1 || rows > 0x7fffffffLL) return fail(TMPI_ERR_INVALID, "maxpool: %lld rows", rows);
  int grid = (int)rows;
  const size_t rows_smem = (size_t)2 * (d.OW + 1) * d.C * (sizeof(T) + 1);
  if (!fwd && d.k == 3 && d.s == 2 && d.p == 1 && kBpThreads % (d.C / V) == 0 && rows_smem <= 96 * 1024 &&
      d.OH == (d.H - 1) / 2 + 1 && d.OW == (d.W - 1) / 2 + 1) {
    static bool attr = false;
    if (!attr) { cudaFuncSetAttribute(maxpool_bwd_rows_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); attr = true; }
    BpDims bd{d.N, d.H, d.W, d.C, d.OH, d.OW};
    maxpool_bwd_rows_kernel<T, V><<<d.N * ((d.H + 1) / 2), kBpThreads, rows_smem, s>>>((const T*)a, (const unsigned char*)idx, (T*)b, bd);
  } else if (fwd && d.k == 3) maxpool_fwd_kernel<T, V, true><<<grid, 256, 0, s>>>((const T*)a, (T*)b, (unsigned char*)idx, d);
  else if (fwd) maxpool_fwd_kernel<T, V, false><<<grid, 256, 0, s>>>((const T*)a, (T*)b, (unsigned char*)idx, d);
  else if (d.k <= 2 * d.s) maxpool_bwd_kernel<T, V, true><<<grid, 256, 0, s>>>((const T*)a, (const unsigned char*)idx, (T*)b, d);
  else maxpool_bwd_kernel<T, V, false><<<grid, 256, 0, s>>>((const T*)a, (const unsigned char*)idx, (T*)b, d);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "maxpool launch: %s", cudaGetErrorString(e));
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

// x: [N, H, W, C] channels-last; y, idx: [N, OH, OW, C]
int tmpi_maxpool_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, int OH, int OW, int k, int s,
                     int p, int dtype, void* stream) {
  PoolDims d{N, H, W, C, OH, OW, k, s, p};
  switch (dtype) {
    case TMPI_BF16: return pool_launch<__nv_bfloat16>(true, x, y, idx, d, (cudaStream_t)stream);
    case TMPI_F16: return pool_launch<__half>(true, x, y, idx, d, (cudaStream_t)stream);
    case TMPI_F32: return pool_launch<float>(true, x, y, idx, d, (cudaStream_t)stream);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "maxpool: dtype %d", dtype);
}

int tmpi_maxpool_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int OH, int OW, int k,
                     int s, int p, int dtype, void* stream) {
  PoolDims d{N, H, W, C, OH, OW, k, s, p};
  switch (dtype) {
    case TMPI_BF16: return pool_launch<__nv_bfloat16>(false, dy, dx, const_cast<void*>(idx), d, (cudaStream_t)stream);
    case TMPI_F16: return pool_launch<__half>(false, dy, dx, const_cast<void*>(idx), d, (cudaStream_t)stream);
    case TMPI_F32: return pool_launch<float>(false, dy, dx, const_cast<void*>(idx), d, (cudaStream_t)stream);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "maxpool: dtype %d", dtype);
}

}  // extern "C"
