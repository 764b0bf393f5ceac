// Fused batch-norm (+ residual add) (+ ReLU), forward and backward, for channels-last activations.
//
// The activation is a [rows, C] matrix (rows = N*H*W, C contiguous).  Training forward:
//   stats    : per-channel sum and sum of squares (one read of x)
//   finalize : mean, 1/std, running statistics (32 x 32 threads per 32 channels)
//   apply    : y = relu((x - mean) * invstd * gamma + beta + residual)   (read x [, residual], write y)
// Backward, with dz = dy * (y > 0):
//   reduce   : dbeta = sum dz, dgamma = sum dz * xhat
//   finalize : (same shape)
//   apply    : dx = gamma * invstd * (dz - dbeta/M - xhat * dgamma/M); dresidual = dz
// A framework graph runs batch-norm, add and ReLU as separate kernels with their own reads and
// writes of the activation; the reference has no such ops at all (its only kernel is `out += in`,
// lib/detail/reduce_kernel.cu).  Every thread owns a fixed group of V channels, so partial sums
// stay in registers; block partials go to scratch and are reduced in block order (deterministic).
// A ReLU layer without a residual does not read y in backward: y > 0 exactly when the affine
// transform of x is positive, and x is read anyway.
#include "vec.cuh"
#include "pool_rows.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include <algorithm>

namespace tmpi {

constexpr int kBnThreads = 256;
constexpr int kBnMaxGrid = 592;     // 148 SMs x 4 resident CTAs

static int bn_grid(size_t nvec) {
  size_t want = (nvec + kBnThreads - 1) / kBnThreads;
  return (int)std::max<size_t>(1, std::min<size_t>(want, kBnMaxGrid));
}

// partial[(block * 2 + which) * C + c]
// MASKX (backward only): the ReLU mask comes from x, gamma and beta instead of y.  A template
// parameter, not a run-time flag: the extra scale / shift registers would otherwise cost the other
// path one resident block per SM.
template <typename T, int V, bool BWD, bool MASKX>
__global__ void __launch_bounds__(kBnThreads, 4) bn_reduce_kernel(
    const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy,
    const float* __restrict__ mean, const float* __restrict__ invstd,
    const float* __restrict__ gamma, const float* __restrict__ beta, const unsigned char* __restrict__ bits,
    size_t nvec, int C, int relu, int reverse, float* __restrict__ partial) {
  const int cvn = C / V;
  const size_t T0 = (size_t)blockIdx.x * kBnThreads + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * kBnThreads;
  // reverse: the walk starts at the end of the tensor (vector nvec-1-T0, then down by the stride), where
  // the lines the producer wrote last are still in L2; the apply pass that follows walks up from the
  // start, which this pass read last.  nvec and the stride are multiples of cvn: the group stays fixed.
  const int cv = reverse ? cvn - 1 - (int)(T0 % cvn) : (int)(T0 % cvn);
  const T* xe = x + (nvec - 1) * V;
  const T* ge = BWD ? dy + (nvec - 1) * V : nullptr;
  const T* ye = (BWD && y) ? y + (nvec - 1) * V : nullptr;
  constexpr bool mask_from_x = BWD && MASKX;
  float a[V], b[V], mu[V], is[V], sc[V], sh[V];
#pragma unroll
  for (int k = 0; k < V; ++k) { a[k] = 0.f; b[k] = 0.f; }
  if (BWD) {
#pragma unroll
    for (int k = 0; k < V; ++k) { mu[k] = mean[cv * V + k]; is[k] = invstd[cv * V + k]; }
    if (mask_from_x) {
#pragma unroll
      for (int k = 0; k < V; ++k) { sc[k] = is[k] * gamma[cv * V + k]; sh[k] = beta[cv * V + k] - mu[k] * sc[k]; }
    }
  }
  // U independent vectors per thread and iteration: the loads of all of them are issued before
  // the first use, so a thread keeps U (forward) or up to 3U (backward) 16-byte loads in flight
  constexpr int U = BWD ? 1 : 4;       // backward already has 2-3 loads per vector and no registers to spare
  // bits (backward, ReLU layers with a residual): one byte per vector written by the forward apply
  // pass, bit k set where the output was positive; replaces the read of y
  auto accumulate = [&](const Pack<T, V>& xv, const Pack<T, V>& gv, const Pack<T, V>& yv, unsigned mb = 0) {
    if (!BWD) {
#pragma unroll
      for (int k = 0; k < V; ++k) { float f = (float)to_acc<T>(xv.v[k]); a[k] += f; b[k] += f * f; }
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float g = (float)to_acc<T>(gv.v[k]);
        if (mask_from_x) {
          if (!((float)to_acc<T>(xv.v[k]) * sc[k] + sh[k] > 0.f)) g = 0.f;
        } else if (relu) {
          if (bits ? !((mb >> k) & 1u) : !((float)to_acc<T>(yv.v[k]) > 0.f)) g = 0.f;
        }
        a[k] += g;
        b[k] += g * ((float)to_acc<T>(xv.v[k]) - mu[k]) * is[k];
      }
    }
  };
  size_t v = T0;
  if constexpr (U > 1)
  for (; v + (U - 1) * stride < nvec; v += U * stride) {
    Pack<T, V> xv[U], gv[U], yv[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      xv[u] = ld_pack<T, V>(reverse ? xe - (v + u * stride) * V : x + (v + u * stride) * V);
      if (BWD) {
        gv[u] = ld_pack<T, V>(reverse ? ge - (v + u * stride) * V : dy + (v + u * stride) * V);
        if (relu && !mask_from_x) yv[u] = ld_pack<T, V>(reverse ? ye - (v + u * stride) * V : y + (v + u * stride) * V);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) accumulate(xv[u], gv[u], yv[u]);
  }
  for (; v < nvec; v += stride) {
    Pack<T, V> xv = ld_pack<T, V>(reverse ? xe - v * V : x + v * V), gv, yv;
    unsigned mb = 0;
    if (BWD) {
      gv = ld_pack<T, V>(reverse ? ge - v * V : dy + v * V);
      if (relu && !mask_from_x) {
        if (bits) mb = bits[reverse ? nvec - 1 - v : v];
        else yv = ld_pack<T, V>(reverse ? ye - v * V : y + v * V);
      }
    }
    accumulate(xv, gv, yv, mb);
  }
  __shared__ float s[kBnThreads][2 * V + 1];
#pragma unroll
  for (int k = 0; k < V; ++k) { s[threadIdx.x][k] = a[k]; s[threadIdx.x][V + k] = b[k]; }
  __syncthreads();
  // thread t < cvn * 2V sums one (channel, which) pair over the threads that share its channel group
  for (int o = threadIdx.x; o < cvn * 2 * V; o += kBnThreads) {
    const int c = o / (2 * V), k = o % (2 * V);   // c: channel group, k: slot
    float t = 0.f;
    for (int g = reverse ? cvn - 1 - c : c; g < kBnThreads; g += cvn) t += s[g][k];   // the threads whose group is c
    const int which = k / V, ch = c * V + (k % V);
    partial[((size_t)blockIdx.x * 2 + which) * C + ch] = t;
  }
}

// Sums the per-block partials of 32 channels with a 32 x 32 thread block: thread (cx, ry) adds the
// blocks ry, ry + 32, ... of channel cx (coalesced over cx), then row 0 adds the 32 slices in order.
// All of a thread's loads are issued before the first add (the trip count is bounded by the largest
// grid): a loop of dependent load-add pairs cost one L2 latency per partial, which made this tiny
// kernel as slow as a bandwidth-bound pass.
constexpr int kBnPartialsPerThread = (kBnMaxGrid + 31) / 32;
__device__ __forceinline__ bool bn_partial_sums(const float* __restrict__ partial, int nblocks, int C, float* s1, float* s2) {
  __shared__ float sh1[32][33], sh2[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float va[kBnPartialsPerThread], vb[kBnPartialsPerThread];
#pragma unroll
  for (int j = 0; j < kBnPartialsPerThread; ++j) {
    const int blk = threadIdx.y + 32 * j;
    const bool ok = c < C && blk < nblocks;
    va[j] = ok ? partial[((size_t)blk * 2) * C + c] : 0.f;
    vb[j] = ok ? partial[((size_t)blk * 2 + 1) * C + c] : 0.f;
  }
  float a = 0.f, b = 0.f;
#pragma unroll
  for (int j = 0; j < kBnPartialsPerThread; ++j) { a += va[j]; b += vb[j]; }
  sh1[threadIdx.y][threadIdx.x] = a;
  sh2[threadIdx.y][threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.y != 0 || c >= C) return false;
  a = 0.f; b = 0.f;
#pragma unroll
  for (int r = 0; r < 32; ++r) { a += sh1[r][threadIdx.x]; b += sh2[r][threadIdx.x]; }
  *s1 = a; *s2 = b;
  return true;
}

__global__ void __launch_bounds__(1024) bn_finalize_fwd_kernel(
    const float* __restrict__ partial, int nblocks, int C, float inv_m, float m_corr, float eps, float momentum,
    float* __restrict__ mean, float* __restrict__ invstd, float* __restrict__ rmean, float* __restrict__ rvar) {
  float s1, s2;
  if (!bn_partial_sums(partial, nblocks, C, &s1, &s2)) return;
  const int c = blockIdx.x * 32 + threadIdx.x;
  const float mu = s1 * inv_m;
  float var = s2 * inv_m - mu * mu;
  if (var < 0.f) var = 0.f;
  mean[c] = mu;
  invstd[c] = rsqrtf(var + eps);
  if (rmean) rmean[c] = (1.f - momentum) * rmean[c] + momentum * mu;
  if (rvar) rvar[c] = (1.f - momentum) * rvar[c] + momentum * var * m_corr;   // unbiased, like torch
}

// acc_gamma / acc_beta (nullable): the parameters' gradient buffers, to which the sums are added as well (the
// caller then needs no separate accumulation kernel)
__global__ void __launch_bounds__(1024) bn_finalize_bwd_kernel(const float* __restrict__ partial, int nblocks, int C,
                                                               float* __restrict__ dgamma, float* __restrict__ dbeta,
                                                               float* __restrict__ acc_gamma = nullptr,
                                                               float* __restrict__ acc_beta = nullptr) {
  float s1, s2;
  if (!bn_partial_sums(partial, nblocks, C, &s1, &s2)) return;
  const int c = blockIdx.x * 32 + threadIdx.x;
  dbeta[c] = s1;
  dgamma[c] = s2;
  if (acc_beta) acc_beta[c] += s1;
  if (acc_gamma) acc_gamma[c] += s2;
}

// BITS: also write the ReLU mask byte of every vector (residual layers only; a template parameter so
// that the other layers keep 32 registers and eight resident blocks)
template <typename T, int V, bool BITS>
__global__ void __launch_bounds__(kBnThreads) bn_apply_fwd_kernel(
    const T* __restrict__ x, const T* __restrict__ res, T* __restrict__ y, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ invstd,
    unsigned char* __restrict__ bits, size_t nvec, int C, int relu) {
  const int cvn = C / V;
  const size_t T0 = (size_t)blockIdx.x * kBnThreads + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * kBnThreads;
  const int cv = (int)(T0 % cvn);
  float sc[V], sh[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int c = cv * V + k;
    sc[k] = invstd[c] * gamma[c];
    sh[k] = beta[c] - mean[c] * sc[k];
  }
  for (size_t v = T0; v < nvec; v += stride) {
    Pack<T, V> xv = ld_pack<T, V>(x + v * V), rv, out;
    unsigned mb = 0;
    if (res) rv = ld_pack<T, V>(res + v * V);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float z = (float)to_acc<T>(xv.v[k]) * sc[k] + sh[k];
      if (res) z += (float)to_acc<T>(rv.v[k]);
      if (relu) z = fmaxf(z, 0.f);
      out.v[k] = from_acc<T>((typename AccOf<T>::type)z);
      if (BITS && (float)to_acc<T>(out.v[k]) > 0.f) mb |= 1u << k;     // what `y > 0` would read back
    }
    st_pack<T, V>(y + v * V, out);
    if (BITS) bits[v] = (unsigned char)mb;
  }
}

template <typename T, int V, bool MASKX>
__global__ void __launch_bounds__(kBnThreads, 4) bn_apply_bwd_kernel(
    const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
    T* __restrict__ dres, const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
    const float* __restrict__ invstd, const float* __restrict__ dgamma, const float* __restrict__ dbeta,
    const unsigned char* __restrict__ bits, size_t nvec, int C, int relu, float inv_m) {
  const int cvn = C / V;
  const size_t T0 = (size_t)blockIdx.x * kBnThreads + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * kBnThreads;
  const int cv = (int)(T0 % cvn);
  constexpr bool mask_from_x = MASKX;
  float mu[V], is[V], k1[V], k2[V], k3[V], sh[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int c = cv * V + k;
    mu[k] = mean[c]; is[k] = invstd[c];
    k1[k] = gamma[c] * is[k];            // dx = k1 * (dz - k2 - xhat * k3); also the forward scale
    k2[k] = dbeta[c] * inv_m;
    k3[k] = dgamma[c] * inv_m;
    sh[k] = mask_from_x ? beta[c] - mu[k] * k1[k] : 0.f;
  }
  for (size_t v = T0; v < nvec; v += stride) {
    Pack<T, V> xv = ld_pack<T, V>(x + v * V), gv = ld_pack<T, V>(dy + v * V), yv, ox, orr;
    unsigned mb = 0;
    if (relu && !mask_from_x) {
      if (bits) mb = bits[v];
      else yv = ld_pack<T, V>(y + v * V);
    }
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float g = (float)to_acc<T>(gv.v[k]);
      if (mask_from_x) {
        if (!((float)to_acc<T>(xv.v[k]) * k1[k] + sh[k] > 0.f)) g = 0.f;
      } else if (relu) {
        if (bits ? !((mb >> k) & 1u) : !((float)to_acc<T>(yv.v[k]) > 0.f)) g = 0.f;
      }
      float xhat = ((float)to_acc<T>(xv.v[k]) - mu[k]) * is[k];
      ox.v[k] = from_acc<T>((typename AccOf<T>::type)(k1[k] * (g - k2[k] - xhat * k3[k])));
      orr.v[k] = from_acc<T>((typename AccOf<T>::type)g);
    }
    st_pack<T, V>(dx + v * V, ox);
    if (dres) st_pack<T, V>(dres + v * V, orr);
  }
}

static int bn_check(int64_t rows, int C, int V) {
  if (rows < 1 || C < V || C % V) return fail(TMPI_ERR_INVALID, "bn: C=%d must be a multiple of %d", C, V);
  int cvn = C / V;
  if (kBnThreads % cvn) return fail(TMPI_ERR_UNSUPPORTED, "bn: C/%d = %d must divide %d", V, cvn, kBnThreads);
  return TMPI_OK;
}

template <typename T>
static int bn_fwd_t(const void* x, const void* res, void* y, const float* gamma, const float* beta, float* rmean,
                    float* rvar, float* smean, float* sinv, int64_t rows, int C, float eps, float momentum, int relu,
                    int training, void* bits, void* scratch, cudaStream_t s, int given_rows = 0) {
  constexpr int V = 16 / sizeof(T);
  int st = bn_check(rows, C, V);
  if (st) return st;
  size_t nvec = (size_t)rows * (C / V);
  int grid = bn_grid(nvec);
  const int reverse = tunable("bn_reverse_stats") != 0;
  if (training) {
    // given_rows > 0: the producer of x (a convolution epilogue) has left that many rows of partial sums in scratch
    if (given_rows > 0) grid = given_rows;
    else
    bn_reduce_kernel<T, V, false, false><<<grid, kBnThreads, 0, s>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                                                     nullptr, nvec, C, 0, reverse, (float*)scratch);
    float m = (float)rows;
    bn_finalize_fwd_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)scratch, grid, C, 1.f / m,
                                                           rows > 1 ? m / (m - 1.f) : 1.f, eps, momentum, smean, sinv,
                                                           rmean, rvar);
  }
  // the apply pass keeps no partials and needs 32 registers: eight blocks per SM
  const int apply_grid = (int)std::max<size_t>(1, std::min<size_t>((nvec + kBnThreads - 1) / kBnThreads, 2 * kBnMaxGrid));
  if (bits)
    bn_apply_fwd_kernel<T, V, true><<<apply_grid, kBnThreads, 0, s>>>((const T*)x, (const T*)res, (T*)y, gamma, beta, smean, sinv,
                                                                      (unsigned char*)bits, nvec, C, relu);
  else
    bn_apply_fwd_kernel<T, V, false><<<apply_grid, kBnThreads, 0, s>>>((const T*)x, (const T*)res, (T*)y, gamma, beta, smean, sinv,
                                                                       nullptr, nvec, C, relu);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bn forward launch: %s", cudaGetErrorString(e));
}

template <typename T>
static int bn_bwd_t(const void* x, const void* y, const void* dy, void* dx, void* dres, const float* gamma,
                    const float* beta, const float* smean, const float* sinv, float* dgamma, float* dbeta, int64_t rows, int C, int relu,
                    const void* bits, void* scratch, cudaStream_t s, float* acc_gamma = nullptr, float* acc_beta = nullptr) {
  constexpr int V = 16 / sizeof(T);
  int st = bn_check(rows, C, V);
  if (st) return st;
  if (relu && !y && !bits && (!beta || dres))
    return fail(TMPI_ERR_INVALID, "bn backward: without y or mask bits the layer needs beta and no residual");
  size_t nvec = (size_t)rows * (C / V);
  int grid = bn_grid(nvec);
  const int reverse = tunable("bn_reverse_stats") != 0;
  const bool maskx = relu && !y && !bits;
  const unsigned char* mb = (const unsigned char*)bits;
  if (maskx)
    bn_reduce_kernel<T, V, true, true><<<grid, kBnThreads, 0, s>>>((const T*)x, nullptr, (const T*)dy, smean, sinv, gamma, beta, nullptr,
                                                                   nvec, C, relu, reverse, (float*)scratch);
  else
    bn_reduce_kernel<T, V, true, false><<<grid, kBnThreads, 0, s>>>((const T*)x, (const T*)y, (const T*)dy, smean, sinv, gamma, beta, mb,
                                                                    nvec, C, relu, reverse, (float*)scratch);
  bn_finalize_bwd_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)scratch, grid, C, dgamma, dbeta, acc_gamma, acc_beta);
  if (maskx)
    bn_apply_bwd_kernel<T, V, true><<<grid, kBnThreads, 0, s>>>((const T*)x, nullptr, (const T*)dy, (T*)dx, (T*)dres, gamma, beta,
                                                                smean, sinv, dgamma, dbeta, nullptr, nvec, C, relu, 1.f / (float)rows);
  else
    bn_apply_bwd_kernel<T, V, false><<<grid, kBnThreads, 0, s>>>((const T*)x, (const T*)y, (const T*)dy, (T*)dx, (T*)dres, gamma, beta,
                                                                 smean, sinv, dgamma, dbeta, mb, nvec, C, relu, 1.f / (float)rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bn backward launch: %s", cudaGetErrorString(e));
}

// ------------------------------------------------------------------ batch-norm + ReLU + max-pool
// Batch-norm + ReLU + 3x3 / stride-2 / pad-1 max-pool as one stage (the ResNet stem after its
// convolution), for channels-last activations.  The normalised full-resolution activation is never
// written: forward reads the convolution output once and writes the pooled tensor and a one-byte
// window index; backward rebuilds, per input position, the gradient that the pool routes to it
// (from the pooled gradient and the index, which stay in L2) and the ReLU mask (from x), inside both
// batch-norm backward passes.  Unfused, the same stage writes and re-reads the full-resolution
// activation once forward and its gradient twice backward.
//
//   z = x * scale[c] + shift[c];  a = max(z, 0);  y[oh, ow] = max over the window of a
//   idx = position of the first maximum in the window (kh * 3 + kw), as in pool.cu
//   dz[ih, iw] = (z > 0) * sum over windows (oh, ow) covering (ih, iw) with idx == this position of dy[oh, ow]
//   then the usual batch-norm backward on dz.
static_assert(kBpThreads == kBnThreads, "same partial layout as the kernels above");


// Both directions stage the rows a block needs in shared memory first (coalesced 16-byte loads), then
// gather from there: the 2.25 windows that cover an input position, and the 9 positions of a window,
// would otherwise each be a separate L2 request, and the stage becomes bound by L2 bandwidth.
//
// forward: one block per (n, oh).  The three input rows of the window go to shared memory already
// normalised, rectified and rounded to T, in a row of W + 2 positions whose first and last hold -1
// (below every rectified value), as do rows outside the image: the window scan needs no bounds checks.
template <typename T, int V>
__global__ void __launch_bounds__(kBpThreads) bn_pool_fwd_kernel(
    const T* __restrict__ x, T* __restrict__ y, unsigned char* __restrict__ idx, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ invstd, BpDims d) {
  extern __shared__ __align__(16) unsigned char s_raw[];
  T* s_a = reinterpret_cast<T*>(s_raw);                         // [3][W + 2][C]
  const int cvn = d.C / V;
  const int n = blockIdx.x / d.OH, oh = blockIdx.x % d.OH;
  const int ih0 = oh * 2 - 1;
  const int cv = threadIdx.x % cvn;                             // kBpThreads is a multiple of cvn: fixed channel group
  const int pw = d.W + 2;
  float sc[V], sh[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int c = cv * V + k;
    sc[k] = invstd[c] * gamma[c];
    sh[k] = beta[c] - mean[c] * sc[k];
  }
  Pack<T, V> neg;
#pragma unroll
  for (int k = 0; k < V; ++k) neg.v[k] = from_acc<T>((typename AccOf<T>::type)(-1.f));
  const T* xin = x + (size_t)n * d.H * d.W * d.C;
  constexpr int U = 4;                                          // global loads in flight per thread
  for (int t0 = threadIdx.x; t0 < 3 * pw * cvn; t0 += U * kBpThreads) {
    Pack<T, V> v[U];
    bool in[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u * kBpThreads;
      const int pos = t / cvn;                                  // (row, padded column)
      const int row = pos / pw, col = pos - row * pw;
      const int ih = ih0 + row, iw = col - 1;
      in[u] = t < 3 * pw * cvn && ih >= 0 && ih < d.H && iw >= 0 && iw < d.W;
      if (in[u]) v[u] = ld_pack<T, V>(xin + ((size_t)ih * d.W + iw) * d.C + cv * V);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int t = t0 + u * kBpThreads;
      if (t >= 3 * pw * cvn) break;
      Pack<T, V> o = neg;
      if (in[u]) {
#pragma unroll
        for (int k = 0; k < V; ++k)
          o.v[k] = from_acc<T>((typename AccOf<T>::type)fmaxf((float)to_acc<T>(v[u].v[k]) * sc[k] + sh[k], 0.f));
      }
      st_pack<T, V>(s_a + (size_t)t * V, o);
    }
  }
  __syncthreads();
  const size_t orow = ((size_t)n * d.OH + oh) * d.OW * d.C;
  for (int t = threadIdx.x; t < d.OW * cvn; t += kBpThreads) {
    const int ow = t / cvn;
    float best[V];
    unsigned char bi[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { best[k] = -2.f; bi[k] = 0; }
#pragma unroll
    for (int q = 0; q < 9; ++q) {
      // padded column of iw = 2 ow - 1 + kw is 2 ow + kw
      Pack<T, V> v = ld_pack<T, V>(s_a + ((size_t)((q / 3) * pw + ow * 2 + q % 3) * cvn + cv) * V);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float a = (float)to_acc<T>(v.v[k]);
        if (a > best[k] || a != a) { best[k] = a; bi[k] = (unsigned char)q; }
      }
    }
    Pack<T, V> out;
    Pack<unsigned char, V> oi;
#pragma unroll
    for (int k = 0; k < V; ++k) { out.v[k] = from_acc<T>((typename AccOf<T>::type)best[k]); oi.v[k] = bi[k]; }
    st_pack<T, V>(y + orow + (size_t)t * V, out);
    st_pack<unsigned char, V>(idx + orow + (size_t)t * V, oi);
  }
}

// backward: see pool_rows.cuh for the staging of the pooled rows and the gather.
// copies `items` packs (the block's two input rows of x, contiguous in memory) to shared memory with
// four loads in flight per thread; the statistics and apply loops then run out of shared memory with
// few registers, so that three blocks fit on an SM
template <typename T, int V>
__device__ __forceinline__ void stage_x_rows(const T* __restrict__ src, T* s_x, int items) {
  constexpr int U = 4;
  for (int t0 = threadIdx.x; t0 < items; t0 += U * kBpThreads) {
    Pack<T, V> v[U];
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (t0 + u * kBpThreads < items) v[u] = ld_pack<T, V>(src + (size_t)(t0 + u * kBpThreads) * V);
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (t0 + u * kBpThreads < items) st_pack<T, V>(s_x + (size_t)(t0 + u * kBpThreads) * V, v[u]);
  }
}

// backward statistics: blocks take row pairs (n, k) round-robin; partial sums per block
template <typename T, int V>
__global__ void __launch_bounds__(kBpThreads, 3) bn_pool_bwd_reduce_kernel(
    const T* __restrict__ x, const T* __restrict__ dy, const unsigned char* __restrict__ idx, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ invstd, BpDims d,
    float* __restrict__ partial) {
  extern __shared__ __align__(16) unsigned char s_raw[];
  const int cvn = d.C / V;
  T* s_dy = reinterpret_cast<T*>(s_raw);
  unsigned char* s_ix = s_raw + (size_t)2 * (d.OW + 1) * d.C * sizeof(T);
  T* s_x = reinterpret_cast<T*>(s_raw + (size_t)2 * (d.OW + 1) * d.C * (sizeof(T) + 1));
  const int cv = threadIdx.x % cvn;
  // b accumulates sum(dz * x); the centred form sum(dz * (x - mean)) / std is recovered at the end,
  // which keeps the loop at two constants per channel
  float a[V], b[V], sc[V], sh[V];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int c = cv * V + k;
    a[k] = 0.f; b[k] = 0.f;
    sc[k] = invstd[c] * gamma[c]; sh[k] = beta[c] - mean[c] * sc[k];
  }
  const int hp = (d.H + 1) / 2, pairs = d.N * hp;
  for (int pr = blockIdx.x; pr < pairs; pr += gridDim.x) {
    const int n = pr / hp, k = pr - n * hp;
    __syncthreads();                                            // the previous pair's gathers are done
    const int rows_here = min(2, d.H - 2 * k);
    const int items = rows_here * d.W * cvn;
    stage_pool_rows<T, V>(dy, idx, d, n, k, s_dy, s_ix);
    stage_x_rows<T, V>(x + ((size_t)n * d.H + 2 * k) * d.W * d.C, s_x, items);
    __syncthreads();
#pragma unroll 1
    for (int t = threadIdx.x; t < items; t += kBpThreads) {
      const int pos = t / cvn;
      const int r = pos / d.W, iw = pos - r * d.W;
      Pack<T, V> xv = ld_pack<T, V>(s_x + (size_t)t * V);
      float g[V];
      pooled_grad<T, V>(s_dy, s_ix, d, k, 2 * k + r, iw, cv, g);
#pragma unroll
      for (int c = 0; c < V; ++c) {
        const float xf = (float)to_acc<T>(xv.v[c]);
        const float gz = (xf * sc[c] + sh[c] > 0.f) ? g[c] : 0.f;
        a[c] += gz;
        b[c] += gz * xf;
      }
    }
  }
  __syncthreads();
  __shared__ float s[kBpThreads][2 * V + 1];
#pragma unroll
  for (int k = 0; k < V; ++k) {
    const int c = cv * V + k;
    s[threadIdx.x][k] = a[k];
    s[threadIdx.x][V + k] = (b[k] - mean[c] * a[k]) * invstd[c];
  }
  __syncthreads();
  for (int o = threadIdx.x; o < cvn * 2 * V; o += kBpThreads) {
    const int c = o / (2 * V), k = o % (2 * V);
    float t = 0.f;
    for (int g = c; g < kBpThreads; g += cvn) t += s[g][k];
    const int which = k / V, ch = c * V + (k % V);
    partial[((size_t)blockIdx.x * 2 + which) * d.C + ch] = t;
  }
}

// backward apply: one block per row pair
template <typename T, int V>
__global__ void __launch_bounds__(kBpThreads, 3) bn_pool_bwd_apply_kernel(
    const T* __restrict__ x, const T* __restrict__ dy, const unsigned char* __restrict__ idx, T* __restrict__ dx,
    const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
    const float* __restrict__ invstd, const float* __restrict__ dgamma, const float* __restrict__ dbeta, BpDims d, float inv_m) {
  extern __shared__ __align__(16) unsigned char s_raw[];
  const int cvn = d.C / V;
  T* s_dy = reinterpret_cast<T*>(s_raw);
  unsigned char* s_ix = s_raw + (size_t)2 * (d.OW + 1) * d.C * sizeof(T);
  T* s_x = reinterpret_cast<T*>(s_raw + (size_t)2 * (d.OW + 1) * d.C * (sizeof(T) + 1));
  const int hp = (d.H + 1) / 2;
  const int n = blockIdx.x / hp, k = blockIdx.x - n * hp;
  const int cv = threadIdx.x % cvn;                  // fixed channel group
  // dx = k1 * (dz - dbeta/M - xhat * dgamma/M) with xhat = (x - mean) * invstd, folded to k1 * dz + ca * x + cb
  float k1[V], sh[V], ca[V], cb[V];
#pragma unroll
  for (int c = 0; c < V; ++c) {
    const int ch = cv * V + c;
    const float mu = mean[ch], is = invstd[ch];
    k1[c] = gamma[ch] * is;
    sh[c] = beta[ch] - mu * k1[c];
    ca[c] = -k1[c] * dgamma[ch] * inv_m * is;
    cb[c] = -k1[c] * dbeta[ch] * inv_m - ca[c] * mu;
  }
  const int rows_here = min(2, d.H - 2 * k);
  const size_t irow = ((size_t)n * d.H + 2 * k) * d.W * d.C;
  const int items = rows_here * d.W * cvn;
  stage_pool_rows<T, V>(dy, idx, d, n, k, s_dy, s_ix);
  stage_x_rows<T, V>(x + irow, s_x, items);
  __syncthreads();
#pragma unroll 1
  for (int t = threadIdx.x; t < items; t += kBpThreads) {
    const int pos = t / cvn;
    const int r = pos / d.W, iw = pos - r * d.W;
    Pack<T, V> xv = ld_pack<T, V>(s_x + (size_t)t * V), ox;
    float g[V];
    pooled_grad<T, V>(s_dy, s_ix, d, k, 2 * k + r, iw, cv, g);
#pragma unroll
    for (int c = 0; c < V; ++c) {
      const float xf = (float)to_acc<T>(xv.v[c]);
      const float gz = (xf * k1[c] + sh[c] > 0.f) ? g[c] : 0.f;
      ox.v[c] = from_acc<T>((typename AccOf<T>::type)(k1[c] * gz + ca[c] * xf + cb[c]));
    }
    st_pack<T, V>(dx + irow + (size_t)t * V, ox);
  }
}

// shared memory of the two stages, and the limit under which they are offered
template <typename T> static size_t bn_pool_fwd_smem(const BpDims& d) { return (size_t)3 * (d.W + 2) * d.C * sizeof(T); }
template <typename T> static size_t bn_pool_bwd_smem(const BpDims& d) {
  return (size_t)2 * (d.OW + 1) * d.C * (sizeof(T) + 1) + (size_t)2 * d.W * d.C * sizeof(T);
}
constexpr size_t kBpMaxSmem = 96 * 1024;

template <typename T>
static int bn_pool_fwd_t(const void* x, void* y, void* idx, const float* gamma, const float* beta, float* rmean, float* rvar,
                         float* smean, float* sinv, int N, int H, int W, int C, float eps, float momentum, int training,
                         void* scratch, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const int64_t rows = (int64_t)N * H * W;
  int st = bn_check(rows, C, V);
  if (st) return st;
  BpDims d{N, H, W, C, (H - 1) / 2 + 1, (W - 1) / 2 + 1};
  if (training) {
    size_t nvec = (size_t)rows * (C / V);
    int grid = bn_grid(nvec);
    bn_reduce_kernel<T, V, false, false><<<grid, kBnThreads, 0, s>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                                                     nullptr, nvec, C, 0, tunable("bn_reverse_stats") != 0, (float*)scratch);
    float m = (float)rows;
    bn_finalize_fwd_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)scratch, grid, C, 1.f / m,
                                                           rows > 1 ? m / (m - 1.f) : 1.f, eps, momentum, smean, sinv, rmean, rvar);
  }
  const size_t smem = bn_pool_fwd_smem<T>(d);
  if (smem > kBpMaxSmem) return fail(TMPI_ERR_UNSUPPORTED, "bn+pool: rows of %d x %d do not fit in shared memory", W, C);
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(bn_pool_fwd_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBpMaxSmem); attr = true; }
  bn_pool_fwd_kernel<T, V><<<N * d.OH, kBpThreads, smem, s>>>((const T*)x, (T*)y, (unsigned char*)idx, gamma, beta, smean, sinv, d);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bn+pool forward launch: %s", cudaGetErrorString(e));
}

template <typename T>
static int bn_pool_bwd_t(const void* x, const void* dy, const void* idx, void* dx, const float* gamma, const float* beta,
                         const float* smean, const float* sinv, float* dgamma, float* dbeta, int N, int H, int W, int C,
                         void* scratch, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  const int64_t rows = (int64_t)N * H * W;
  int st = bn_check(rows, C, V);
  if (st) return st;
  BpDims d{N, H, W, C, (H - 1) / 2 + 1, (W - 1) / 2 + 1};
  const int pairs = N * ((H + 1) / 2);
  const int grid = std::min(pairs, kBnMaxGrid);
  const size_t smem = bn_pool_bwd_smem<T>(d);
  if (smem > kBpMaxSmem) return fail(TMPI_ERR_UNSUPPORTED, "bn+pool: rows of %d x %d do not fit in shared memory", W, C);
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(bn_pool_bwd_reduce_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBpMaxSmem);
    cudaFuncSetAttribute(bn_pool_bwd_apply_kernel<T, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBpMaxSmem);
    attr = true;
  }
  bn_pool_bwd_reduce_kernel<T, V><<<grid, kBpThreads, smem, s>>>((const T*)x, (const T*)dy, (const unsigned char*)idx, gamma, beta,
                                                              smean, sinv, d, (float*)scratch);
  bn_finalize_bwd_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)scratch, grid, C, dgamma, dbeta);
  bn_pool_bwd_apply_kernel<T, V><<<pairs, kBpThreads, smem, s>>>((const T*)x, (const T*)dy, (const unsigned char*)idx, (T*)dx, gamma,
                                                              beta, smean, sinv, dgamma, dbeta, d, 1.f / (float)rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bn+pool backward launch: %s", cudaGetErrorString(e));
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

size_t tmpi_bn_scratch_bytes(int channels) { return (size_t)kBnMaxGrid * 2 * channels * sizeof(float); }

// training != 0: batch statistics are computed, saved in save_mean / save_invstd and folded into the
// running statistics.  training == 0: save_mean / save_invstd are inputs (mean and 1/std to apply).
// mask_bits (nullable): one byte per 16-byte vector of y, bit k set where element k is positive; the
// backward of a ReLU layer reads it in place of y.
int tmpi_bn_relu_fwd(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                     float* running_mean, float* running_var, float* save_mean, float* save_invstd, int64_t rows,
                     int channels, float eps, float momentum, int relu, int training, int dtype, void* mask_bits,
                     void* scratch, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bn_fwd_t<__nv_bfloat16>(x, residual, y, gamma, beta, running_mean, running_var, save_mean,
                                                   save_invstd, rows, channels, eps, momentum, relu, training, mask_bits, scratch, s);
    case TMPI_F16: return bn_fwd_t<__half>(x, residual, y, gamma, beta, running_mean, running_var, save_mean, save_invstd,
                                           rows, channels, eps, momentum, relu, training, mask_bits, scratch, s);
    case TMPI_F32: return bn_fwd_t<float>(x, residual, y, gamma, beta, running_mean, running_var, save_mean, save_invstd,
                                          rows, channels, eps, momentum, relu, training, mask_bits, scratch, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bn: dtype %d", dtype);
}

// Training forward whose statistics pass has been done already: `partials` holds `partial_rows` (<= 592) rows of
// per-channel partial sums and sums of squares of x, [row][2][channels] floats, as tmpi_conv_fwd writes them.
int tmpi_bn_relu_fwd_partials(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                              float* running_mean, float* running_var, float* save_mean, float* save_invstd, int64_t rows,
                              int channels, float eps, float momentum, int relu, int dtype, void* mask_bits,
                              void* partials, int partial_rows, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  if (partial_rows < 1 || partial_rows > kBnMaxGrid) return fail(TMPI_ERR_INVALID, "bn: 1..%d rows of partial sums", kBnMaxGrid);
  if (dtype != TMPI_BF16) return fail(TMPI_ERR_UNSUPPORTED, "bn from partial sums: bf16 only");
  return bn_fwd_t<__nv_bfloat16>(x, residual, y, gamma, beta, running_mean, running_var, save_mean, save_invstd, rows, channels,
                                 eps, momentum, relu, 1, mask_bits, partials, s, partial_rows);
}

// The ReLU mask comes from mask_bits when given (see tmpi_bn_relu_fwd), else from y, else - ReLU layers
// without a residual only - it is recomputed from x, gamma and beta.
int tmpi_bn_relu_bwd(const void* x, const void* y, const void* dy, void* dx, void* dresidual, const float* gamma,
                     const float* beta, const float* save_mean, const float* save_invstd, float* dgamma, float* dbeta, int64_t rows,
                     int channels, int relu, int dtype, const void* mask_bits, void* scratch, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bn_bwd_t<__nv_bfloat16>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta,
                                                   rows, channels, relu, mask_bits, scratch, s);
    case TMPI_F16: return bn_bwd_t<__half>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta, rows,
                                           channels, relu, mask_bits, scratch, s);
    case TMPI_F32: return bn_bwd_t<float>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta, rows,
                                          channels, relu, mask_bits, scratch, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bn: dtype %d", dtype);
}

// tmpi_bn_relu_bwd that also adds dgamma / dbeta to acc_gamma / acc_beta (the parameters' gradient buffers; nullable).
int tmpi_bn_relu_bwd_acc(const void* x, const void* y, const void* dy, void* dx, void* dresidual, const float* gamma,
                         const float* beta, const float* save_mean, const float* save_invstd, float* dgamma, float* dbeta,
                         int64_t rows, int channels, int relu, int dtype, const void* mask_bits, void* scratch,
                         float* acc_gamma, float* acc_beta, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bn_bwd_t<__nv_bfloat16>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta,
                                                   rows, channels, relu, mask_bits, scratch, s, acc_gamma, acc_beta);
    case TMPI_F16: return bn_bwd_t<__half>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta, rows,
                                           channels, relu, mask_bits, scratch, s, acc_gamma, acc_beta);
    case TMPI_F32: return bn_bwd_t<float>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta, rows,
                                          channels, relu, mask_bits, scratch, s, acc_gamma, acc_beta);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bn: dtype %d", dtype);
}

// Batch-norm + ReLU + max-pool (3x3, stride 2, pad 1) in one stage.  x: [N, H, W, C] channels-last;
// y, idx: [N, OH, OW, C] with OH = (H - 1) / 2 + 1.  Other arguments as tmpi_bn_relu_fwd / _bwd.
int tmpi_bn_relu_pool_fwd(const void* x, void* y, void* idx, const float* gamma, const float* beta, float* running_mean,
                          float* running_var, float* save_mean, float* save_invstd, int N, int H, int W, int channels,
                          float eps, float momentum, int training, int dtype, void* scratch, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bn_pool_fwd_t<__nv_bfloat16>(x, y, idx, gamma, beta, running_mean, running_var, save_mean, save_invstd,
                                                        N, H, W, channels, eps, momentum, training, scratch, s);
    case TMPI_F16: return bn_pool_fwd_t<__half>(x, y, idx, gamma, beta, running_mean, running_var, save_mean, save_invstd, N, H, W,
                                                channels, eps, momentum, training, scratch, s);
    case TMPI_F32: return bn_pool_fwd_t<float>(x, y, idx, gamma, beta, running_mean, running_var, save_mean, save_invstd, N, H, W,
                                               channels, eps, momentum, training, scratch, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bn+pool: dtype %d", dtype);
}

int tmpi_bn_relu_pool_bwd(const void* x, const void* dy, const void* idx, void* dx, const float* gamma, const float* beta,
                          const float* save_mean, const float* save_invstd, float* dgamma, float* dbeta, int N, int H, int W,
                          int channels, int dtype, void* scratch, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bn_pool_bwd_t<__nv_bfloat16>(x, dy, idx, dx, gamma, beta, save_mean, save_invstd, dgamma, dbeta, N, H, W,
                                                        channels, scratch, s);
    case TMPI_F16: return bn_pool_bwd_t<__half>(x, dy, idx, dx, gamma, beta, save_mean, save_invstd, dgamma, dbeta, N, H, W, channels,
                                                scratch, s);
    case TMPI_F32: return bn_pool_bwd_t<float>(x, dy, idx, dx, gamma, beta, save_mean, save_invstd, dgamma, dbeta, N, H, W, channels,
                                               scratch, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bn+pool: dtype %d", dtype);
}

}  // extern "C"
