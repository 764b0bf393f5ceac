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
    const float* __restrict__ gamma, const float* __restrict__ beta,
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
  auto accumulate = [&](const Pack<T, V>& xv, const Pack<T, V>& gv, const Pack<T, V>& yv) {
    if (!BWD) {
#pragma unroll
      for (int k = 0; k < V; ++k) { float f = (float)to_acc<T>(xv.v[k]); a[k] += f; b[k] += f * f; }
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) {
        float g = (float)to_acc<T>(gv.v[k]);
        if (mask_from_x) {
          if (!((float)to_acc<T>(xv.v[k]) * sc[k] + sh[k] > 0.f)) g = 0.f;
        } else if (relu && !((float)to_acc<T>(yv.v[k]) > 0.f)) g = 0.f;
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
    if (BWD) {
      gv = ld_pack<T, V>(reverse ? ge - v * V : dy + v * V);
      if (relu && !mask_from_x) yv = ld_pack<T, V>(reverse ? ye - v * V : y + v * V);
    }
    accumulate(xv, gv, yv);
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

__global__ void __launch_bounds__(1024) bn_finalize_bwd_kernel(const float* __restrict__ partial, int nblocks, int C,
                                                               float* __restrict__ dgamma, float* __restrict__ dbeta) {
  float s1, s2;
  if (!bn_partial_sums(partial, nblocks, C, &s1, &s2)) return;
  const int c = blockIdx.x * 32 + threadIdx.x;
  dbeta[c] = s1;
  dgamma[c] = s2;
}

template <typename T, int V>
__global__ void __launch_bounds__(kBnThreads) bn_apply_fwd_kernel(
    const T* __restrict__ x, const T* __restrict__ res, T* __restrict__ y, const float* __restrict__ gamma,
    const float* __restrict__ beta, const float* __restrict__ mean, const float* __restrict__ invstd,
    size_t nvec, int C, int relu) {
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
    if (res) rv = ld_pack<T, V>(res + v * V);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float z = (float)to_acc<T>(xv.v[k]) * sc[k] + sh[k];
      if (res) z += (float)to_acc<T>(rv.v[k]);
      if (relu) z = fmaxf(z, 0.f);
      out.v[k] = from_acc<T>((typename AccOf<T>::type)z);
    }
    st_pack<T, V>(y + v * V, out);
  }
}

template <typename T, int V, bool MASKX>
__global__ void __launch_bounds__(kBnThreads, 4) bn_apply_bwd_kernel(
    const T* __restrict__ x, const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
    T* __restrict__ dres, const float* __restrict__ gamma, const float* __restrict__ beta, const float* __restrict__ mean,
    const float* __restrict__ invstd, const float* __restrict__ dgamma, const float* __restrict__ dbeta,
    size_t nvec, int C, int relu, float inv_m) {
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
    if (relu && !mask_from_x) yv = ld_pack<T, V>(y + v * V);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float g = (float)to_acc<T>(gv.v[k]);
      if (mask_from_x) {
        if (!((float)to_acc<T>(xv.v[k]) * k1[k] + sh[k] > 0.f)) g = 0.f;
      } else if (relu && !((float)to_acc<T>(yv.v[k]) > 0.f)) g = 0.f;
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
                    int training, void* scratch, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  int st = bn_check(rows, C, V);
  if (st) return st;
  size_t nvec = (size_t)rows * (C / V);
  int grid = bn_grid(nvec);
  const int reverse = tunable("bn_reverse_stats") != 0;
  if (training) {
    bn_reduce_kernel<T, V, false, false><<<grid, kBnThreads, 0, s>>>((const T*)x, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nvec, C, 0, reverse,
                                                              (float*)scratch);
    float m = (float)rows;
    bn_finalize_fwd_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)scratch, grid, C, 1.f / m,
                                                           rows > 1 ? m / (m - 1.f) : 1.f, eps, momentum, smean, sinv,
                                                           rmean, rvar);
  }
  // the apply pass keeps no partials and needs 32 registers: eight blocks per SM
  const int apply_grid = (int)std::max<size_t>(1, std::min<size_t>((nvec + kBnThreads - 1) / kBnThreads, 2 * kBnMaxGrid));
  bn_apply_fwd_kernel<T, V><<<apply_grid, kBnThreads, 0, s>>>((const T*)x, (const T*)res, (T*)y, gamma, beta, smean, sinv, nvec, C, relu);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bn forward launch: %s", cudaGetErrorString(e));
}

template <typename T>
static int bn_bwd_t(const void* x, const void* y, const void* dy, void* dx, void* dres, const float* gamma,
                    const float* beta, const float* smean, const float* sinv, float* dgamma, float* dbeta, int64_t rows, int C, int relu,
                    void* scratch, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  int st = bn_check(rows, C, V);
  if (st) return st;
  if (relu && !y && (!beta || dres)) return fail(TMPI_ERR_INVALID, "bn backward: without y the layer needs beta and no residual");
  size_t nvec = (size_t)rows * (C / V);
  int grid = bn_grid(nvec);
  const int reverse = tunable("bn_reverse_stats") != 0;
  const bool maskx = relu && !y;
  if (maskx)
    bn_reduce_kernel<T, V, true, true><<<grid, kBnThreads, 0, s>>>((const T*)x, nullptr, (const T*)dy, smean, sinv, gamma, beta, nvec,
                                                                   C, relu, reverse, (float*)scratch);
  else
    bn_reduce_kernel<T, V, true, false><<<grid, kBnThreads, 0, s>>>((const T*)x, (const T*)y, (const T*)dy, smean, sinv, gamma, beta,
                                                                    nvec, C, relu, reverse, (float*)scratch);
  bn_finalize_bwd_kernel<<<(C + 31) / 32, dim3(32, 32), 0, s>>>((const float*)scratch, grid, C, dgamma, dbeta);
  if (maskx)
    bn_apply_bwd_kernel<T, V, true><<<grid, kBnThreads, 0, s>>>((const T*)x, nullptr, (const T*)dy, (T*)dx, (T*)dres, gamma, beta,
                                                                smean, sinv, dgamma, dbeta, nvec, C, relu, 1.f / (float)rows);
  else
    bn_apply_bwd_kernel<T, V, false><<<grid, kBnThreads, 0, s>>>((const T*)x, (const T*)y, (const T*)dy, (T*)dx, (T*)dres, gamma, beta,
                                                                 smean, sinv, dgamma, dbeta, nvec, C, relu, 1.f / (float)rows);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bn backward launch: %s", cudaGetErrorString(e));
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

size_t tmpi_bn_scratch_bytes(int channels) { return (size_t)kBnMaxGrid * 2 * channels * sizeof(float); }

// training != 0: batch statistics are computed, saved in save_mean / save_invstd and folded into the
// running statistics.  training == 0: save_mean / save_invstd are inputs (mean and 1/std to apply).
int tmpi_bn_relu_fwd(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                     float* running_mean, float* running_var, float* save_mean, float* save_invstd, int64_t rows,
                     int channels, float eps, float momentum, int relu, int training, int dtype, void* scratch,
                     void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bn_fwd_t<__nv_bfloat16>(x, residual, y, gamma, beta, running_mean, running_var, save_mean,
                                                   save_invstd, rows, channels, eps, momentum, relu, training, scratch, s);
    case TMPI_F16: return bn_fwd_t<__half>(x, residual, y, gamma, beta, running_mean, running_var, save_mean, save_invstd,
                                           rows, channels, eps, momentum, relu, training, scratch, s);
    case TMPI_F32: return bn_fwd_t<float>(x, residual, y, gamma, beta, running_mean, running_var, save_mean, save_invstd,
                                          rows, channels, eps, momentum, relu, training, scratch, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bn: dtype %d", dtype);
}

// y == nullptr (ReLU layers without a residual only): the ReLU mask is recomputed from x, gamma and beta.
int tmpi_bn_relu_bwd(const void* x, const void* y, const void* dy, void* dx, void* dresidual, const float* gamma,
                     const float* beta, const float* save_mean, const float* save_invstd, float* dgamma, float* dbeta, int64_t rows,
                     int channels, int relu, int dtype, void* scratch, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bn_bwd_t<__nv_bfloat16>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta,
                                                   rows, channels, relu, scratch, s);
    case TMPI_F16: return bn_bwd_t<__half>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta, rows,
                                           channels, relu, scratch, s);
    case TMPI_F32: return bn_bwd_t<float>(x, y, dy, dx, dresidual, gamma, beta, save_mean, save_invstd, dgamma, dbeta, rows,
                                          channels, relu, scratch, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bn: dtype %d", dtype);
}

}  // extern "C"
