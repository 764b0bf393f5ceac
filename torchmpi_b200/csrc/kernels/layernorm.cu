// Layer normalisation over the last dimension, forward and backward, for [rows, C] activations.
//
// One warp per row: a lane owns C / 32 elements (packs of 16 bytes, strided by the warp so that the
// warp's loads are contiguous), the row statistics are two warp reductions, and the row is read once.
// Backward computes dx and, in the same pass, the lane's share of dgamma and dbeta in registers over
// all the rows its warp visits; the block's warps are summed through shared memory into one partial
// per block and a second kernel adds the partials in block order (deterministic).  A framework
// graph runs this as three kernels with three reads of dy and x (dx, then the two parameter
// reductions).  The reference has no normalisation layer of its own (it trains Torch7 modules).
#include "vec.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include <algorithm>

namespace tmpi {

constexpr int kLnThreads = 256, kLnWarps = kLnThreads / 32;
constexpr int kLnMaxGrid = 296;           // forward: two blocks per SM; backward (about 200 registers): half of it, one per SM

// NP = packs per lane (C = 32 * NP * V)
template <typename T, int V, int NP>
__global__ void __launch_bounds__(kLnThreads) ln_fwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma,
                                                            const T* __restrict__ beta, T* __restrict__ y,
                                                            float* __restrict__ mean, float* __restrict__ rstd, int rows, float eps) {
  constexpr int C = 32 * NP * V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float g[NP][V], b[NP][V];
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    Pack<T, V> gv = ld_pack<T, V>(gamma + (p * 32 + lane) * V), bv = ld_pack<T, V>(beta + (p * 32 + lane) * V);
#pragma unroll
    for (int k = 0; k < V; ++k) { g[p][k] = (float)to_acc<T>(gv.v[k]); b[p][k] = (float)to_acc<T>(bv.v[k]); }
  }
  for (int r = blockIdx.x * kLnWarps + warp; r < rows; r += gridDim.x * kLnWarps) {
    const T* xr = x + (size_t)r * C;
    Pack<T, V> xv[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) xv[p] = ld_pack<T, V>(xr + (p * 32 + lane) * V);
    float s = 0.f;
#pragma unroll
    for (int p = 0; p < NP; ++p)
#pragma unroll
      for (int k = 0; k < V; ++k) s += (float)to_acc<T>(xv[p].v[k]);
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(~0u, s, o);
    const float mu = s * (1.f / C);
    float q = 0.f;
#pragma unroll
    for (int p = 0; p < NP; ++p)
#pragma unroll
      for (int k = 0; k < V; ++k) { const float d = (float)to_acc<T>(xv[p].v[k]) - mu; q += d * d; }
    for (int o = 16; o; o >>= 1) q += __shfl_xor_sync(~0u, q, o);
    const float rs = rsqrtf(q * (1.f / C) + eps);
    if (lane == 0) { mean[r] = mu; rstd[r] = rs; }
    T* yr = y + (size_t)r * C;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      Pack<T, V> o;
#pragma unroll
      for (int k = 0; k < V; ++k)
        o.v[k] = from_acc<T>((typename AccOf<T>::type)(((float)to_acc<T>(xv[p].v[k]) - mu) * rs * g[p][k] + b[p][k]));
      st_pack<T, V>(yr + (p * 32 + lane) * V, o);
    }
  }
}

// partial[(block * 2 + which) * C + c], which: 0 = dbeta, 1 = dgamma
template <typename T, int V, int NP>
__global__ void __launch_bounds__(kLnThreads) ln_bwd_kernel(const T* __restrict__ x, const T* __restrict__ dy,
                                                            const T* __restrict__ gamma, const float* __restrict__ mean,
                                                            const float* __restrict__ rstd, T* __restrict__ dx,
                                                            float* __restrict__ partial, int rows) {
  constexpr int C = 32 * NP * V;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float g[NP][V], db[NP][V], dg[NP][V];
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    Pack<T, V> gv = ld_pack<T, V>(gamma + (p * 32 + lane) * V);
#pragma unroll
    for (int k = 0; k < V; ++k) { g[p][k] = (float)to_acc<T>(gv.v[k]); db[p][k] = 0.f; dg[p][k] = 0.f; }
  }
  for (int r = blockIdx.x * kLnWarps + warp; r < rows; r += gridDim.x * kLnWarps) {
    const T* xr = x + (size_t)r * C;
    const T* gr = dy + (size_t)r * C;
    Pack<T, V> xv[NP], yv[NP];
#pragma unroll
    for (int p = 0; p < NP; ++p) { xv[p] = ld_pack<T, V>(xr + (p * 32 + lane) * V); yv[p] = ld_pack<T, V>(gr + (p * 32 + lane) * V); }
    const float mu = mean[r], rs = rstd[r];
    float s1 = 0.f, s2 = 0.f;               // sum(dy * gamma), sum(dy * gamma * xhat)
#pragma unroll
    for (int p = 0; p < NP; ++p)
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float d = (float)to_acc<T>(yv[p].v[k]);
        const float xh = ((float)to_acc<T>(xv[p].v[k]) - mu) * rs;
        db[p][k] += d;
        dg[p][k] += d * xh;
        s1 += d * g[p][k];
        s2 += d * g[p][k] * xh;
      }
    for (int o = 16; o; o >>= 1) { s1 += __shfl_xor_sync(~0u, s1, o); s2 += __shfl_xor_sync(~0u, s2, o); }
    s1 *= 1.f / C; s2 *= 1.f / C;
    T* dr = dx + (size_t)r * C;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      Pack<T, V> o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float d = (float)to_acc<T>(yv[p].v[k]);
        const float xh = ((float)to_acc<T>(xv[p].v[k]) - mu) * rs;
        o.v[k] = from_acc<T>((typename AccOf<T>::type)(rs * (d * g[p][k] - s1 - xh * s2)));
      }
      st_pack<T, V>(dr + (p * 32 + lane) * V, o);
    }
  }
  // the block's eight warps hold the same columns: they add into shared memory one after the other
  // (warp order, so the sum is reproducible)
  __shared__ float s[2][32 * NP * V];
  for (int w = 0; w < kLnWarps; ++w) {
    if (warp == w) {
#pragma unroll
      for (int p = 0; p < NP; ++p)
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const int c = (p * 32 + lane) * V + k;
          s[0][c] = (w ? s[0][c] : 0.f) + db[p][k];
          s[1][c] = (w ? s[1][c] : 0.f) + dg[p][k];
        }
    }
    __syncthreads();
  }
  for (int o = threadIdx.x; o < 2 * C; o += kLnThreads) {
    const int which = o / C, c = o - which * C;
    partial[((size_t)blockIdx.x * 2 + which) * C + c] = s[which][c];
  }
}

template <typename T>
__global__ void __launch_bounds__(256) ln_finalize_kernel(const float* __restrict__ partial, int nblocks, int C,
                                                          T* __restrict__ dgamma, T* __restrict__ dbeta) {
  const int o = blockIdx.x * blockDim.x + threadIdx.x;      // (which, c)
  if (o >= 2 * C) return;
  const int which = o / C, c = o - which * C;
  float t = 0.f;
  int blk = 0;
  for (; blk + 4 <= nblocks; blk += 4) {                     // four loads in flight, added in block order
    const float a0 = partial[((size_t)blk * 2 + which) * C + c], a1 = partial[((size_t)(blk + 1) * 2 + which) * C + c];
    const float a2 = partial[((size_t)(blk + 2) * 2 + which) * C + c], a3 = partial[((size_t)(blk + 3) * 2 + which) * C + c];
    t += a0; t += a1; t += a2; t += a3;
  }
  for (; blk < nblocks; ++blk) t += partial[((size_t)blk * 2 + which) * C + c];
  (which ? dgamma : dbeta)[c] = from_acc<T>((typename AccOf<T>::type)t);
}

static int ln_grid(int rows) { return std::max(1, std::min((rows + kLnWarps - 1) / kLnWarps, kLnMaxGrid)); }

template <typename T, int NP>
static cudaError_t ln_launch(bool fwd, const void* x, const void* a, const void* gamma, const void* beta, void* out, float* mean,
                             float* rstd, float* partial, void* dgamma, void* dbeta, int rows, float eps, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  constexpr int C = 32 * NP * V;
  const int grid = fwd ? ln_grid(rows) : std::min(ln_grid(rows), kLnMaxGrid / 2);
  if (fwd) {
    ln_fwd_kernel<T, V, NP><<<grid, kLnThreads, 0, s>>>((const T*)x, (const T*)gamma, (const T*)beta, (T*)out, mean, rstd, rows, eps);
  } else {
    ln_bwd_kernel<T, V, NP><<<grid, kLnThreads, 0, s>>>((const T*)x, (const T*)a, (const T*)gamma, mean, rstd, (T*)out, partial, rows);
    ln_finalize_kernel<T><<<(2 * C + 255) / 256, 256, 0, s>>>(partial, grid, C, (T*)dgamma, (T*)dbeta);
  }
  return cudaGetLastError();
}

template <typename T>
static int ln_dispatch(bool fwd, const void* x, const void* a, const void* gamma, const void* beta, void* out, float* mean,
                       float* rstd, float* partial, void* dgamma, void* dbeta, int rows, int C, float eps, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  if (rows < 1 || C % (32 * V)) return fail(TMPI_ERR_UNSUPPORTED, "layernorm: C=%d must be a multiple of %d", C, 32 * V);
  cudaError_t e;
  switch (C / (32 * V)) {
    case 1: e = ln_launch<T, 1>(fwd, x, a, gamma, beta, out, mean, rstd, partial, dgamma, dbeta, rows, eps, s); break;
    case 2: e = ln_launch<T, 2>(fwd, x, a, gamma, beta, out, mean, rstd, partial, dgamma, dbeta, rows, eps, s); break;
    case 3: e = ln_launch<T, 3>(fwd, x, a, gamma, beta, out, mean, rstd, partial, dgamma, dbeta, rows, eps, s); break;
    case 4: e = ln_launch<T, 4>(fwd, x, a, gamma, beta, out, mean, rstd, partial, dgamma, dbeta, rows, eps, s); break;
    case 5: e = ln_launch<T, 5>(fwd, x, a, gamma, beta, out, mean, rstd, partial, dgamma, dbeta, rows, eps, s); break;
    case 6: e = ln_launch<T, 6>(fwd, x, a, gamma, beta, out, mean, rstd, partial, dgamma, dbeta, rows, eps, s); break;
    case 8: e = ln_launch<T, 8>(fwd, x, a, gamma, beta, out, mean, rstd, partial, dgamma, dbeta, rows, eps, s); break;
    default: return fail(TMPI_ERR_UNSUPPORTED, "layernorm: C=%d is not covered (%d elements per lane)", C, C / 32);
  }
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "layernorm launch: %s", cudaGetErrorString(e));
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

// 1 if tmpi_layernorm_* cover this width and type
int tmpi_layernorm_supported(int channels, int dtype) {
  const int V = dtype == TMPI_F32 ? 4 : 8;
  if (dtype != TMPI_F32 && dtype != TMPI_BF16 && dtype != TMPI_F16) return 0;
  if (channels % (32 * V)) return 0;
  const int np = channels / (32 * V);
  return np >= 1 && np <= 8 && np != 7;
}

size_t tmpi_layernorm_scratch_bytes(int channels) { return (size_t)kLnMaxGrid * 2 * channels * sizeof(float); }

// y = (x - mean) * rstd * gamma + beta per row; mean / rstd ([rows], fp32) are kept for backward.
// gamma, beta, x, y share the dtype.
int tmpi_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int rows,
                       int channels, float eps, int dtype, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return ln_dispatch<__nv_bfloat16>(true, x, nullptr, gamma, beta, y, mean, rstd, nullptr, nullptr, nullptr, rows, channels, eps, s);
    case TMPI_F16: return ln_dispatch<__half>(true, x, nullptr, gamma, beta, y, mean, rstd, nullptr, nullptr, nullptr, rows, channels, eps, s);
    case TMPI_F32: return ln_dispatch<float>(true, x, nullptr, gamma, beta, y, mean, rstd, nullptr, nullptr, nullptr, rows, channels, eps, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "layernorm: dtype %d", dtype);
}

// dx, dgamma, dbeta from dy in one pass over (x, dy); scratch: tmpi_layernorm_scratch_bytes(channels).
int tmpi_layernorm_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd, void* dx,
                       void* dgamma, void* dbeta, int rows, int channels, int dtype, void* scratch, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  float* m = const_cast<float*>(mean);
  float* r = const_cast<float*>(rstd);
  switch (dtype) {
    case TMPI_BF16: return ln_dispatch<__nv_bfloat16>(false, x, dy, gamma, nullptr, dx, m, r, (float*)scratch, dgamma, dbeta, rows, channels, 0.f, s);
    case TMPI_F16: return ln_dispatch<__half>(false, x, dy, gamma, nullptr, dx, m, r, (float*)scratch, dgamma, dbeta, rows, channels, 0.f, s);
    case TMPI_F32: return ln_dispatch<float>(false, x, dy, gamma, nullptr, dx, m, r, (float*)scratch, dgamma, dbeta, rows, channels, 0.f, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "layernorm: dtype %d", dtype);
}

}  // extern "C"
