// Bias gradient of a linear layer, optionally fused with the GELU backward that precedes it:
//   dz = dy * gelu'(z)   (written; skipped when z == nullptr, then dz = dy)
//   db[c] = sum over rows of dz[r, c]
// One pass over dy (and z): a framework graph runs the GELU backward and the column sum as two
// kernels, the second re-reading dz.  Columns are processed in slabs of 1024 (128 threads x one
// 16-byte pack), two rows at a time per block; every thread keeps its eight column sums in
// registers, blocks write partials and a second kernel adds them in block order (deterministic).
// The GELU forward with the same approximation of the normal distribution lives here too.
#include "vec.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include <algorithm>

namespace tmpi {

constexpr int kBgThreads = 256, kBgCols = 128;      // 128 column groups x 2 rows per block
constexpr int kBgMaxRowBlocks = 4 * 148;            // partial rows the scratch buffer holds
constexpr int kBgFinCols = 32, kBgFinGroups = 32;   // finalize: 32 columns x 32 groups of partial rows per block

// gelu(z) = z * Phi(z);  d/dz [z * Phi(z)] = Phi(z) + z * phi(z).  Phi through the rational erf approximation of Abramowitz and
// Stegun 7.1.26 (absolute error 1.5e-7), which shares its exp(-z^2 / 2) with phi: one ex2, one rcp and a
// dozen FMAs per element keep the kernel memory bound where erff() made it ALU bound.
__device__ __forceinline__ void normal_parts(float z, float* cdf, float* e) {
  *e = __expf(-0.5f * z * z);
  const float t = __fdividef(1.f, fmaf(0.3275911f * 0.70710678118654752f, fabsf(z), 1.f));
  float poly = fmaf(1.061405429f, t, -1.453152027f);
  poly = fmaf(poly, t, 1.421413741f);
  poly = fmaf(poly, t, -0.284496736f);
  poly = fmaf(poly, t, 0.254829592f);
  const float q = 0.5f * poly * t * *e;                 // 1 - Phi(|z|)
  *cdf = z >= 0.f ? 1.f - q : q;
}

__device__ __forceinline__ float gelu_grad(float z) {
  float cdf, e;
  normal_parts(z, &cdf, &e);
  return fmaf(z * 0.3989422804014327f, e, cdf);
}

__device__ __forceinline__ float gelu_value(float z) {
  float cdf, e;
  normal_parts(z, &cdf, &e);
  return z * cdf;
}

// y = gelu(z), one 16-byte pack per thread and step, four steps in flight.
template <typename T, int V>
__global__ void __launch_bounds__(256) gelu_fwd_kernel(const T* __restrict__ z, T* __restrict__ y, size_t npacks) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  constexpr int U = 4;
  for (; i + (U - 1) * stride < npacks; i += U * stride) {
    Pack<T, V> a[U];
#pragma unroll
    for (int u = 0; u < U; ++u) a[u] = ld_pack<T, V>(z + (i + u * stride) * V);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      Pack<T, V> o;
#pragma unroll
      for (int k = 0; k < V; ++k) o.v[k] = from_acc<T>((typename AccOf<T>::type)gelu_value((float)to_acc<T>(a[u].v[k])));
      st_pack<T, V>(y + (i + u * stride) * V, o);
    }
  }
  for (; i < npacks; i += stride) {
    Pack<T, V> a = ld_pack<T, V>(z + i * V), o;
#pragma unroll
    for (int k = 0; k < V; ++k) o.v[k] = from_acc<T>((typename AccOf<T>::type)gelu_value((float)to_acc<T>(a.v[k])));
    st_pack<T, V>(y + i * V, o);
  }
}

template <typename T>
static int gelu_fwd_t(const void* z, void* y, size_t n, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  if (n % V || ((uintptr_t)z & 15) || ((uintptr_t)y & 15))
    return fail(TMPI_ERR_UNSUPPORTED, "gelu_fwd: n=%zu must be a multiple of %d and the pointers 16-byte aligned", n, V);
  const size_t npacks = n / V;
  if (!npacks) return TMPI_OK;
  const int blocks = (int)std::min<size_t>((npacks + 255) / 256, (size_t)148 * 8);
  gelu_fwd_kernel<T, V><<<blocks, 256, 0, s>>>((const T*)z, (T*)y, npacks);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "gelu_fwd launch: %s", cudaGetErrorString(e));
}

// partial[blockIdx.y * C + c]
template <typename T, int V, bool GELU>
__global__ void __launch_bounds__(kBgThreads, 4)
bias_grad_kernel(const T* __restrict__ dy, const T* __restrict__ z, T* __restrict__ dz, float* __restrict__ partial,
                 int rows, int C) {
  const int tx = threadIdx.x % kBgCols, ty = threadIdx.x / kBgCols;
  const int col = (blockIdx.x * kBgCols + tx) * V;
  float acc[V];
#pragma unroll
  for (int k = 0; k < V; ++k) acc[k] = 0.f;
  constexpr int U = GELU ? 2 : 4;                       // rows in flight per thread (63 registers either way)
  const int step = 2 * gridDim.y;
  auto one = [&](const Pack<T, V>& g, const Pack<T, V>& a, size_t at) {
    if (GELU) {
      Pack<T, V> o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float v = (float)to_acc<T>(g.v[k]) * gelu_grad((float)to_acc<T>(a.v[k]));
        o.v[k] = from_acc<T>((typename AccOf<T>::type)v);
        acc[k] += (float)to_acc<T>(o.v[k]);             // the sum of what is stored
      }
      st_pack<T, V>(dz + at, o);
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] += (float)to_acc<T>(g.v[k]);
    }
  };
  int r = blockIdx.y * 2 + ty;
  for (; r + (U - 1) * step < rows; r += U * step) {
    Pack<T, V> g[U], a[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const size_t at = (size_t)(r + u * step) * C + col;
      g[u] = ld_pack<T, V>(dy + at);
      if (GELU) a[u] = ld_pack<T, V>(z + at);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) one(g[u], a[u], (size_t)(r + u * step) * C + col);
  }
  for (; r < rows; r += step) {
    const size_t at = (size_t)r * C + col;
    Pack<T, V> g = ld_pack<T, V>(dy + at), a;
    if (GELU) a = ld_pack<T, V>(z + at);
    one(g, a, at);
  }
  __shared__ float s[kBgCols][V + 1];
  if (ty == 1) {
#pragma unroll
    for (int k = 0; k < V; ++k) s[tx][k] = acc[k];
  }
  __syncthreads();
  if (ty == 0) {
#pragma unroll
    for (int k = 0; k < V; ++k) partial[(size_t)blockIdx.y * C + col + k] = acc[k] + s[tx][k];
  }
}

// One block per 32 columns; 32 warps each add a contiguous range of the partial rows, then warp 0 adds
// the 32 sums in order: the result does not depend on the launch.
template <typename T>
__global__ void __launch_bounds__(kBgFinCols * kBgFinGroups)
bias_grad_finalize_kernel(const float* __restrict__ partial, int nblocks, int C, T* __restrict__ db) {
  const int cx = threadIdx.x % kBgFinCols, grp = threadIdx.x / kBgFinCols;
  const int c = blockIdx.x * kBgFinCols + cx;            // C is a multiple of 32
  const int per = (nblocks + kBgFinGroups - 1) / kBgFinGroups;
  int b = grp * per;
  const int end = min(nblocks, b + per);
  float t = 0.f;
  for (; b + 8 <= end; b += 8) {                        // eight loads in flight, added in row order
    float a[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) a[u] = partial[(size_t)(b + u) * C + c];
#pragma unroll
    for (int u = 0; u < 8; ++u) t += a[u];
  }
  for (; b < end; ++b) t += partial[(size_t)b * C + c];
  __shared__ float s[kBgFinGroups][kBgFinCols];
  s[grp][cx] = t;
  __syncthreads();
  if (grp == 0) {
    float sum = s[0][cx];
#pragma unroll
    for (int g = 1; g < kBgFinGroups; ++g) sum += s[g][cx];
    db[c] = from_acc<T>((typename AccOf<T>::type)sum);
  }
}

template <typename T>
static int bias_grad_t(const void* dy, const void* z, void* dz, void* db, int rows, int C, void* scratch, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  if (rows < 1 || C % (kBgCols * V)) return fail(TMPI_ERR_UNSUPPORTED, "bias_grad: C=%d must be a multiple of %d", C, kBgCols * V);
  if (z && !dz) return fail(TMPI_ERR_INVALID, "bias_grad: z given without an output for dz");
  const int slabs = C / (kBgCols * V);
  const int per_sm = 4;                                  // resident blocks per SM
  const int rb = std::max(1, std::min((rows + 1) / 2, std::max(1, per_sm * 148 / slabs)));
  const dim3 grid(slabs, rb);
  if (z) bias_grad_kernel<T, V, true><<<grid, kBgThreads, 0, s>>>((const T*)dy, (const T*)z, (T*)dz, (float*)scratch, rows, C);
  else bias_grad_kernel<T, V, false><<<grid, kBgThreads, 0, s>>>((const T*)dy, nullptr, nullptr, (float*)scratch, rows, C);
  bias_grad_finalize_kernel<T><<<C / kBgFinCols, kBgFinCols * kBgFinGroups, 0, s>>>((const float*)scratch, rb, C, (T*)db);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bias_grad launch: %s", cudaGetErrorString(e));
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

size_t tmpi_bias_grad_scratch_bytes(int channels) { return (size_t)kBgMaxRowBlocks * channels * sizeof(float); }

// db[c] = sum_r dz[r, c] with dz = dy * gelu'(z) written to `dz` when z is given, else dz = dy (nothing written).
// dy, z, dz: [rows, channels]; db: [channels]; all of `dtype`.
int tmpi_bias_grad(const void* dy, const void* z, void* dz, void* db, int rows, int channels, int dtype, void* scratch,
                   void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return bias_grad_t<__nv_bfloat16>(dy, z, dz, db, rows, channels, scratch, s);
    case TMPI_F16: return bias_grad_t<__half>(dy, z, dz, db, rows, channels, scratch, s);
    case TMPI_F32: return bias_grad_t<float>(dy, z, dz, db, rows, channels, scratch, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "bias_grad: dtype %d", dtype);
}

// y = gelu(z) (erf form) for n elements of `dtype`; the forward companion of tmpi_bias_grad's derivative.
int tmpi_gelu_fwd(const void* z, void* y, size_t n, int dtype, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_BF16: return gelu_fwd_t<__nv_bfloat16>(z, y, n, s);
    case TMPI_F16: return gelu_fwd_t<__half>(z, y, n, s);
    case TMPI_F32: return gelu_fwd_t<float>(z, y, n, s);
  }
  return fail(TMPI_ERR_UNSUPPORTED, "gelu_fwd: dtype %d", dtype);
}

}  // extern "C"
