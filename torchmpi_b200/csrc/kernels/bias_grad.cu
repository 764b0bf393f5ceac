// Bias gradient of a linear layer, optionally fused with the GELU backward that precedes it:
//   dz = dy * gelu'(z)   (written; skipped when z == nullptr, then dz = dy)
//   db[c] = sum over rows of dz[r, c]
// One pass over dy (and z): a framework graph runs the GELU backward and the column sum as two
// kernels, the second re-reading dz.  Columns are processed in slabs of 1024 (128 threads x one
// 16-byte pack), two rows at a time per block; every thread keeps its eight column sums in
// registers, blocks write partials and a second kernel adds them in block order (deterministic).
#include "vec.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include <algorithm>

namespace tmpi {

constexpr int kBgThreads = 256, kBgCols = 128;      // 128 column groups x 2 rows per block
constexpr int kBgMaxRowBlocks = 148;

__device__ __forceinline__ float gelu_grad(float z) {
  const float cdf = 0.5f * (1.f + erff(z * 0.70710678118654752f));
  const float pdf = 0.3989422804014327f * __expf(-0.5f * z * z);
  return cdf + z * pdf;
}

// partial[blockIdx.y * C + c]
template <typename T, int V>
__global__ void __launch_bounds__(kBgThreads) bias_grad_kernel(const T* __restrict__ dy, const T* __restrict__ z, T* __restrict__ dz,
                                                               float* __restrict__ partial, int rows, int C) {
  const int tx = threadIdx.x % kBgCols, ty = threadIdx.x / kBgCols;
  const int col = (blockIdx.x * kBgCols + tx) * V;
  float acc[V];
#pragma unroll
  for (int k = 0; k < V; ++k) acc[k] = 0.f;
  constexpr int U = 4;                                  // rows in flight per thread
  const int step = 2 * gridDim.y;
  int r = blockIdx.y * 2 + ty;
  for (; r + (U - 1) * step < rows; r += U * step) {
    Pack<T, V> g[U], a[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      g[u] = ld_pack<T, V>(dy + (size_t)(r + u * step) * C + col);
      if (z) a[u] = ld_pack<T, V>(z + (size_t)(r + u * step) * C + col);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (z) {
        Pack<T, V> o;
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const float v = (float)to_acc<T>(g[u].v[k]) * gelu_grad((float)to_acc<T>(a[u].v[k]));
          o.v[k] = from_acc<T>((typename AccOf<T>::type)v);
          acc[k] += (float)to_acc<T>(o.v[k]);           // the sum of what is stored
        }
        st_pack<T, V>(dz + (size_t)(r + u * step) * C + col, o);
      } else {
#pragma unroll
        for (int k = 0; k < V; ++k) acc[k] += (float)to_acc<T>(g[u].v[k]);
      }
    }
  }
  for (; r < rows; r += step) {
    Pack<T, V> g = ld_pack<T, V>(dy + (size_t)r * C + col);
    if (z) {
      Pack<T, V> a = ld_pack<T, V>(z + (size_t)r * C + col), o;
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float v = (float)to_acc<T>(g.v[k]) * gelu_grad((float)to_acc<T>(a.v[k]));
        o.v[k] = from_acc<T>((typename AccOf<T>::type)v);
        acc[k] += (float)to_acc<T>(o.v[k]);
      }
      st_pack<T, V>(dz + (size_t)r * C + col, o);
    } else {
#pragma unroll
      for (int k = 0; k < V; ++k) acc[k] += (float)to_acc<T>(g.v[k]);
    }
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

template <typename T>
__global__ void __launch_bounds__(256) bias_grad_finalize_kernel(const float* __restrict__ partial, int nblocks, int C,
                                                                 T* __restrict__ db) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float t = 0.f;
  int b = 0;
  for (; b + 4 <= nblocks; b += 4) {                    // four loads in flight, added in block order
    const float a0 = partial[(size_t)b * C + c], a1 = partial[(size_t)(b + 1) * C + c];
    const float a2 = partial[(size_t)(b + 2) * C + c], a3 = partial[(size_t)(b + 3) * C + c];
    t += a0; t += a1; t += a2; t += a3;
  }
  for (; b < nblocks; ++b) t += partial[(size_t)b * C + c];
  db[c] = from_acc<T>((typename AccOf<T>::type)t);
}

template <typename T>
static int bias_grad_t(const void* dy, const void* z, void* dz, void* db, int rows, int C, void* scratch, cudaStream_t s) {
  constexpr int V = 16 / sizeof(T);
  if (rows < 1 || C % (kBgCols * V)) return fail(TMPI_ERR_UNSUPPORTED, "bias_grad: C=%d must be a multiple of %d", C, kBgCols * V);
  if (z && !dz) return fail(TMPI_ERR_INVALID, "bias_grad: z given without an output for dz");
  const int slabs = C / (kBgCols * V);
  const int rb = std::max(1, std::min((rows + 1) / 2, std::max(1, 2 * kBgMaxRowBlocks / slabs)));
  bias_grad_kernel<T, V><<<dim3(slabs, rb), kBgThreads, 0, s>>>((const T*)dy, (const T*)z, (T*)dz, (float*)scratch, rows, C);
  bias_grad_finalize_kernel<T><<<(C + 255) / 256, 256, 0, s>>>((const float*)scratch, rb, C, (T*)db);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "bias_grad launch: %s", cudaGetErrorString(e));
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

size_t tmpi_bias_grad_scratch_bytes(int channels) { return (size_t)2 * kBgMaxRowBlocks * channels * sizeof(float); }

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

}  // extern "C"
