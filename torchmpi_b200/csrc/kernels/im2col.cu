// Patch matrix of the ResNet stem: a 7 x 7, stride-2, pad-3 convolution over a channels-last input
// with 3 channels, written as col[N*OH*OW, 160] (147 = 7*7*3 patch values in (kh, kw, c) order, then
// zeros) so that the convolution becomes one tensor-core GEMM with the [Cout, 160] weight matrix.
// Library convolutions pad the 3 input channels to 8 and run the stem at a few percent of the
// tensor peak; the reference has no convolution of its own (it trains Torch7 modules).
//
// One block per output row (n, oh): the 7 input rows it needs go to shared memory with 16-byte
// loads, then every thread assembles 16-byte chunks of the patch rows and stores them coalesced.
#include "vec.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"

namespace tmpi {

constexpr int kStemK = 7, kStemC = 3, kStemStride = 2, kStemPad = 3;
constexpr int kStemPatch = kStemK * kStemK * kStemC;      // 147
constexpr int kStemKPad = 160;                            // patch row length in the GEMM (16-byte multiple)
constexpr int kStemThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kStemThreads) stem_im2col_kernel(const T* __restrict__ x, T* __restrict__ col,
                                                                   int H, int W, int OH, int OW) {
  extern __shared__ __align__(16) unsigned char s_raw[];
  T* s_in = reinterpret_cast<T*>(s_raw);                  // [7][W * 3]
  const int row_elems = W * kStemC;
  const int n = blockIdx.x / OH, oh = blockIdx.x % OH;
  const int vec_per_row = row_elems * (int)sizeof(T) / 16;
  for (int i = threadIdx.x; i < kStemK * vec_per_row; i += kStemThreads) {
    const int kh = i / vec_per_row, v = i % vec_per_row;
    const int ih = oh * kStemStride - kStemPad + kh;
    uint4 u = make_uint4(0, 0, 0, 0);
    if (ih >= 0 && ih < H) u = __ldg(reinterpret_cast<const uint4*>(x + ((size_t)n * H + ih) * row_elems) + v);
    reinterpret_cast<uint4*>(s_in + (size_t)kh * row_elems)[v] = u;
  }
  __syncthreads();
  constexpr int V = 16 / sizeof(T);
  constexpr int chunks_per_row = kStemKPad / V;
  T* out = col + ((size_t)n * OH + oh) * OW * kStemKPad;
  for (int q = threadIdx.x; q < OW * chunks_per_row; q += kStemThreads) {
    const int ow = q / chunks_per_row, k0 = (q % chunks_per_row) * V;
    const int base = (ow * kStemStride - kStemPad) * kStemC;    // element index of (kw = 0, c = 0) in an input row
    Pack<T, V> o;
#pragma unroll
    for (int j = 0; j < V; ++j) {
      const int k = k0 + j;
      const int kh = k / (kStemK * kStemC), idx = base + (k - kh * (kStemK * kStemC));
      T v = T(0.f);
      if (k < kStemPatch && idx >= 0 && idx < row_elems) v = s_in[kh * row_elems + idx];
      o.v[j] = v;
    }
    st_pack<T, V>(out + (size_t)ow * kStemKPad + k0, o);
  }
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

int tmpi_stem_patch_width(void) { return kStemKPad; }

// x: [N, H, W, 3] (channels-last), col: [N * OH * OW, 160] with OH = (H + 6 - 7) / 2 + 1, same for OW.
int tmpi_stem_im2col(const void* x, void* col, int N, int H, int W, int dtype, void* stream) {
  if (N < 1 || H < 1 || W < 1) return fail(TMPI_ERR_INVALID, "stem im2col: empty input");
  const int OH = (H + 2 * kStemPad - kStemK) / kStemStride + 1, OW = (W + 2 * kStemPad - kStemK) / kStemStride + 1;
  const size_t es = dtype == TMPI_F32 ? 4 : 2;
  if ((W * kStemC * es) % 16 || ((uintptr_t)x & 15) || ((uintptr_t)col & 15))
    return fail(TMPI_ERR_UNSUPPORTED, "stem im2col: input rows must be 16-byte multiples and the buffers 16-byte aligned");
  const size_t smem = (size_t)kStemK * W * kStemC * es;
  if (smem > 200 * 1024) return fail(TMPI_ERR_UNSUPPORTED, "stem im2col: image too wide (%d)", W);
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = N * OH;
#define TMPI_STEM_LAUNCH(T)                                                                                       \
  do {                                                                                                            \
    if (smem > 48 * 1024) cudaFuncSetAttribute(stem_im2col_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    stem_im2col_kernel<T><<<grid, kStemThreads, smem, s>>>((const T*)x, (T*)col, H, W, OH, OW);                   \
  } while (0)
  switch (dtype) {
    case TMPI_BF16: TMPI_STEM_LAUNCH(__nv_bfloat16); break;
    case TMPI_F16: TMPI_STEM_LAUNCH(__half); break;
    case TMPI_F32: TMPI_STEM_LAUNCH(float); break;
    default: return fail(TMPI_ERR_UNSUPPORTED, "stem im2col: dtype %d", dtype);
  }
#undef TMPI_STEM_LAUNCH
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "stem im2col launch: %s", cudaGetErrorString(e));
}

}  // extern "C"
