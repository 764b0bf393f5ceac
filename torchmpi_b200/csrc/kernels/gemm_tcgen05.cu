// bf16 GEMM on the 5th-generation tensor cores: C[M,N] = act(A[M,K] * B[N,K]^T + bias).
//
// A and B are row-major with K contiguous (an nn.Linear weight is exactly B).  Operands are staged
// by TMA into 128-byte-swizzled shared-memory tiles, multiplied by tcgen05.mma into fp32
// accumulators that live in tensor memory, and read back with tcgen05.ld for the epilogue (bias,
// GELU, bf16 store).  See gemm_core.cuh for the roles.  Tiles are visited in bands of 16 M-tiles
// so that the CTAs running at one time share B panels in L2.  The reference has no GEMM
// (its model-parallel example calls Torch's Linear, examples/mnist/mnist_modelparallel.lua:30-60).
#include "gemm_core.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"
#include <cstring>
#include <mutex>

namespace tmpi {
namespace gemm {

constexpr int BAND = 16;   // M-tiles per band

// tile index -> (m_blk, n_blk): within a band of BAND tile-rows, consecutive tiles walk down the
// rows first, so the ~148 concurrent tiles cover few distinct B panels and a band of A panels.
__device__ __forceinline__ void band_order(int t, int tiles_m, int tiles_n, int* m_blk, int* n_blk) {
  const int per_band = BAND * tiles_n;
  const int band = t / per_band;
  const int rows = min(BAND, tiles_m - band * BAND);
  const int r = t - band * per_band;
  *m_blk = band * BAND + r % rows;
  *n_blk = r / rows;
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, __nv_bfloat16* __restrict__ C, const Problem p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *tiles, *staging;
  Shared* sh;
  carve(smem_raw, &tiles, &sh, &staging);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  setup(sh, tiles, warp, &map_a, &map_b);

  const int total = p.tiles_m * p.tiles_n;
  auto order = [&](int it, int* m_blk, int* n_blk) -> bool {
    const int t = blockIdx.x + it * gridDim.x;
    if (t >= total) return false;
    band_order(t, p.tiles_m, p.tiles_n, m_blk, n_blk);
    return true;
  };
  if (warp == 0) {
    if (sm100::elect_one()) producer(sh, tiles, p, &map_a, &map_b, order, [](int, const CUtensorMap**, int*) { return true; });
  } else if (warp == 1) {
    if (sm100::elect_one()) mma_issuer(sh, tiles, p, order);
  } else if (p.tma_store) {
    epilogue_tma(sh, staging, p, warp & 3, lane, order,
                 [&](int m_blk, const CUtensorMap** m, int* row0) { *m = &map_c; *row0 = m_blk * BM; });
  } else {
    epilogue(sh, p, warp & 3, lane, order,
             [&](int, int row) { return C + (size_t)row * p.N; });
  }
  teardown(sh, warp);
}

}  // namespace gemm

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  });
  return fn;
}

// Tensor map of a row-major [rows, cols] bf16 matrix (cols contiguous, leading dimension ld elements)
// with a box of box_rows x 64 columns and the 128-byte swizzle.
int make_tmap_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(TMPI_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled is not available");
  if (((uintptr_t)base & 15) || (ld * 2) % 16) return fail(TMPI_ERR_INVALID, "TMA operand must be 16-byte aligned with a 16-byte multiple row pitch");
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)gemm::BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(TMPI_ERR_CUDA, "cuTensorMapEncodeTiled failed (CUresult %d)", (int)r);
  return TMPI_OK;
}

int gemm_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

bool gemm_pair_applicable(const void* C, int M, int N, int K, int flags);
int launch_gemm_pair(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int epilogue,
                     int* status_word, cudaStream_t stream, int64_t lda, int64_t ldb, int64_t ldc);

static int* gemm_status_word() {
  static int* dev_ptr = nullptr;
  static int* host_ptr = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    if (cudaHostAlloc((void**)&host_ptr, sizeof(int), cudaHostAllocMapped) == cudaSuccess) {
      *host_ptr = 0;
      cudaHostGetDevicePointer((void**)&dev_ptr, host_ptr, 0);
    }
  });
  return dev_ptr;
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

int tmpi_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int epilogue,
                   void* stream) {
  if (M < 1 || N < 1 || K < 1) return fail(TMPI_ERR_INVALID, "gemm: empty problem");
  const bool k_rows = !(epilogue & gemm::A_IS_KM) || !(epilogue & gemm::B_IS_KN);   // some operand has K contiguous
  if (k_rows && K % 8) return fail(TMPI_ERR_INVALID, "gemm: K must be a multiple of 8 (16-byte rows for TMA)");
  if ((epilogue & gemm::EPI_BIAS) && !bias) return fail(TMPI_ERR_INVALID, "gemm: bias epilogue without bias");
  if (tunable("gemm_pair") && gemm_pair_applicable(C, M, N, K, epilogue))
    return launch_gemm_pair(A, B, C, bias, M, N, K, epilogue, gemm_status_word(), (cudaStream_t)stream, 0, 0, 0);
  if (epilogue & (gemm::B_IS_KN | gemm::A_IS_KM))
    return fail(TMPI_ERR_UNSUPPORTED, "gemm: operands given as [K, M] / [K, N] need the CTA-pair kernel (M, N >= 256, M, N %% 8 == 0)");
  CUtensorMap ma, mb;
  int st = make_tmap_bf16(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, gemm::BM);
  if (st) return st;
  // a narrow output (one column tile, N <= 128) stages and multiplies only the rows of B that exist
  const int mma_n = N <= gemm::BN / 2 ? (N + 15) / 16 * 16 : 0;
  st = make_tmap_bf16(&mb, B, (uint64_t)N, (uint64_t)K, (uint64_t)K, mma_n ? mma_n : gemm::BN);
  if (st) return st;
  gemm::Problem p{};
  p.mma_n = mma_n;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + gemm::BM - 1) / gemm::BM;
  p.tiles_n = (N + gemm::BN - 1) / gemm::BN;
  p.k_blocks = (K + gemm::BK - 1) / gemm::BK;
  p.epilogue = epilogue;
  p.bias = (const __nv_bfloat16*)bias;
  p.status = gemm_status_word();
  CUtensorMap mc;
  memset(&mc, 0, sizeof(mc));
  p.tma_store = (N % 8 == 0 && ((uintptr_t)C & 15) == 0) ? 1 : 0;
  if (p.tma_store && (st = make_tmap_bf16(&mc, C, (uint64_t)M, (uint64_t)N, (uint64_t)N, gemm::BM))) return st;
  static std::once_flag attr_once;
  std::call_once(attr_once, [] {
    cudaFuncSetAttribute(gemm::gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gemm::SMEM_BYTES);
  });
  int grid = std::min(p.tiles_m * p.tiles_n, gemm_sm_count());
  gemm::gemm_bf16_kernel<<<grid, gemm::THREADS, gemm::SMEM_BYTES, (cudaStream_t)stream>>>(ma, mb, mc, (__nv_bfloat16*)C, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : fail(TMPI_ERR_CUDA, "gemm launch: %s", cudaGetErrorString(e));
}

// The same product with explicit row pitches (elements) of A, B and C as stored: the extents need not
// be multiples of 8 as long as the pitches are (a [T, 50257] logit matrix kept in rows of 50264
// elements).  CTA-pair kernel only: M, N >= 256.
int tmpi_gemm_bf16_ex(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int64_t lda,
                      int64_t ldb, int64_t ldc, int epilogue, void* stream) {
  if (M < 256 || N < 256 || K < 1) return fail(TMPI_ERR_UNSUPPORTED, "gemm_ex: needs M, N >= 256 (got %d x %d x %d)", M, N, K);
  if ((epilogue & gemm::EPI_BIAS) && !bias) return fail(TMPI_ERR_INVALID, "gemm: bias epilogue without bias");
  if ((lda | ldb | ldc) % 8 || lda <= 0 || ldb <= 0 || ldc <= 0)
    return fail(TMPI_ERR_INVALID, "gemm_ex: row pitches must be positive multiples of 8 elements");
  if (((uintptr_t)A | (uintptr_t)B | (uintptr_t)C) & 15) return fail(TMPI_ERR_INVALID, "gemm_ex: operands must be 16-byte aligned");
  return launch_gemm_pair(A, B, C, bias, M, N, K, epilogue, gemm_status_word(), (cudaStream_t)stream, lda, ldb, ldc);
}

// Non-zero after a GEMM CTA gave up on a bounded wait (1000 + the point where it happened); clears it.
int tmpi_gemm_status(void) {
  int* d = gemm_status_word();
  (void)d;
  static int* host = nullptr;
  if (!host && d) {
    // the mapped host pointer of the same word
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, d) == cudaSuccess) host = (int*)at.hostPointer;
  }
  if (!host) return 0;
  int v = *(volatile int*)host;
  if (v) *(volatile int*)host = 0;
  return v;
}

}  // extern "C"
