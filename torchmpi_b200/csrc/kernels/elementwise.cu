// Single-GPU hot ops: fused SGD step, softmax cross-entropy forward+backward,
// abs-mean/variance statistics, EASGD elastic step, Downpour accumulation.
//
// The reference performs each of these as several cutorch kernels per tensor
// (torchmpi/BlockSequential.lua:159-170, torchmpi/init.lua:372-381,
// torchmpi/parameterserver/easgdupdate.lua:73-75,
// torchmpi/parameterserver/downpourupdate.lua:49-59); each is one pass here.
#include "collectives.cuh"
#include "../include/tmpi_c_api.h"
#include "../runtime/common.h"

namespace tmpi {

static int cuda_fail(cudaError_t e, const char* what) {
  return fail(TMPI_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

// SM count of the current device (cached per device; a race writes the same value twice).
static int sm_count() {
  static int n[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!n[dev]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
    n[dev] = v;
  }
  return n[dev];
}

// ------------------------------------------------------------------ softmax cross-entropy
// One block per row.  loss_rows[r] = logsumexp(x_r) - x_r[label]; dlogits = (softmax - onehot) * gscale.
// The last block to finish adds the row losses in row order (deterministic) into loss_out[0].
template <typename T>
__global__ void __launch_bounds__(256) xent_kernel(const T* __restrict__ logits, const long long* __restrict__ labels,
                                                   int rows, int cols, int ld, float* __restrict__ loss_out,
                                                   T* __restrict__ dlogits, float gscale,
                                                   float* __restrict__ row_loss, unsigned* __restrict__ counter) {
  __shared__ float s_red[32];
  __shared__ float s_bcast;
  __shared__ bool s_last;
  const int r = blockIdx.x;
  const T* x = logits + (size_t)r * ld;               // ld: row pitch in elements (>= cols)
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;

  float m = -INFINITY;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) m = fmaxf(m, (float)to_acc<T>(x[c]));
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o));
  if (lane == 0) s_red[warp] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = s_red[0];
    for (int w = 1; w < nwarp; ++w) v = fmaxf(v, s_red[w]);
    s_bcast = v;
  }
  __syncthreads();
  m = s_bcast;
  float sum = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) sum += __expf((float)to_acc<T>(x[c]) - m);
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(~0u, sum, o);
  __syncthreads();
  if (lane == 0) s_red[warp] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = 0.f;
    for (int w = 0; w < nwarp; ++w) v += s_red[w];
    s_bcast = v;
  }
  __syncthreads();
  sum = s_bcast;
  const float inv = 1.f / sum;
  const int label = (int)labels[r];
  if (dlogits) {
    T* d = dlogits + (size_t)r * ld;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      float p = __expf((float)to_acc<T>(x[c]) - m) * inv;
      d[c] = from_acc<T>((typename AccOf<T>::type)((p - (c == label ? 1.f : 0.f)) * gscale));
    }
    for (int c = cols + threadIdx.x; c < ld; c += blockDim.x) d[c] = from_acc<T>((typename AccOf<T>::type)0.f);
  }
  if (threadIdx.x == 0) {
    float xl = (label >= 0 && label < cols) ? (float)to_acc<T>(x[label]) : m;
    row_loss[r] = __logf(sum) + m - xl;
    __threadfence();
    s_last = atomicAdd(counter, 1u) == (unsigned)rows - 1;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    float v = 0.f;
    for (int i = threadIdx.x; i < rows; i += blockDim.x) v += row_loss[i];   // fixed per-thread order
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(~0u, v, o);
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < nwarp; ++w) t += s_red[w];
      loss_out[0] = t;
      *counter = 0;
    }
  }
}

// Codecs between a 16-byte pack of T and fp32 lanes, for the row staged in shared memory.
template <typename T> struct RowPack;
template <> struct RowPack<float> {
  static constexpr int V = 4;
  using E = float;                                  // the type exp(x - max) is kept in between the passes
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    f[0] = __uint_as_float(u.x); f[1] = __uint_as_float(u.y); f[2] = __uint_as_float(u.z); f[3] = __uint_as_float(u.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
  }
  static __device__ __forceinline__ void unpack_e(const uint4& u, float* f) { unpack(u, f); }
  static __device__ __forceinline__ uint4 pack_e(const float* f) { return pack(f); }
  static __device__ __forceinline__ float max(const uint4& u, float m) {
    return fmaxf(fmaxf(fmaxf(__uint_as_float(u.x), __uint_as_float(u.y)), fmaxf(__uint_as_float(u.z), __uint_as_float(u.w))), m);
  }
};
template <> struct RowPack<__half> {
  static constexpr int V = 8;
  using E = __half;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int k = 0; k < 4; ++k) { float2 v = __half22float2(h[k]); f[2 * k] = v.x; f[2 * k + 1] = v.y; }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { __half2 h = __floats2half2_rn(f[2 * k], f[2 * k + 1]); w[k] = *reinterpret_cast<uint32_t*>(&h); }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  static __device__ __forceinline__ void unpack_e(const uint4& u, float* f) { unpack(u, f); }
  static __device__ __forceinline__ uint4 pack_e(const float* f) { return pack(f); }
  static __device__ __forceinline__ float max(const uint4& u, float m) {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
    __half2 a = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return fmaxf(fmaxf(__low2float(a), __high2float(a)), m);
  }
};

template <> struct RowPack<__nv_bfloat16> {
  static constexpr int V = 8;
  using E = __half;
  static __device__ __forceinline__ void unpack(const uint4& u, float* f) {   // bf16 -> fp32 is a shift or a mask
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) { f[2 * k] = __uint_as_float(w[k] << 16); f[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u); }
  }
  static __device__ __forceinline__ uint4 pack(const float* f) {
    uint32_t w[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) { __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]); w[k] = *reinterpret_cast<uint32_t*>(&h); }
    return make_uint4(w[0], w[1], w[2], w[3]);
  }
  // exp(x - max) lies in (0, 1]: kept as fp16 (11 bits of mantissa in the same two bytes) between the passes.
  // Read back without conversion instructions (they are the slow ones here): the 15 value bits of a non-negative
  // half, moved to the top of an fp32 mantissa, are the half's value times 2^-112, subnormals included.
  static __device__ __forceinline__ void unpack_e(const uint4& u, float* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      f[2 * k] = __uint_as_float((w[k] << 13) & 0x0fffe000u) * 0x1p112f;
      f[2 * k + 1] = __uint_as_float((w[k] >> 3) & 0x0fffe000u) * 0x1p112f;
    }
  }
  static __device__ __forceinline__ uint4 pack_e(const float* f) { return RowPack<__half>::pack(f); }
  static __device__ __forceinline__ float max(const uint4& u, float m) {      // two elements per instruction
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    __nv_bfloat162 a = __hmax2(__hmax2(h[0], h[1]), __hmax2(h[2], h[3]));
    return fmaxf(fmaxf(__low2float(a), __high2float(a)), m);
  }
};
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// One block per row with the row staged in shared memory: the logits are read from HBM once and the gradient is
// written once.  The aligned body of the row travels as asynchronous 16-byte copies that are all in flight together
// (the row keeps its global misalignment in shared memory, so aligned global packs land on aligned shared addresses;
// rows of 50257 bf16 start on 2-byte boundaries only, and a few head and tail elements move as scalars).  Every
// thread works on the same packs in all passes, so only the two reductions need the block.  The second pass replaces
// the logits in shared memory by exp(x - max) (fp32 for fp32 logits, fp16 otherwise), so the gradient pass is one multiplication per element
// and the exponential is evaluated once; the label's entry is recomputed in fp32 by one thread at the end.
template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS) xent_row_smem_kernel(
    const T* __restrict__ logits, const long long* __restrict__ labels, int rows, int cols, int ld,
    float* __restrict__ loss_out, T* __restrict__ dlogits, float gscale, float* __restrict__ row_loss,
    unsigned* __restrict__ counter) {
  extern __shared__ __align__(16) unsigned char s_row_raw[];
  __shared__ float s_red[32];
  __shared__ float s_bcast;
  __shared__ bool s_last;
  using RP = RowPack<T>;
  using E = typename RP::E;
  constexpr int V = RP::V;
  constexpr float kLog2e = 1.4426950408889634f;
  const int r = blockIdx.x, tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = THREADS >> 5;
  const T* x = logits + (size_t)r * ld;               // ld: row pitch in elements (>= cols)
  const unsigned mis = (unsigned)((uintptr_t)x & 15);
  T* srow = reinterpret_cast<T*>(s_row_raw + mis);
  int head = mis ? (int)((16 - mis) / sizeof(T)) : 0;
  if (head > cols) head = cols;
  const int nvec = (cols - head) / V, tail0 = head + nvec * V;
  const uint4* gx = reinterpret_cast<const uint4*>(x + head);
  uint4* sx = reinterpret_cast<uint4*>(srow + head);
  const int label = (int)labels[r];

  // pass 1: global -> shared, then the maximum of this thread's packs
  {
    const uint32_t s0 = (uint32_t)__cvta_generic_to_shared(sx);
    for (int i = tid; i < nvec; i += THREADS)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s0 + 16u * (uint32_t)i), "l"(gx + i) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  float m = -INFINITY;
  for (int c = tid; c < head; c += THREADS) { T v = x[c]; srow[c] = v; m = fmaxf(m, (float)to_acc<T>(v)); }
  for (int c = tail0 + tid; c < cols; c += THREADS) { T v = x[c]; srow[c] = v; m = fmaxf(m, (float)to_acc<T>(v)); }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  for (int i = tid; i < nvec; i += THREADS) m = RP::max(sx[i], m);
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(~0u, m, o));
  if (lane == 0) s_red[warp] = m;
  __syncthreads();                                    // also: the whole row is in shared memory
  float xl = 0.f;
  if (tid == 0) {
    float v = s_red[0];
    for (int w = 1; w < nwarp; ++w) v = fmaxf(v, s_red[w]);
    s_bcast = v;
    xl = (label >= 0 && label < cols) ? (float)to_acc<T>(srow[label]) : v;   // before pass 2 overwrites the row
  }
  __syncthreads();
  m = s_bcast;
  const float mL = m * kLog2e;

  // pass 2: exponentials, kept in shared memory in place of the logits, and their sum
  float sum0 = 0.f, sum1 = 0.f;
  auto scalar_exp = [&](int c) {
    float e = ex2_approx(fmaf((float)to_acc<T>(srow[c]), kLog2e, -mL));
    sum0 += e;
    reinterpret_cast<E*>(srow)[c] = from_acc<E>((typename AccOf<E>::type)e);
  };
  for (int c = tid; c < head; c += THREADS) scalar_exp(c);
  for (int c = tail0 + tid; c < cols; c += THREADS) scalar_exp(c);
  for (int i = tid; i < nvec; i += THREADS) {
    float f[V];
    RP::unpack(sx[i], f);
#pragma unroll
    for (int j = 0; j < V; ++j) f[j] = ex2_approx(fmaf(f[j], kLog2e, -mL));
#pragma unroll
    for (int j = 0; j < V; j += 2) { sum0 += f[j]; sum1 += f[j + 1]; }
    sx[i] = RP::pack_e(f);
  }
  float sum = sum0 + sum1;
  for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(~0u, sum, o);
  if (lane == 0) s_red[warp] = sum;                   // s_red was last read before the previous barrier
  __syncthreads();
  if (tid == 0) {
    float v = 0.f;
    for (int w = 0; w < nwarp; ++w) v += s_red[w];
    s_bcast = v;
  }
  __syncthreads();
  sum = s_bcast;
  const float inv = 1.f / sum;

  // pass 3: gradient = exp * (gscale / sum), written once; the label's entry afterwards
  if (dlogits) {
    T* d = dlogits + (size_t)r * ld;
    const float k = inv * gscale;
    for (int c = cols + tid; c < ld; c += THREADS) d[c] = from_acc<T>((typename AccOf<T>::type)0.f);   // pitch padding
    auto scalar_grad = [&](int c) {
      d[c] = from_acc<T>((typename AccOf<T>::type)((float)to_acc<E>(reinterpret_cast<const E*>(srow)[c]) * k));
    };
    for (int c = tid; c < head; c += THREADS) scalar_grad(c);
    for (int c = tail0 + tid; c < cols; c += THREADS) scalar_grad(c);
    if ((((uintptr_t)d) & 15) == mis) {
      uint4* gd = reinterpret_cast<uint4*>(d + head);
      for (int i = tid; i < nvec; i += THREADS) {
        float f[V];
        RP::unpack_e(sx[i], f);
#pragma unroll
        for (int j = 0; j < V; ++j) f[j] *= k;
        gd[i] = RP::pack(f);
      }
    } else {
      for (int c = head + tid; c < tail0; c += THREADS) scalar_grad(c);
    }
    __syncthreads();                                  // the label's entry is overwritten after every other store
    if (tid == 0 && label >= 0 && label < cols)
      d[label] = from_acc<T>((typename AccOf<T>::type)((ex2_approx(fmaf(xl, kLog2e, -mL)) * inv - 1.f) * gscale));
  }
  if (tid == 0) {
    row_loss[r] = __logf(sum) + m - xl;
    __threadfence();
    s_last = atomicAdd(counter, 1u) == (unsigned)rows - 1;
  }
  __syncthreads();
  if (s_last) {
    __threadfence();
    float v = 0.f;
    for (int i = tid; i < rows; i += THREADS) v += row_loss[i];   // fixed per-thread order
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(~0u, v, o);
    if (lane == 0) s_red[warp] = v;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
      for (int w = 0; w < nwarp; ++w) t += s_red[w];
      loss_out[0] = t;
      *counter = 0;
    }
  }
}

// ------------------------------------------------------------------ abs-mean / variance
constexpr int kStatBlocks = 148 * 8;          // every resident slot of 256 threads on the SMs
constexpr int kStatThreads = 256;

template <typename T>
__device__ __forceinline__ void absstat_body(const T* __restrict__ x, size_t n, double* __restrict__ out2,
                                             double* __restrict__ partial, unsigned* __restrict__ counter) {
  __shared__ double s1[kStatThreads / 32], s2[kStatThreads / 32];
  __shared__ bool s_last;
  double a = 0.0, b = 0.0;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  // 16-byte packs over the aligned body (two loads in flight per thread), single elements before and after it
  constexpr int V = 16 / sizeof(T);
  const size_t mis = ((uintptr_t)x & 15) / sizeof(T);
  const size_t head = mis ? (V - mis < n ? V - mis : n) : 0;
  const size_t nv = (n - head) / V, tail0 = head + nv * V;
  for (size_t i = t0; i < head; i += stride) { double v = fabs((double)to_acc<T>(x[i])); a += v; b += v * v; }
  for (size_t i = tail0 + t0; i < n; i += stride) { double v = fabs((double)to_acc<T>(x[i])); a += v; b += v * v; }
  const T* xb = x + head;
  size_t i = t0;
  if constexpr (sizeof(T) == 8) {
    for (; i < nv; i += stride) {
      Pack<T, V> p0 = ld_pack<T, V>(xb + i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) { double v = fabs((double)to_acc<T>(p0.v[k])); a += v; b += v * v; }
    }
  } else {
    // Four packs in flight per thread; their 16 to 32 elements are summed in fp32 (a short chain, so the rounding
    // stays near 1e-7 relative) and only the two partial sums go through the slow fp32 -> fp64 conversion.
    constexpr int U = 4;
    auto fold = [&](const Pack<T, V>& p, float& fa, float& fb) {
#pragma unroll
      for (int k = 0; k < V; ++k) { float v = fabsf((float)to_acc<T>(p.v[k])); fa += v; fb = fmaf(v, v, fb); }
    };
    for (; i + (U - 1) * stride < nv; i += U * stride) {
      Pack<T, V> p[U];
#pragma unroll
      for (int u = 0; u < U; ++u) p[u] = ld_pack<T, V>(xb + (i + u * stride) * V);
      float fa = 0.f, fb = 0.f;
#pragma unroll
      for (int u = 0; u < U; ++u) fold(p[u], fa, fb);
      a += (double)fa; b += (double)fb;
    }
    for (; i < nv; i += stride) {
      Pack<T, V> p0 = ld_pack<T, V>(xb + i * V);
      float fa = 0.f, fb = 0.f;
      fold(p0, fa, fb);
      a += (double)fa; b += (double)fb;
    }
  }
  for (int o = 16; o; o >>= 1) { a += __shfl_xor_sync(~0u, a, o); b += __shfl_xor_sync(~0u, b, o); }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s1[warp] = a; s2[warp] = b; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double ta = 0.0, tb = 0.0;
    for (int w = 0; w < kStatThreads / 32; ++w) { ta += s1[w]; tb += s2[w]; }
    partial[2 * blockIdx.x] = ta; partial[2 * blockIdx.x + 1] = tb;
    __threadfence();
    s_last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (s_last) {                  // the last block sums the partials: a fixed tree, the same bits on every run
    __threadfence();
    double ta = 0.0, tb = 0.0;
    for (unsigned i = threadIdx.x; i < gridDim.x; i += kStatThreads) { ta += partial[2 * i]; tb += partial[2 * i + 1]; }
    for (int o = 16; o; o >>= 1) { ta += __shfl_xor_sync(~0u, ta, o); tb += __shfl_xor_sync(~0u, tb, o); }
    __syncthreads();
    if (lane == 0) { s1[warp] = ta; s2[warp] = tb; }
    __syncthreads();
    if (threadIdx.x == 0) {
      ta = 0.0; tb = 0.0;
      for (int w = 0; w < kStatThreads / 32; ++w) { ta += s1[w]; tb += s2[w]; }
      out2[0] = ta; out2[1] = tb;
      *counter = 0;   // ready for the next launch
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kStatThreads) absstat_kernel(const T* x, size_t n, double* out2, double* partial,
                                                               unsigned* counter) {
  absstat_body<T>(x, n, out2, partial, counter);
}

// ------------------------------------------------------------------ EASGD / Downpour
template <typename T, int V>
__global__ void __launch_bounds__(256) easgd_kernel(T* __restrict__ local, const T* __restrict__ center,
                                                    T* __restrict__ delta, size_t nv, float alpha) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    Pack<T, V> x = ld_pack<T, V>(local + i * V), c = ld_pack<T, V>(center + i * V), d;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float xv = (float)to_acc<T>(x.v[k]);
      float dv = (float)to_acc<T>(c.v[k]) - xv;
      x.v[k] = from_acc<T>((typename AccOf<T>::type)(xv + alpha * dv));
      d.v[k] = from_acc<T>((typename AccOf<T>::type)(-alpha * dv));
    }
    st_pack<T, V>(local + i * V, x);
    st_pack<T, V>(delta + i * V, d);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(256) accum_kernel(T* __restrict__ acc, const T* __restrict__ g, size_t nv,
                                                    float scale, int zero_first) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += (size_t)gridDim.x * blockDim.x) {
    Pack<T, V> a = ld_pack<T, V>(acc + i * V), x = ld_pack<T, V>(g + i * V);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float av = zero_first ? 0.f : (float)to_acc<T>(a.v[k]);
      a.v[k] = from_acc<T>((typename AccOf<T>::type)(av + scale * (float)to_acc<T>(x.v[k])));
    }
    st_pack<T, V>(acc + i * V, a);
  }
}


static bool aligned16(const void* p) { return ((uintptr_t)p & 15) == 0; }

}  // namespace tmpi

using namespace tmpi;

#define DISPATCH_FLOAT(dtype, ...)                                      \
  switch (dtype) {                                                      \
    case TMPI_F32: { using T = float; __VA_ARGS__; } break;                  \
    case TMPI_BF16: { using T = __nv_bfloat16; __VA_ARGS__; } break;         \
    case TMPI_F16: { using T = __half; __VA_ARGS__; } break;                 \
    case TMPI_F64: { using T = double; __VA_ARGS__; } break;                 \
    default: return fail(TMPI_ERR_UNSUPPORTED, "dtype %d not supported here", dtype); \
  }

template <typename T>
static cudaError_t launch_xent(const void* logits, const int64_t* labels, int rows, int cols, int ld, float* loss_sum, void* dlogits,
                               float gscale, float* row_loss, unsigned* counter, cudaStream_t s) {
  // 512 threads measured faster than 1024 (0.37 against 0.39 ms for 8192 x 50257 bf16)
  constexpr int kThreads = 512;
  constexpr size_t kMaxRowBytes = 112 * 1024;          // two such blocks per SM
  const size_t row_bytes = (size_t)cols * sizeof(T) + 16;
  if (row_bytes <= kMaxRowBytes && ((uintptr_t)logits % sizeof(T)) == 0) {
    // the attribute belongs to the (function, device) pair; setting it is cheap, so every call does it
    cudaError_t ae = cudaFuncSetAttribute(xent_row_smem_kernel<T, kThreads>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)kMaxRowBytes);
    if (ae != cudaSuccess) return ae;
    xent_row_smem_kernel<T, kThreads><<<rows, kThreads, row_bytes, s>>>((const T*)logits, (const long long*)labels, rows, cols, ld,
                                                                        loss_sum, (T*)dlogits, gscale, row_loss, counter);
  } else {
    xent_kernel<T><<<rows, 256, 0, s>>>((const T*)logits, (const long long*)labels, rows, cols, ld, loss_sum, (T*)dlogits, gscale,
                                        row_loss, counter);
  }
  return cudaGetLastError();
}

extern "C" {

int tmpi_sgd_momentum(void* weight, int wdt, const void* grad, int gdt, void* master, void* momentum, size_t n,
                      float lr, float mc, float damp, float wd, float gscale, int nesterov, int first_step,
                      int zero_grads, void* stream) {
  if (wdt != gdt) return fail(TMPI_ERR_INVALID, "sgd: weight and gradient dtypes differ");
  size_t es = dtype_size(wdt), V = 16 / es;
  if (n % V || !aligned16(weight) || !aligned16(grad) || !aligned16(master) || !aligned16(momentum))
    return fail(TMPI_ERR_INVALID, "sgd: buffers must be 16-byte aligned and hold a multiple of %zu elements", V);
  SgdArgs a{};
  a.P.n = 1; a.P.me = 0; a.P.base[0] = nullptr; a.P.status = nullptr;
  // with a null heap base the "offsets" are the absolute addresses
  a.grad_off = (size_t)grad; a.weight_off = (size_t)weight;
  a.master = (float*)master; a.momentum = (float*)momentum; a.n = n;
  a.lr = lr; a.momentum_coef = mc; a.dampening = damp; a.weight_decay = wd; a.grad_scale = gscale;
  a.nesterov = nesterov; a.first_step = first_step; a.zero_grads = zero_grads; a.use_nvls = 0;
  size_t nv = n / V;
  int grid = (int)std::min<size_t>((nv + 511) / 512, (size_t)sm_count() * 2);
  cudaError_t e = launch_allreduce_sgd(gdt, wdt, &a, 1, grid < 1 ? 1 : grid, 512, (cudaStream_t)stream);
  return e == cudaSuccess ? TMPI_OK : cuda_fail(e, "sgd_momentum launch");
}

size_t tmpi_xent_scratch_bytes(int rows) { return (size_t)rows * sizeof(float) + 256; }

// ld: row pitch of logits and dlogits in elements (0 or cols: dense rows).  The columns between cols and
// ld are not read; in dlogits they are set to zero.
int tmpi_xent_fwd_bwd_ld(const void* logits, int dtype, const int64_t* labels, int rows, int cols, int ld, float* loss_sum,
                         void* dlogits, float gscale, void* scratch, void* stream);

int tmpi_xent_fwd_bwd(const void* logits, int dtype, const int64_t* labels, int rows, int cols, float* loss_sum,
                      void* dlogits, float gscale, void* scratch, void* stream) {
  return tmpi_xent_fwd_bwd_ld(logits, dtype, labels, rows, cols, cols, loss_sum, dlogits, gscale, scratch, stream);
}

int tmpi_xent_fwd_bwd_ld(const void* logits, int dtype, const int64_t* labels, int rows, int cols, int ld, float* loss_sum,
                         void* dlogits, float gscale, void* scratch, void* stream) {
  if (rows < 1 || cols < 1) return fail(TMPI_ERR_INVALID, "xent: empty input");
  if (ld == 0) ld = cols;
  if (ld < cols) return fail(TMPI_ERR_INVALID, "xent: row pitch %d below the row length %d", ld, cols);
  // scratch layout: [counter (256 B, zero before first use)] [row losses]
  unsigned* counter = (unsigned*)scratch;
  float* row_loss = (float*)((char*)scratch + 256);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  switch (dtype) {
    case TMPI_F32: e = launch_xent<float>(logits, labels, rows, cols, ld, loss_sum, dlogits, gscale, row_loss, counter, s); break;
    case TMPI_BF16: e = launch_xent<__nv_bfloat16>(logits, labels, rows, cols, ld, loss_sum, dlogits, gscale, row_loss, counter, s); break;
    case TMPI_F16: e = launch_xent<__half>(logits, labels, rows, cols, ld, loss_sum, dlogits, gscale, row_loss, counter, s); break;
    default: return fail(TMPI_ERR_UNSUPPORTED, "xent: dtype %d", dtype);
  }
  return e == cudaSuccess ? TMPI_OK : cuda_fail(e, "xent launch");
}

size_t tmpi_absmean_var_scratch_bytes(void) { return 256 + (size_t)kStatBlocks * 2 * sizeof(double); }

// scratch: [counter, 256 B, zero before first use][2 doubles per block]
int tmpi_absmean_var(const void* x, int dtype, size_t n, double* out2, void* scratch, void* stream) {
  unsigned* counter = (unsigned*)scratch;
  double* partial = (double*)((char*)scratch + 256);
  int grid = (int)std::min<size_t>((n + kStatThreads - 1) / kStatThreads, (size_t)kStatBlocks);
  if (grid < 1) grid = 1;
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case TMPI_F32: absstat_kernel<float><<<grid, kStatThreads, 0, s>>>((const float*)x, n, out2, partial, counter); break;
    case TMPI_F64: absstat_kernel<double><<<grid, kStatThreads, 0, s>>>((const double*)x, n, out2, partial, counter); break;
    case TMPI_BF16: absstat_kernel<__nv_bfloat16><<<grid, kStatThreads, 0, s>>>((const __nv_bfloat16*)x, n, out2, partial, counter); break;
    case TMPI_F16: absstat_kernel<__half><<<grid, kStatThreads, 0, s>>>((const __half*)x, n, out2, partial, counter); break;
    default: return fail(TMPI_ERR_UNSUPPORTED, "absmean_var: dtype %d", dtype);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : cuda_fail(e, "absmean_var launch");
}

int tmpi_easgd_elastic(void* local, const void* center, void* delta, size_t n, int dtype, float alpha, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  bool vec = aligned16(local) && aligned16(center) && aligned16(delta);
  DISPATCH_FLOAT(dtype, {
    constexpr int V = 16 / sizeof(T);
    if (vec && n % V == 0) {
      size_t nv = n / V;
      int grid = (int)std::min<size_t>((nv + 255) / 256, (size_t)sm_count() * 8);
      easgd_kernel<T, V><<<grid < 1 ? 1 : grid, 256, 0, s>>>((T*)local, (const T*)center, (T*)delta, nv, alpha);
    } else {
      int grid = (int)std::min<size_t>((n + 255) / 256, (size_t)sm_count() * 8);
      easgd_kernel<T, 1><<<grid < 1 ? 1 : grid, 256, 0, s>>>((T*)local, (const T*)center, (T*)delta, n, alpha);
    }
  });
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : cuda_fail(e, "easgd launch");
}

int tmpi_downpour_accum(void* accum, const void* grad, size_t n, int dtype, float scale, int zero_first, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  bool vec = aligned16(accum) && aligned16(grad);
  DISPATCH_FLOAT(dtype, {
    constexpr int V = 16 / sizeof(T);
    if (vec && n % V == 0) {
      size_t nv = n / V;
      int grid = (int)std::min<size_t>((nv + 255) / 256, (size_t)sm_count() * 8);
      accum_kernel<T, V><<<grid < 1 ? 1 : grid, 256, 0, s>>>((T*)accum, (const T*)grad, nv, scale, zero_first);
    } else {
      int grid = (int)std::min<size_t>((n + 255) / 256, (size_t)sm_count() * 8);
      accum_kernel<T, 1><<<grid < 1 ? 1 : grid, 256, 0, s>>>((T*)accum, (const T*)grad, n, scale, zero_first);
    }
  });
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? TMPI_OK : cuda_fail(e, "downpour launch");
}

}  // extern "C"

// ------------------------------------------------------------------ allocation-free cross-entropy
// See ../include/tmpi_noalloc.h.  The scratch of the cross-entropy kernel (a completion counter
// and one partial loss per row) lives in this file-scope device array instead of a buffer the
// caller would have to allocate.  Every GPU that loads the library carries the array until the
// process exits.  All calls on a device share it, so two calls whose kernels overlap on that
// device race on it; it also keeps the previous call's contents, which is why the counter is
// cleared on the caller's stream before every launch.
#include "../include/tmpi_noalloc.h"
#include <mutex>

namespace tmpi {
namespace {
static __device__ __align__(256) unsigned char g_xent_static_scratch[256 + TMPI_XENT_NOALLOC_MAX_ROWS * sizeof(float)];
constexpr int kMaxDevices = 64;
void* g_xent_static_ptr[kMaxDevices] = {};
std::mutex g_xent_static_mu;

// The array's name in host code is only a handle for the runtime, not a device address: ask for
// the address once per device, with that device current, and hand that pointer to the kernel.
int xent_static_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(TMPI_ERR_UNSUPPORTED, "device index %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lk(g_xent_static_mu);
  if (!g_xent_static_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_xent_static_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(static cross-entropy scratch)");
    g_xent_static_ptr[dev] = p;
  }
  *out = g_xent_static_ptr[dev];
  return TMPI_OK;
}
}  // namespace
}  // namespace tmpi

extern "C" int tmpi_xent_fwd_bwd_noalloc(const void* logits, int dtype, const int64_t* labels, int rows, int cols,
                                         float* loss_sum, void* dlogits, float grad_scale, void* stream) {
  if (rows < 1 || cols < 1) return fail(TMPI_ERR_INVALID, "xent (no-alloc): empty input");
  if (rows > TMPI_XENT_NOALLOC_MAX_ROWS)
    return fail(TMPI_ERR_INVALID, "xent (no-alloc): %d rows exceed the built-in scratch for %d rows; "
                "use tmpi_xent_fwd_bwd with a caller-provided scratch buffer", rows, TMPI_XENT_NOALLOC_MAX_ROWS);
  void* scratch = nullptr;
  int st = xent_static_scratch(&scratch);
  if (st) return st;
  // the completion counter must start at zero whatever an earlier (possibly failed) call left behind
  cudaError_t e = cudaMemsetAsync(scratch, 0, 256, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "clearing the static scratch counter");
  return tmpi_xent_fwd_bwd(logits, dtype, labels, rows, cols, loss_sum, dlogits, grad_scale, scratch, stream);
}
