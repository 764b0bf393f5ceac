// Fused gradient allreduce + SGD(momentum) step over one flat bucket.
//
// One kernel per bucket does what the reference spreads over an allreduce per
// parameter tensor (torchmpi/nn.lua:49-56) and torchnet's per-tensor
// `w:add(-lr, gw)` update: each rank owns 1/N of the bucket, sums that shard of
// the gradients straight out of every peer's memory (or through the switch with
// multimem.ld_reduce), applies scale, weight decay, momentum and the update to
// its fp32 master shard, and stores the new low-precision weights into every
// peer's weight bucket (or multimem.st).  Optimizer state therefore exists once
// per element in the job, NVLink carries gradients in and weights out (the same
// bytes as an allreduce), and every replica receives the same bits because a
// single rank computes each element.  After the closing barrier a rank clears
// its own gradient bucket, so no separate zero_grad pass is needed either.
// With one rank the kernel is a plain fused SGD step.
#include "collectives.cuh"
#include "../include/tmpi_c_api.h"

namespace tmpi {

int sgd_barriers_used(int n) { return n > 1 ? 2 : 0; }

template <typename T, int V>
__device__ __forceinline__ void load_f32(const float* p, float (&x)[V]) {
#pragma unroll
  for (int i = 0; i < V; i += 4) {
    float4 f = *reinterpret_cast<const float4*>(p + i);
    x[i] = f.x; x[i + 1] = f.y; x[i + 2] = f.z; x[i + 3] = f.w;
  }
}
template <int V>
__device__ __forceinline__ void store_f32(float* p, const float (&x)[V]) {
#pragma unroll
  for (int i = 0; i < V; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
}

template <typename T, int V>
__device__ void body_ar_sgd(const SgdArgs& a, int* s_abort) {
  const Peers& P = a.P;
  const int N = P.n;
  const size_t nv = a.n / V;
  const size_t per = nv / N;               // the host pads buckets to a multiple of V * N
  const size_t lo = per * P.me, hi = lo + per;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t t0 = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (N > 1 && !peer_barrier(P, 1, 100, s_abort)) return;

  for (size_t i = lo + t0; i < hi; i += stride) {
    float g[V];
    if (a.use_nvls && Multimem<T>::ok) {
      uint4 u = Multimem<T>::ld_reduce(at<T>(P.mc_base, a.grad_off) + i * V);
      Pack<T, V> x = *reinterpret_cast<Pack<T, V>*>(&u);
#pragma unroll
      for (int k = 0; k < V; ++k) g[k] = (float)to_acc<T>(x.v[k]);
    } else {
      Pack<T, V> x[kMaxPeers > 8 ? 8 : kMaxPeers];
      if (N <= 8) {
#pragma unroll
        for (int m = 0; m < 8; ++m)
          if (m < N) x[m] = ld_pack_peer<T, V>(at<T>(P.base[m], a.grad_off) + i * V);
#pragma unroll
        for (int k = 0; k < V; ++k) g[k] = (float)to_acc<T>(x[0].v[k]);
#pragma unroll
        for (int m = 1; m < 8; ++m)
          if (m < N) {
#pragma unroll
            for (int k = 0; k < V; ++k) g[k] += (float)to_acc<T>(x[m].v[k]);
          }
      } else {
        for (int m = 0; m < N; ++m) {
          Pack<T, V> y = ld_pack_peer<T, V>(at<T>(P.base[m], a.grad_off) + i * V);
#pragma unroll
          for (int k = 0; k < V; ++k) g[k] = (m == 0 ? 0.f : g[k]) + (float)to_acc<T>(y.v[k]);
        }
      }
    }
    const size_t li = (i - lo) * V;      // index into this rank's fp32 shards
    float w[V];
    if (a.master) {
      load_f32<T, V>(a.master + li, w);
    } else {
      Pack<T, V> x = ld_pack<T, V>(at<T>(P.base[P.me], a.weight_off) + i * V);
#pragma unroll
      for (int k = 0; k < V; ++k) w[k] = (float)to_acc<T>(x.v[k]);
    }
    float mom[V];
    if (a.momentum && !a.first_step) load_f32<T, V>(a.momentum + li, mom);
    Pack<T, V> wout;
#pragma unroll
    for (int k = 0; k < V; ++k) {
      float gg = g[k] * a.grad_scale;
      if (a.weight_decay != 0.f) gg += a.weight_decay * w[k];
      if (a.momentum) {
        mom[k] = a.first_step ? gg : a.momentum_coef * mom[k] + (1.f - a.dampening) * gg;
        gg = a.nesterov ? gg + a.momentum_coef * mom[k] : mom[k];
      }
      w[k] -= a.lr * gg;
      wout.v[k] = from_acc<T>((typename AccOf<T>::type)w[k]);
    }
    if (a.master) store_f32<V>(a.master + li, w);
    if (a.momentum) store_f32<V>(a.momentum + li, mom);
    if (a.use_nvls && Multimem<T>::ok) {
      multimem_st(at<T>(P.mc_base, a.weight_off) + i * V, *reinterpret_cast<uint4*>(&wout));
    } else {
      for (int m = 0; m < N; ++m) st_pack_peer<T, V>(at<T>(P.base[m], a.weight_off) + i * V, wout);
    }
  }

  if (N > 1 && !peer_barrier(P, 2, 101, s_abort)) return;
  if (a.zero_grads) {
    // every peer's block b has read the parts of my gradients that my block b now clears
    Pack<T, V> z;
#pragma unroll
    for (int k = 0; k < V; ++k) z.v[k] = from_acc<T>((typename AccOf<T>::type)0);
    T* gmine = at<T>(P.base[P.me], a.grad_off);
    for (int s = 0; s < N; ++s)
      for (size_t i = per * s + t0; i < per * (s + 1); i += stride) st_pack<T, V>(gmine + i * V, z);
  }
}

template <typename T, int V>
__global__ void __launch_bounds__(512) ar_sgd_kernel(const __grid_constant__ SgdArgs a) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  TMPI_DBG_ENTER(a.P, nullptr, 0, nullptr, 0);
  __syncthreads();
  body_ar_sgd<T, V>(a, &s_abort);
}

template <typename T, int V>
__global__ void __launch_bounds__(512) ar_sgd_kernel_emu(const __grid_constant__ SgdArgsPack pack) {
  __shared__ int s_abort;
  if (threadIdx.x == 0) s_abort = 0;
  TMPI_DBG_ENTER(pack.r[blockIdx.y].P, nullptr, 0, nullptr, 0);
  __syncthreads();
  body_ar_sgd<T, V>(pack.r[blockIdx.y], &s_abort);
}

template <typename T, int V>
cudaError_t launch_sgd_typed(const SgdArgs* args, int nranks, int grid, int threads, cudaStream_t s) {
  if (nranks == 1) {
    ar_sgd_kernel<T, V><<<grid, threads, 0, s>>>(args[0]);
    return cudaGetLastError();
  }
  SgdArgsPack pack;
  for (int r = 0; r < nranks && r < 8; ++r) pack.r[r] = args[r];
  void* params[] = {&pack};
  return cudaLaunchCooperativeKernel((void*)ar_sgd_kernel_emu<T, V>, dim3(grid, nranks), dim3(threads), params, 0, s);
}

cudaError_t launch_allreduce_sgd(int gdt, int wdt, const SgdArgs* args, int nranks, int grid, int threads,
                                 cudaStream_t s) {
  if (gdt != wdt) return cudaErrorInvalidValue;
  if (grid < 1) grid = 1;
  if (grid > kMaxBlocks) grid = kMaxBlocks;
  if (threads > 512) threads = 512;
  switch (gdt) {
    case TMPI_BF16: return launch_sgd_typed<__nv_bfloat16, 8>(args, nranks, grid, threads, s);
    case TMPI_F16: return launch_sgd_typed<__half, 8>(args, nranks, grid, threads, s);
    case TMPI_F32: return launch_sgd_typed<float, 4>(args, nranks, grid, threads, s);
  }
  return cudaErrorInvalidValue;
}

}  // namespace tmpi
