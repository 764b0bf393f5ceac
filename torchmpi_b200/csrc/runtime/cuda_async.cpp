// Asynchronous collectives, the fused allreduce+SGD entry point and the GPU
// parameter-server client calls.
//
// Asynchronous flavour: the caller's stream records an event, an ordered pool
// thread makes the lane's own high-priority stream wait for it, launches the
// collective there and records a completion event into the handle.  The caller
// goes on enqueueing compute; `wait` (host) or `stream_wait` (device) joins.
// This is the role of the reference's collective offload pool and its
// high-priority streams (lib/collectives_cuda.cpp:771-803,
// lib/resources.cpp:1055-1094), with one in-order worker per lane so that the
// kernels that wait on one another are launched in the same order on every rank.
#include "cuda_state.h"
#include <cstring>
#include <vector>

namespace tmpi {

#define CK(call)                                          \
  do {                                                    \
    cudaError_t e__ = (call);                             \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

struct GroupCopy {
  std::vector<int> members;
  tmpi_group_t g;
  explicit GroupCopy(const tmpi_group_t* src, int lane) : members(src->members, src->members + src->nmembers) {
    g.members = members.data(); g.nmembers = src->nmembers; g.me = src->me; g.lane = lane;
  }
  GroupCopy(const GroupCopy& o) : members(o.members), g(o.g) { g.members = members.data(); }
};

template <typename Fn>
static uint64_t launch_async(void* user_stream, int lane, Fn fn) {
  CudaHeap& h = heap();
  if (!h.live) return make_ready_handle(fail(TMPI_ERR_STATE, "CUDA heap not created"));
  cudaEvent_t ready = nullptr;
  if (cudaEventCreateWithFlags(&ready, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventRecord(ready, (cudaStream_t)user_stream) != cudaSuccess)
    return make_ready_handle(fail(TMPI_ERR_CUDA, "could not record the producer event"));
  int device = h.device;
  cudaStream_t ls = h.lane_stream[lane];
  return submit_ordered(lane, [=]() -> int {
    cudaSetDevice(device);
    cudaError_t e = cudaStreamWaitEvent(ls, ready, 0);
    cudaEventDestroy(ready);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamWaitEvent");
    int st = fn(ls);
    if (st) return st;
    cudaEvent_t done = nullptr;
    CK(cudaEventCreateWithFlags(&done, cudaEventDisableTiming));
    CK(cudaEventRecord(done, ls));
    handle_set_event(0, done);
    return TMPI_OK;
  });
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

uint64_t tmpi_cuda_allreduce_async(const void* in, void* out, size_t n, int dtype, double scale,
                                   const tmpi_group_t* g, int algo, void* stream) {
  GroupCopy gc(g, LANE_ASYNC);
  return launch_async(stream, LANE_ASYNC, [=](cudaStream_t ls) {
    return tmpi_cuda_allreduce(in, out, n, dtype, scale, &gc.g, algo, ls);
  });
}

uint64_t tmpi_cuda_broadcast_async(void* buf, size_t n, int dtype, int root, const tmpi_group_t* g, void* stream) {
  GroupCopy gc(g, LANE_ASYNC);
  return launch_async(stream, LANE_ASYNC, [=](cudaStream_t ls) {
    return tmpi_cuda_broadcast(buf, n, dtype, root, &gc.g, ls);
  });
}

// Fused allreduce + SGD over one bucket.  In emulation `master` / `momentum` hold the shards of
// all ranks back to back (shard r at r * n / nmembers).
int tmpi_cuda_allreduce_sgd(const tmpi_sgd_bucket_t* b, const tmpi_group_t* g, int algo, void* stream) {
  CudaHeap& h = heap();
  if (!h.live) return fail(TMPI_ERR_STATE, "CUDA heap not created");
  const int N = g->nmembers;
  size_t es = dtype_size(b->grad_dtype), V = 16 / es;
  if (b->n % (V * N)) return fail(TMPI_ERR_INVALID, "bucket of %zu elements is not a multiple of %zu", b->n, V * N);
  if ((b->grad_off & 15) || (b->weight_off & 15)) return fail(TMPI_ERR_INVALID, "bucket offsets must be 16-byte aligned");
  bool nvls = h.mc_base && N == h.world && N > 1 && tunable("use_nvls") && (algo == 3 || (algo == 0 &&
              b->n * es >= (size_t)tunable("nvls_min_bytes")));
  int threads = 512;
  int grid = grid_for(b->n / V / N, threads, "opt_max_ctas");
  std::lock_guard<std::mutex> lk(h.mu);
  auto fill = [&](int me, SgdArgs* a) -> int {
    memset(a, 0, sizeof(*a));
    int st = fill_peers(&a->P, g->members, N, me, g->lane);
    if (st) return st;
    size_t shard = b->n / N;
    a->grad_off = b->grad_off; a->weight_off = b->weight_off; a->n = b->n;
    a->master = b->master ? (float*)b->master + (h.emulated ? shard * me : 0) : nullptr;
    a->momentum = b->momentum ? (float*)b->momentum + (h.emulated ? shard * me : 0) : nullptr;
    a->lr = b->lr; a->momentum_coef = b->momentum_coef; a->dampening = b->dampening;
    a->weight_decay = b->weight_decay; a->grad_scale = b->grad_scale;
    a->nesterov = b->nesterov; a->first_step = b->first_step; a->zero_grads = b->zero_grads;
    a->use_nvls = nvls ? 1 : 0;
    return TMPI_OK;
  };
  int nb = sgd_barriers_used(N);
  if (h.emulated) {
    std::vector<SgdArgs> args(N);
    for (int me = 0; me < N; ++me) { int st = fill(me, &args[me]); if (st) return st; }
    if (grid * N > 256) grid = std::max(1, 256 / N);
    cudaError_t e = launch_allreduce_sgd(b->grad_dtype, b->weight_dtype, args.data(), N, grid, threads, (cudaStream_t)stream);
    if (e != cudaSuccess) return cuda_fail(e, "allreduce_sgd launch (emulated)");
    for (int me = 0; me < N; ++me) advance_epochs(g->members, N, me, g->lane, nb);
    return TMPI_OK;
  }
  SgdArgs a;
  int st = fill(g->me, &a);
  if (st) return st;
  cudaError_t e = launch_allreduce_sgd(b->grad_dtype, b->weight_dtype, &a, 1, grid, threads, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "allreduce_sgd launch");
  advance_epochs(g->members, N, g->me, g->lane, nb);
  return TMPI_OK;
}

static int ps_launch(size_t shard_off, void* data, size_t n, int dtype, int rule, const tmpi_group_t* g, void* stream) {
  CudaHeap& h = heap();
  if (!h.live) return fail(TMPI_ERR_STATE, "CUDA heap not created");
  PsArgs a;
  memset(&a, 0, sizeof(a));
  {
    std::lock_guard<std::mutex> lk(h.mu);
    int st = fill_peers(&a.P, g->members, g->nmembers, g->me, LANE_PS);
    if (st) return st;
  }
  a.shard_off = shard_off; a.data = data; a.n = n; a.rule = rule;
  int grid = grid_for(n / g->nmembers + 1, 512, "ps_max_ctas");
  cudaError_t e = launch_ps(dtype, &a, grid, 512, (cudaStream_t)stream);
  return e == cudaSuccess ? TMPI_OK : cuda_fail(e, "parameter-server kernel launch");
}

int tmpi_cuda_ps_push(size_t shard_off, const void* data, size_t n, int dtype, int rule,
                      const tmpi_group_t* g, void* stream) {
  if (rule < 0 || rule > 2) return fail(TMPI_ERR_INVALID, "unknown update rule %d", rule);
  return ps_launch(shard_off, const_cast<void*>(data), n, dtype, rule, g, stream);
}

int tmpi_cuda_ps_pull(size_t shard_off, void* data, size_t n, int dtype, const tmpi_group_t* g, void* stream) {
  return ps_launch(shard_off, data, n, dtype, -1, g, stream);
}

// Asynchronous client requests: served by the parameter-server pool, which owns the PS stream.
uint64_t tmpi_cuda_ps_push_async(size_t shard_off, const void* data, size_t n, int dtype, int rule,
                                 const tmpi_group_t* g, void* stream) {
  GroupCopy gc(g, LANE_PS);
  return launch_async(stream, LANE_PS, [=](cudaStream_t ls) {
    return tmpi_cuda_ps_push(shard_off, data, n, dtype, rule, &gc.g, ls);
  });
}

uint64_t tmpi_cuda_ps_pull_async(size_t shard_off, void* data, size_t n, int dtype,
                                 const tmpi_group_t* g, void* stream) {
  GroupCopy gc(g, LANE_PS);
  return launch_async(stream, LANE_PS, [=](cudaStream_t ls) {
    return tmpi_cuda_ps_pull(shard_off, data, n, dtype, &gc.g, ls);
  });
}

}  // extern "C"
