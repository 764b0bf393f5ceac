// Host front end of the GPU collectives: algorithm choice, staging of tensors
// that live outside the symmetric heap, epoch bookkeeping, asynchronous launch
// on the pool's comm stream.
//
// Size dispatch (reference: small tensors go to stock MPI, large ones to the
// chunked ring, lib/collectives_cuda.cpp:294-307,635-662): up to
// `oneshot_max_bytes` the one-shot push kernel (one barrier, latency bound);
// above it the two-shot kernel, or the NVLS kernel when the heap has a multicast
// mapping, the group is the whole heap and the type is a float type.
#include "cuda_state.h"
#include <algorithm>
#include <cstring>
#include <vector>

namespace tmpi {

#define CK(call)                                          \
  do {                                                    \
    cudaError_t e__ = (call);                             \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

static bool in_heap(const void* p, size_t bytes, size_t* off) {
  CudaHeap& h = heap();
  const char* b = h.base[h.rank];
  const char* q = (const char*)p;
  if (!h.live || h.emulated || q < b || q + bytes > b + h.total_bytes) return false;
  *off = (size_t)(q - b);
  return true;
}

static bool is_float_type(int dt) { return dt == TMPI_F16 || dt == TMPI_BF16 || dt == TMPI_F32; }
static bool whole_heap(const tmpi_group_t* g) { return g->nmembers == heap().world; }
static bool al16(size_t x) { return (x & 15) == 0; }

static int pick_algo(int algo, size_t bytes, int dtype, const tmpi_group_t* g) {
  CudaHeap& h = heap();
  bool nvls_ok = h.mc_base && whole_heap(g) && is_float_type(dtype) && tunable("use_nvls");
  if (algo == 3 && !nvls_ok) algo = 2;
  if (algo != 0) return algo;
  if (bytes <= (size_t)tunable("oneshot_max_bytes") && bytes <= h.slot_bytes) return 1;
  // with two ranks the switch reduction moves more bytes per link than the peer-to-peer two-shot
  if (nvls_ok && g->nmembers > 2 && bytes >= (size_t)tunable("nvls_min_bytes")) return 3;
  return 2;
}

// Launches one collective op for every rank this process drives (1, or all in emulation).
// per_rank(r, me, &args) fills the op-specific fields for heap rank members[me].
template <typename Fill>
static int run_op(int op, int dtype, const tmpi_group_t* g, int vec, size_t items, cudaStream_t s, Fill fill,
                  const char* cta_cap = "comm_max_ctas") {
  CudaHeap& h = heap();
  int threads = (int)tunable("comm_threads");
  if (threads < 32 || threads > 1024) threads = 512;
  int grid = grid_for(items, threads, cta_cap);
  int nb = barriers_used(op, g->nmembers);
  std::lock_guard<std::mutex> lk(h.mu);
  if (h.emulated) {
    std::vector<CollArgs> args(g->nmembers);
    for (int me = 0; me < g->nmembers; ++me) {
      memset(&args[me], 0, sizeof(CollArgs));
      int st = fill_peers(&args[me].P, g->members, g->nmembers, me, g->lane);
      if (st) return st;
      fill(me, &args[me]);
    }
    if (grid * g->nmembers > 256) grid = std::max(1, 256 / g->nmembers);   // keep the cooperative grid resident
    cudaError_t e = launch_collective(op, dtype, args.data(), g->nmembers, vec, grid, threads, s);
    if (e != cudaSuccess) return cuda_fail(e, "collective launch (emulated)");
    for (int me = 0; me < g->nmembers; ++me) advance_epochs(g->members, g->nmembers, me, g->lane, nb);
    return TMPI_OK;
  }
  CollArgs a;
  memset(&a, 0, sizeof(a));
  int st = fill_peers(&a.P, g->members, g->nmembers, g->me, g->lane);
  if (st) return st;
  fill(g->me, &a);
  cudaError_t e = launch_collective(op, dtype, &a, 1, vec, grid, threads, s);
  if (e != cudaSuccess) return cuda_fail(e, "collective launch");
  advance_epochs(g->members, g->nmembers, g->me, g->lane, nb);
  return TMPI_OK;
}

// ---- allreduce on symmetric buffers
static int allreduce_heap(size_t in_off, size_t out_off, size_t n, int dtype, double scale,
                          const tmpi_group_t* g, int algo, cudaStream_t s) {
  CudaHeap& h = heap();
  size_t es = dtype_size(dtype), V = 16 / es;
  bool vec = al16(in_off) && al16(out_off) && n % V == 0;
  algo = pick_algo(algo, n * es, dtype, g);
  if (algo == 3 && !vec) algo = 2;
  if (g->nmembers == 1) algo = 2;
  size_t items = (vec ? n / V : n);
  if (algo == 1 && n * es <= h.slot_bytes) {
    size_t slots = oneshot_slots_off(h, g->lane);
    return run_op(OP_AR_ONESHOT, dtype, g, vec, items, s, [&](int me, CollArgs* a) {
      char* b = h.base[g->members[me]];
      a->in = b + in_off; a->out = b + out_off; a->in_off = slots; a->aux = h.slot_bytes;
      a->n = n; a->scale = (float)scale; a->root = h.world;
    });
  }
  if (algo == 4) {
    if (in_off != out_off) {
      if (h.emulated) return fail(TMPI_ERR_UNSUPPORTED, "ring allreduce is in place");
      CK(cudaMemcpyAsync(h.base[h.rank] + out_off, h.base[h.rank] + in_off, n * es, cudaMemcpyDeviceToDevice, s));
    }
    return run_op(OP_AR_RING, dtype, g, vec, items / g->nmembers + 1, s, [&](int, CollArgs* a) {
      a->out_off = out_off; a->n = n; a->scale = (float)scale;
    });
  }
  int op = algo == 3 ? OP_AR_NVLS : OP_AR_TWOSHOT;
  return run_op(op, dtype, g, vec, items / g->nmembers + 1, s, [&](int, CollArgs* a) {
    a->in_off = in_off; a->out_off = out_off; a->n = n; a->scale = (float)scale;
  }, algo == 3 ? "nvls_max_ctas" : "comm_max_ctas");
}

// ---- allreduce on arbitrary device pointers
static int allreduce_any(const void* in, void* out, size_t n, int dtype, double scale,
                         const tmpi_group_t* g, int algo, cudaStream_t s) {
  CudaHeap& h = heap();
  if (h.emulated) return fail(TMPI_ERR_UNSUPPORTED, "emulated heaps only take heap offsets");
  size_t es = dtype_size(dtype), V = 16 / es, bytes = n * es;
  if (!es) return fail(TMPI_ERR_INVALID, "bad dtype %d", dtype);
  size_t io, oo;
  if (in_heap(in, bytes, &io) && in_heap(out, bytes, &oo)) return allreduce_heap(io, oo, n, dtype, scale, g, algo, s);
  int a = pick_algo(algo, bytes, dtype, g);
  if (a == 1 && bytes <= h.slot_bytes) {
    bool vec = al16((size_t)in) && al16((size_t)out) && n % V == 0;
    size_t slots = oneshot_slots_off(h, g->lane);
    return run_op(OP_AR_ONESHOT, dtype, g, vec, vec ? n / V : n, s, [&](int, CollArgs* ar) {
      ar->in = in; ar->out = out; ar->in_off = slots; ar->aux = h.slot_bytes;
      ar->n = n; ar->scale = (float)scale; ar->root = h.world;
    });
  }
  if (g->lane > 1) return fail(TMPI_ERR_INVALID, "lane %d has no bounce buffer", g->lane);
  size_t boff = bounce_off(h, g->lane);
  // use_staged_collectives (the reference's knob for its staged ring): always copy in, reduce in the heap, copy out
  if ((a == 2 || a == 1) && !tunable("use_staged_collectives")) {
    // two-shot straight from / to the caller's tensors: the bounce region is only scratch
    // (R slots + one result slice per chunk), no copy kernels around the collective
    const int R = g->nmembers;
    bool vec = al16((size_t)in) && al16((size_t)out) && n % V == 0;
    const size_t W = vec ? V : 1;                                  // elements per pack
    size_t per_max = h.bounce_bytes / ((size_t)(R + 1) * W * es);  // packs per slot that fit
    per_max = per_max / 16 * 16;                                   // keep slot starts 16-pack aligned
    if (per_max == 0) return fail(TMPI_ERR_STATE, "staging_bytes too small for a %d-rank two-shot", R);
    const size_t chunk = per_max * R * W;                          // elements per launch
    for (size_t off = 0; off < n; off += chunk) {
      const size_t m = std::min(chunk, n - off);
      const size_t per = ((m / W) + R - 1) / R;
      int st = run_op(OP_AR_TWOSHOT_ANY, dtype, g, vec, per, s, [&](int, CollArgs* ar) {
        ar->in = (const char*)in + off * es; ar->out = (char*)out + off * es;
        ar->in_off = boff; ar->out_off = boff + (size_t)R * per * W * es;
        ar->n = m; ar->scale = (float)scale;
      });
      if (st) return st;
    }
    return TMPI_OK;
  }
  // NVLS and ring keep the symmetric kernels: bounce through the heap in chunks (copy in, reduce, copy out)
  size_t chunk = h.bounce_bytes / es / (V * g->nmembers) * (V * g->nmembers);
  for (size_t off = 0; off < n; off += chunk) {
    size_t m = std::min(chunk, n - off);
    size_t padded = (m + V * g->nmembers - 1) / (V * g->nmembers) * (V * g->nmembers);
    CK(cudaMemcpyAsync(h.base[h.rank] + boff, (const char*)in + off * es, m * es, cudaMemcpyDeviceToDevice, s));
    int st = allreduce_heap(boff, boff, padded, dtype, scale, g, a == 1 ? 2 : a, s);
    if (st) return st;
    CK(cudaMemcpyAsync((char*)out + off * es, h.base[h.rank] + boff, m * es, cudaMemcpyDeviceToDevice, s));
  }
  return TMPI_OK;
}

// ---- broadcast
static int broadcast_heap(size_t off, size_t n, int dtype, int root, const tmpi_group_t* g, int algo, cudaStream_t s) {
  CudaHeap& h = heap();
  size_t bytes = n * dtype_size(dtype);
  bool vec = al16(off) && bytes % 16 == 0;
  size_t items = vec ? bytes / 16 : bytes;
  int op = OP_BCAST_PULL;
  // with two ranks a multicast store also sends the data back to the root: the pull is faster there
  bool mc_ok = h.mc_base && whole_heap(g) && vec && tunable("use_nvls");
  const bool mc_auto = mc_ok && g->nmembers > 2;
  // 0 auto, 1 pull, 2 chunked, 3 multicast store from the root, 4 scatter by peer loads + multicast stores by everyone,
  // 5 scatter by peer loads + plain stores into the other members (any heap backend)
  if (algo == 0) algo = (int)tunable("broadcast_algo");
  if (algo == 3 && mc_ok) op = OP_BCAST_MC;
  else if (algo == 4 && mc_ok) op = OP_BCAST_SCATTER_MC;
  else if (algo == 5 && g->nmembers > 2) op = OP_BCAST_SCATTER_PUSH;
  else if (algo == 2) op = OP_BCAST_CHUNKED;
  else if (algo == 0) {
    // large: scatter + push in one pass (measured ahead of the multicast variants and of NCCL on 4 GPUs from 16 MiB)
    if (g->nmembers > 2 && vec && bytes >= (size_t)tunable("bcast_scatter_min_bytes")) op = OP_BCAST_SCATTER_PUSH;
    else if (mc_auto && bytes >= (size_t)tunable("nvls_min_bytes")) op = OP_BCAST_MC;
    else if (bytes > (size_t)tunable("broadcast_size_gpu_tree_based") && g->nmembers > 2) op = OP_BCAST_CHUNKED;
  }
  return run_op(op, TMPI_U8, g, vec, items, s, [&](int, CollArgs* a) {
    a->out_off = off; a->n = bytes; a->root = root;
  }, op == OP_BCAST_MC ? "bcast_max_ctas" : (op == OP_BCAST_SCATTER_MC || op == OP_BCAST_SCATTER_PUSH) ? "bcast_scatter_max_ctas" : "comm_max_ctas");
}

static int broadcast_any(void* buf, size_t n, int dtype, int root, const tmpi_group_t* g, cudaStream_t s) {
  CudaHeap& h = heap();
  if (h.emulated) return fail(TMPI_ERR_UNSUPPORTED, "emulated heaps only take heap offsets");
  size_t es = dtype_size(dtype), bytes = n * es, off;
  if (in_heap(buf, bytes, &off)) return broadcast_heap(off, n, dtype, root, g, 0, s);
  if (g->lane > 1) return fail(TMPI_ERR_INVALID, "lane %d has no bounce buffer", g->lane);
  // the root pushes straight from its tensor into every peer's scratch; the peers copy out inside
  // the same kernel (no copy kernels around the collective)
  size_t boff = bounce_off(h, g->lane);
  size_t chunk = h.bounce_bytes & ~size_t(15);
  const bool mc = h.mc_base && whole_heap(g) && g->nmembers > 2 && tunable("use_nvls");
  for (size_t o = 0; o < bytes; o += chunk) {
    size_t m = std::min(chunk, bytes - o);
    char* p = (char*)buf + o;
    bool vec = al16((size_t)p) && m % 16 == 0;
    int st = run_op(OP_BCAST_ANY, TMPI_U8, g, vec, vec ? m / 16 : m, s, [&](int, CollArgs* a) {
      a->out = p; a->in_off = boff; a->n = m; a->root = root; a->aux = (mc && vec) ? 1 : 0;
    });
    if (st) return st;
  }
  return TMPI_OK;
}

// ---- ops with a symmetric source and a local destination: reduce, allgather(v), reduce_scatter
static int stage_in(const void* in, size_t bytes, const tmpi_group_t* g, cudaStream_t s, size_t* off) {
  CudaHeap& h = heap();
  if (in_heap(in, bytes, off)) return TMPI_OK;
  if (g->lane > 1) return fail(TMPI_ERR_INVALID, "lane %d has no bounce buffer", g->lane);
  if (bytes > h.bounce_bytes) return -1;   // caller chunks
  *off = bounce_off(h, g->lane);
  CK(cudaMemcpyAsync(h.base[h.rank] + *off, in, bytes, cudaMemcpyDeviceToDevice, s));
  return TMPI_OK;
}

}  // namespace tmpi

using namespace tmpi;

static int check_group(const tmpi_group_t* g) {
  if (!heap().live) return fail(TMPI_ERR_STATE, "CUDA heap not created");
  if (!g || !g->members || g->nmembers < 1) return fail(TMPI_ERR_INVALID, "missing group");
  return TMPI_OK;
}

extern "C" {

int tmpi_cuda_allreduce(const void* in, void* out, size_t n, int dtype, double scale,
                        const tmpi_group_t* g, int algo, void* stream) {
  int st = check_group(g);
  return st ? st : allreduce_any(in, out, n, dtype, scale, g, algo, (cudaStream_t)stream);
}

int tmpi_cuda_allreduce_heap(size_t in_off, size_t out_off, size_t n, int dtype, double scale,
                             const tmpi_group_t* g, int algo, void* stream) {
  int st = check_group(g);
  return st ? st : allreduce_heap(in_off, out_off, n, dtype, scale, g, algo, (cudaStream_t)stream);
}

int tmpi_cuda_broadcast(void* buf, size_t n, int dtype, int root, const tmpi_group_t* g, void* stream) {
  int st = check_group(g);
  if (st) return st;
  if (root < 0 || root >= g->nmembers) return fail(TMPI_ERR_INVALID, "bad root %d", root);
  return broadcast_any(buf, n, dtype, root, g, (cudaStream_t)stream);
}

int tmpi_cuda_broadcast_heap(size_t off, size_t n, int dtype, int root, const tmpi_group_t* g, int algo, void* stream) {
  int st = check_group(g);
  if (st) return st;
  if (root < 0 || root >= g->nmembers) return fail(TMPI_ERR_INVALID, "bad root %d", root);
  return broadcast_heap(off, n, dtype, root, g, algo, (cudaStream_t)stream);
}

// out is only written at the root.  Inputs larger than the bounce buffer are processed in chunks.
int tmpi_cuda_reduce(const void* in, void* out, size_t n, int dtype, int root, const tmpi_group_t* g, void* stream) {
  int st = check_group(g);
  if (st) return st;
  CudaHeap& h = heap();
  cudaStream_t s = (cudaStream_t)stream;
  size_t es = dtype_size(dtype), V = 16 / es;
  size_t chunk = h.bounce_bytes / es / V * V;
  size_t whole = 0;
  bool direct = h.emulated || in_heap(in, n * es, &whole);
  if (h.emulated) whole = (size_t)in;              // emulation: `in` and `out` are heap offsets
  for (size_t o = 0; o < n; o += direct ? n : chunk) {
    size_t m = direct ? n : std::min(chunk, n - o);
    size_t off = whole;
    if (!direct && (st = stage_in((const char*)in + o * es, m * es, g, s, &off))) return st;
    char* dst = h.emulated ? (char*)out : (char*)out + o * es;
    bool vec = al16(off) && al16((size_t)dst) && m % V == 0;
    // with a multicast mapping the root lets the switch do the sum (bf16 / f16 / f32, whole heap, large enough)
    const bool nvls = vec && h.mc_base && whole_heap(g) && g->nmembers > 2 && tunable("use_nvls") &&
                      (dtype == TMPI_BF16 || dtype == TMPI_F16 || dtype == TMPI_F32) &&
                      m * es >= (size_t)tunable("nvls_min_bytes");
    st = run_op(OP_REDUCE, dtype, g, vec, vec ? m / V : m, s, [&](int me, CollArgs* a) {
      a->in_off = off; a->out = h.emulated ? (void*)(h.base[g->members[me]] + (size_t)out) : (void*)dst;
      a->n = m; a->scale = 1.f; a->root = root; a->aux = nvls ? 1 : 0;
    }, nvls ? "nvls_max_ctas" : "comm_max_ctas");
    if (st) return st;
  }
  return TMPI_OK;
}

int tmpi_cuda_allgatherv(const void* in, void* out, size_t n_in, const int64_t* counts, int dtype,
                         const tmpi_group_t* g, void* stream) {
  int st = check_group(g);
  if (st) return st;
  CudaHeap& h = heap();
  cudaStream_t s = (cudaStream_t)stream;
  size_t es = dtype_size(dtype);
  std::vector<size_t> bytes(g->nmembers);
  size_t maxb = 0, prefix = 0;
  bool vec = al16((size_t)out);
  for (int i = 0; i < g->nmembers; ++i) {
    bytes[i] = (counts ? (size_t)counts[i] : n_in) * es;
    maxb = std::max(maxb, bytes[i]);
    if (bytes[i] % 16 || prefix % 16) vec = false;   // every chunk must start and end on 16 bytes
    prefix += bytes[i];
  }
  if (!h.emulated && bytes[g->me] != n_in * es) return fail(TMPI_ERR_INVALID, "counts[me] != n_in");
  size_t off = 0;
  if (h.emulated) {
    off = (size_t)in;                                // emulation: `in` and `out` are heap offsets
  } else if (!in_heap(in, n_in * es, &off)) {
    if (maxb > h.bounce_bytes)
      return fail(TMPI_ERR_UNSUPPORTED, "allgather chunk of %zu bytes exceeds the bounce buffer (%zu); "
                  "place it in the symmetric heap or raise staging_bytes", maxb, h.bounce_bytes);
    if ((st = stage_in(in, n_in * es, g, s, &off))) return st;
  }
  if (!al16(off)) vec = false;
  return run_op(OP_ALLGATHER, TMPI_U8, g, vec, maxb / (vec ? 16 : 1) + 1, s, [&](int me, CollArgs* a) {
    a->in_off = off;
    a->out = h.emulated ? (void*)(h.base[g->members[me]] + (size_t)out) : out;
    for (int i = 0; i < g->nmembers; ++i) a->cnt[i] = bytes[i];
  });
}

int tmpi_cuda_allgather(const void* in, void* out, size_t n_in, int dtype, const tmpi_group_t* g, void* stream) {
  return tmpi_cuda_allgatherv(in, out, n_in, nullptr, dtype, g, stream);
}

int tmpi_cuda_reduce_scatter(const void* in, void* out, size_t n_out, int dtype, double scale,
                             const tmpi_group_t* g, void* stream) {
  int st = check_group(g);
  if (st) return st;
  CudaHeap& h = heap();
  cudaStream_t s = (cudaStream_t)stream;
  size_t es = dtype_size(dtype), V = 16 / es, total = n_out * g->nmembers;
  size_t off = 0;
  if (h.emulated) off = (size_t)in;
  else if (!in_heap(in, total * es, &off)) {
    if (total * es > h.bounce_bytes)
      return fail(TMPI_ERR_UNSUPPORTED, "reduce_scatter input of %zu bytes exceeds the bounce buffer (%zu); "
                  "place it in the symmetric heap or raise staging_bytes", total * es, h.bounce_bytes);
    if ((st = stage_in(in, total * es, g, s, &off))) return st;
  }
  bool vec = al16(off) && al16((size_t)out) && n_out % V == 0;
  return run_op(OP_REDUCE_SCATTER, dtype, g, vec, vec ? n_out / V : n_out, s, [&](int me, CollArgs* a) {
    a->in_off = off; a->out = h.emulated ? (void*)(h.base[g->members[me]] + (size_t)out) : out;
    a->n = n_out; a->scale = (float)scale;
  });
}

int tmpi_cuda_barrier(const tmpi_group_t* g, void* stream) {
  int st = check_group(g);
  return st ? st : run_op(OP_BARRIER, TMPI_U8, g, 0, 1, (cudaStream_t)stream, [](int, CollArgs*) {});
}

int tmpi_cuda_test_wait_timeout(int64_t budget_ms, void* stream) {
  CudaHeap& h = heap();
  if (!h.live) return fail(TMPI_ERR_STATE, "CUDA heap not created");
  int members[1] = {h.emulated ? 0 : h.rank};
  Peers P;
  int st = fill_peers(&P, members, 1, 0, LANE_SYNC);
  if (st) return st;
  P.budget_ns = (unsigned long long)budget_ms * 1000000ull;
  cudaError_t e = launch_wait_probe(P, (cudaStream_t)stream);
  if (e != cudaSuccess) return cuda_fail(e, "wait probe");
  CK(cudaStreamSynchronize((cudaStream_t)stream));
  int code, where, peer;
  tmpi_cuda_collective_status(LANE_SYNC, &code, &where, &peer);
  return code;   // 3 == timeout reported by the device, context still usable
}

}  // extern "C"
