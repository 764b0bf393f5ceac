// Host symmetric heap over POSIX shared memory, and the one-sided CPU
// collectives that run on it.
//
// CPU ranks of one host each create one segment and map every peer's.  The
// collectives are the host twins of the GPU kernels (one-shot, two-shot and
// ring allreduce, pull broadcast, root reduce, all-gather): a rank copies its
// input into its own segment, signals, and reads the peers' segments directly.
// They replace the reference's MPI point-to-point ring / tree
// (lib/detail/collectives.cpp:27-326) for ranks that share a host, and serve
// as the executable model of the flag protocol the GPU kernels use.
//
// Signalling: segment r holds one counter per writer w (`sig[w]`), bumped by w
// with release order; r counts what it has consumed from w.  Because every
// collective that involves a pair of ranks is issued in the same order on both
// (all of them run on one ordered lane), the counters never need resetting.
// Every wait is bounded by the host_wait_budget_ms tunable.
#include "common.h"
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <atomic>
#include <chrono>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tmpi {
namespace {

constexpr int kMaxWorld = 64;
constexpr size_t kHeaderBytes = 4096;

struct Header {
  std::atomic<uint32_t> sig[kMaxWorld];   // sig[w]: signals received from writer w
  std::atomic<uint32_t> magic;
};
static_assert(sizeof(Header) <= kHeaderBytes, "header too large");

struct Heap {
  bool live = false;
  int rank = 0, world = 1;
  size_t seg_bytes = 0;       // whole segment
  size_t stage_bytes = 0;     // each of the two staging regions
  size_t arena_bytes = 0;     // parameter-server arena
  std::string my_name;
  char* base[kMaxWorld] = {};
  uint32_t consumed[kMaxWorld] = {};
  size_t arena_used = 0;
};
Heap H;
std::mutex g_mu;  // protects create/attach/destroy and the arena

Header* hdr(int r) { return reinterpret_cast<Header*>(H.base[r]); }
char* stageA(int r) { return H.base[r] + kHeaderBytes; }
char* stageB(int r) { return H.base[r] + kHeaderBytes + H.stage_bytes; }
char* arena(int r) { return H.base[r] + kHeaderBytes + 2 * H.stage_bytes; }

using Clock = std::chrono::steady_clock;

inline void spin_pause(int iter) {
  if (iter < 64) return;
  if (iter < 4096) { std::this_thread::yield(); return; }
  std::this_thread::sleep_for(std::chrono::microseconds(50));
}

// signal every other member, then wait for a signal from each
int group_barrier(const int* members, int n, int me, int64_t timeout_ms) {
  if (n <= 1) return TMPI_OK;
  int my = members[me];
  for (int i = 0; i < n; ++i) {
    if (i == me) continue;
    hdr(members[i])->sig[my].fetch_add(1, std::memory_order_release);
  }
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  for (int i = 0; i < n; ++i) {
    if (i == me) continue;
    int p = members[i];
    uint32_t want = ++H.consumed[p];
    int iter = 0;
    while ((int32_t)(hdr(my)->sig[p].load(std::memory_order_acquire) - want) < 0) {
      spin_pause(iter++);
      if ((iter & 1023) == 0 && Clock::now() > deadline) {
        --H.consumed[p];
        return fail(TMPI_ERR_TIMEOUT, "shm barrier: rank %d never heard from rank %d within %lld ms",
                    my, p, (long long)timeout_ms);
      }
    }
  }
  return TMPI_OK;
}

int64_t budget() { return tunable("host_wait_budget_ms"); }

// ---- typed helpers
template <typename T> inline double to_acc(T v) { return (double)v; }
template <> inline double to_acc<__nv_bfloat16>(__nv_bfloat16 v) { return (double)__bfloat162float(v); }
template <> inline double to_acc<__half>(__half v) { return (double)__half2float(v); }
template <typename T> inline T from_acc(double v) { return (T)v; }
template <> inline __nv_bfloat16 from_acc<__nv_bfloat16>(double v) { return __float2bfloat16((float)v); }
template <> inline __half from_acc<__half>(double v) { return __float2half((float)v); }

// dst[i] = scale * sum_k srcs[k][i]; float types accumulate in the next wider type
template <typename T, typename Acc>
void sum_into(T* dst, const T* const* srcs, int nsrc, size_t n, double scale) {
  for (size_t i = 0; i < n; ++i) {
    Acc a = (Acc)to_acc<T>(srcs[0][i]);
    for (int k = 1; k < nsrc; ++k) a += (Acc)to_acc<T>(srcs[k][i]);
    if (scale != 1.0) a = (Acc)(a * scale);
    dst[i] = from_acc<T>((double)a);
  }
}
template <typename T>
void sum_into_int(T* dst, const T* const* srcs, int nsrc, size_t n, double scale) {
  for (size_t i = 0; i < n; ++i) {
    T a = srcs[0][i];
    for (int k = 1; k < nsrc; ++k) a = (T)(a + srcs[k][i]);
    if (scale != 1.0) a = (T)((double)a * scale);
    dst[i] = a;
  }
}

void typed_sum(int dtype, void* dst, const void* const* srcs, int nsrc, size_t n, double scale) {
  switch (dtype) {
    case TMPI_U8: sum_into_int<uint8_t>((uint8_t*)dst, (const uint8_t* const*)srcs, nsrc, n, scale); break;
    case TMPI_I8: sum_into_int<int8_t>((int8_t*)dst, (const int8_t* const*)srcs, nsrc, n, scale); break;
    case TMPI_I16: sum_into_int<int16_t>((int16_t*)dst, (const int16_t* const*)srcs, nsrc, n, scale); break;
    case TMPI_I32: sum_into_int<int32_t>((int32_t*)dst, (const int32_t* const*)srcs, nsrc, n, scale); break;
    case TMPI_I64: sum_into_int<int64_t>((int64_t*)dst, (const int64_t* const*)srcs, nsrc, n, scale); break;
    case TMPI_F16: sum_into<__half, float>((__half*)dst, (const __half* const*)srcs, nsrc, n, scale); break;
    case TMPI_BF16: sum_into<__nv_bfloat16, float>((__nv_bfloat16*)dst, (const __nv_bfloat16* const*)srcs, nsrc, n, scale); break;
    case TMPI_F32: sum_into<float, float>((float*)dst, (const float* const*)srcs, nsrc, n, scale); break;
    case TMPI_F64: sum_into<double, double>((double*)dst, (const double* const*)srcs, nsrc, n, scale); break;
  }
}

int check_group(const int* members, int n, int me) {
  if (!H.live) return fail(TMPI_ERR_STATE, "host heap not created");
  if (n < 1 || n > kMaxWorld || me < 0 || me >= n) return fail(TMPI_ERR_INVALID, "bad group (%d members, me %d)", n, me);
  if (members[me] != H.rank) return fail(TMPI_ERR_INVALID, "members[me]=%d is not this rank (%d)", members[me], H.rank);
  for (int i = 0; i < n; ++i)
    if (members[i] < 0 || members[i] >= H.world || !H.base[members[i]])
      return fail(TMPI_ERR_STATE, "peer %d is not attached", members[i]);
  return TMPI_OK;
}

// shard [b, e) of n elements for group index i: floor(n/size) each, the
// first n mod size get one more (the parameter server's rule,
// lib/parameterserver.cpp:282-294)
void shard(size_t n, int size, int i, size_t* b, size_t* e) {
  size_t q = n / size, r = n % size;
  *b = (size_t)i * q + ((size_t)i < r ? (size_t)i : r);
  *e = *b + q + ((size_t)i < r ? 1 : 0);
}

}  // namespace

// exposed to the other runtime files
void shm_shard(size_t n, int size, int i, size_t* b, size_t* e) { shard(n, size, i, b, e); }

// ---- the collectives proper (run on the ordered shm lane)
int shm_allreduce_impl(const void* in, void* out, size_t n, int dtype, double scale,
                       std::vector<int> members, int me, int algo) {
  int st = check_group(members.data(), (int)members.size(), me);
  if (st) return st;
  int N = (int)members.size();
  size_t es = dtype_size(dtype);
  if (!es) return fail(TMPI_ERR_INVALID, "bad dtype %d", dtype);
  if (N == 1) {
    const void* s[1] = {in};
    if (scale != 1.0) typed_sum(dtype, out, s, 1, n, scale);
    else if (out != in) memcpy(out, in, n * es);
    return TMPI_OK;
  }
  size_t chunk = H.stage_bytes / es;
  if (algo == 0) algo = (n * es <= (size_t)tunable("small_cpu_allreduce_size") * 4) ? 1 : 2;
  int my = members[me];
  int64_t tmo = budget();
  for (size_t off = 0; off < n; off += chunk) {
    size_t m = n - off < chunk ? n - off : chunk;
    memcpy(stageA(my), (const char*)in + off * es, m * es);
    if ((st = group_barrier(members.data(), N, me, tmo))) return st;
    if (algo == 1) {
      // one-shot: everybody reads everything, fixed member order => identical bits
      std::vector<const void*> srcs(N);
      for (int k = 0; k < N; ++k) srcs[k] = stageA(members[k]);
      typed_sum(dtype, (char*)out + off * es, srcs.data(), N, m, scale);
      if ((st = group_barrier(members.data(), N, me, tmo))) return st;
    } else if (algo == 4) {
      // chunked ring on the working copies in region A (kept as the
      // comparison variant of the reference's algorithm)
      for (int phase = 0; phase < 2; ++phase)
        for (int s = 0; s < N - 1; ++s) {
          int c = tmpi_ring_recv_chunk(me, N, s, phase);
          size_t b, e; shard(m, N, c, &b, &e);
          int prev = members[(me + N - 1) % N];
          char* mine = stageA(my) + b * es;
          const char* theirs = stageA(prev) + b * es;
          if (phase == 0) {
            const void* srcs[2] = {mine, theirs};
            typed_sum(dtype, mine, srcs, 2, e - b, 1.0);
          } else {
            memcpy(mine, theirs, (e - b) * es);
          }
          if ((st = group_barrier(members.data(), N, me, tmo))) return st;
        }
      const void* s1[1] = {stageA(my)};
      if (scale != 1.0) typed_sum(dtype, (char*)out + off * es, s1, 1, m, scale);
      else memcpy((char*)out + off * es, stageA(my), m * es);
      if ((st = group_barrier(members.data(), N, me, tmo))) return st;
    } else {
      // two-shot: reduce my shard from every peer, publish it, gather the rest
      size_t b, e; shard(m, N, me, &b, &e);
      std::vector<const void*> srcs(N);
      for (int k = 0; k < N; ++k) srcs[k] = stageA(members[k]) + b * es;
      typed_sum(dtype, stageB(my) + b * es, srcs.data(), N, e - b, scale);
      if ((st = group_barrier(members.data(), N, me, tmo))) return st;
      for (int k = 0; k < N; ++k) {
        size_t kb, ke; shard(m, N, k, &kb, &ke);
        memcpy((char*)out + (off + kb) * es, stageB(members[k]) + kb * es, (ke - kb) * es);
      }
      if ((st = group_barrier(members.data(), N, me, tmo))) return st;
    }
  }
  return TMPI_OK;
}

int shm_broadcast_impl(void* buf, size_t n, int dtype, int root, std::vector<int> members, int me) {
  int st = check_group(members.data(), (int)members.size(), me);
  if (st) return st;
  int N = (int)members.size();
  if (root < 0 || root >= N) return fail(TMPI_ERR_INVALID, "bad root %d", root);
  if (N == 1) return TMPI_OK;
  size_t es = dtype_size(dtype), chunk = H.stage_bytes / es;
  int64_t tmo = budget();
  for (size_t off = 0; off < n; off += chunk) {
    size_t m = n - off < chunk ? n - off : chunk;
    if (me == root) memcpy(stageA(members[root]), (char*)buf + off * es, m * es);
    if ((st = group_barrier(members.data(), N, me, tmo))) return st;
    if (me != root) memcpy((char*)buf + off * es, stageA(members[root]), m * es);
    if ((st = group_barrier(members.data(), N, me, tmo))) return st;
  }
  return TMPI_OK;
}

int shm_reduce_impl(const void* in, void* out, size_t n, int dtype, int root, std::vector<int> members, int me) {
  int st = check_group(members.data(), (int)members.size(), me);
  if (st) return st;
  int N = (int)members.size();
  if (root < 0 || root >= N) return fail(TMPI_ERR_INVALID, "bad root %d", root);
  size_t es = dtype_size(dtype), chunk = H.stage_bytes / es;
  if (N == 1) { if (out != in) memcpy(out, in, n * es); return TMPI_OK; }
  int64_t tmo = budget();
  for (size_t off = 0; off < n; off += chunk) {
    size_t m = n - off < chunk ? n - off : chunk;
    memcpy(stageA(members[me]), (const char*)in + off * es, m * es);
    if ((st = group_barrier(members.data(), N, me, tmo))) return st;
    if (me == root) {
      std::vector<const void*> srcs(N);
      for (int k = 0; k < N; ++k) srcs[k] = stageA(members[k]);
      typed_sum(dtype, (char*)out + off * es, srcs.data(), N, m, 1.0);
    }
    if ((st = group_barrier(members.data(), N, me, tmo))) return st;
  }
  return TMPI_OK;
}

}  // namespace tmpi

namespace tmpi {

int shm_allgather_impl(const void* in, void* out, size_t n_in, std::vector<int64_t> counts, int dtype,
                       std::vector<int> members, int me) {
  int st = check_group(members.data(), (int)members.size(), me);
  if (st) return st;
  int N = (int)members.size();
  size_t es = dtype_size(dtype);
  if (counts.empty()) counts.assign(N, (int64_t)n_in);
  if ((size_t)counts[me] != n_in) return fail(TMPI_ERR_INVALID, "counts[me] != n_in");
  std::vector<size_t> offs(N + 1, 0);
  size_t maxc = 0;
  for (int k = 0; k < N; ++k) { offs[k + 1] = offs[k] + (size_t)counts[k]; if ((size_t)counts[k] > maxc) maxc = counts[k]; }
  if (N == 1) { if (out != in) memcpy(out, in, n_in * es); return TMPI_OK; }
  size_t chunk = H.stage_bytes / es;
  int64_t tmo = budget();
  for (size_t off = 0; off < maxc; off += chunk) {
    size_t mine = n_in > off ? (n_in - off < chunk ? n_in - off : chunk) : 0;
    if (mine) memcpy(stageA(members[me]), (const char*)in + off * es, mine * es);
    if ((st = group_barrier(members.data(), N, me, tmo))) return st;
    for (int k = 0; k < N; ++k) {
      size_t ck = (size_t)counts[k];
      size_t m = ck > off ? (ck - off < chunk ? ck - off : chunk) : 0;
      if (m) memcpy((char*)out + (offs[k] + off) * es, stageA(members[k]), m * es);
    }
    if ((st = group_barrier(members.data(), N, me, tmo))) return st;
  }
  return TMPI_OK;
}

namespace {
constexpr int kShmLane = 62;  // ordered lane reserved for host-heap collectives
std::vector<int> vec(const int* p, int n) { return std::vector<int>(p, p + n); }
int run_sync(std::function<int()> fn) {
  // sync calls take the same lane so that they stay ordered after async ones
  uint64_t h = submit_ordered(kShmLane, std::move(fn));
  return tmpi_handle_wait(h, -1);
}
}  // namespace
}  // namespace tmpi

using namespace tmpi;

extern "C" {

int tmpi_shm_create(const char* name, size_t bytes, int rank, int world, void** base) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (H.live) return fail(TMPI_ERR_STATE, "host heap already created");
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
    return fail(TMPI_ERR_INVALID, "bad rank/world %d/%d (max %d)", rank, world, kMaxWorld);
  size_t stage = (bytes / 4) & ~size_t(4095);
  if (stage < 4096) return fail(TMPI_ERR_INVALID, "host heap of %zu bytes is too small", bytes);
  size_t total = kHeaderBytes + 2 * stage + (bytes - 2 * stage);
  shm_unlink(name);
  int fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
  if (fd < 0) return fail(TMPI_ERR_SYS, "shm_open(%s): %s", name, strerror(errno));
  if (ftruncate(fd, (off_t)total) != 0) { close(fd); shm_unlink(name); return fail(TMPI_ERR_SYS, "ftruncate: %s", strerror(errno)); }
  void* p = mmap(nullptr, total, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) { shm_unlink(name); return fail(TMPI_ERR_SYS, "mmap: %s", strerror(errno)); }
  H = Heap();
  H.live = true; H.rank = rank; H.world = world;
  H.seg_bytes = total; H.stage_bytes = stage; H.arena_bytes = bytes - 2 * stage;
  H.my_name = name;
  H.base[rank] = (char*)p;
  new (p) Header();
  for (auto& s : hdr(rank)->sig) s.store(0);
  hdr(rank)->magic.store(0x544d5049u, std::memory_order_release);
  if (base) *base = p;
  return TMPI_OK;
}

int tmpi_shm_attach(int peer, const char* name) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (!H.live) return fail(TMPI_ERR_STATE, "host heap not created");
  if (peer < 0 || peer >= H.world) return fail(TMPI_ERR_INVALID, "bad peer %d", peer);
  if (peer == H.rank || H.base[peer]) return TMPI_OK;
  int fd = shm_open(name, O_RDWR, 0600);
  if (fd < 0) return fail(TMPI_ERR_SYS, "shm_open(%s): %s", name, strerror(errno));
  struct stat sb;
  if (fstat(fd, &sb) != 0 || (size_t)sb.st_size != H.seg_bytes) {
    close(fd);
    return fail(TMPI_ERR_STATE, "segment %s has %lld bytes, expected %zu", name, (long long)sb.st_size, H.seg_bytes);
  }
  void* p = mmap(nullptr, H.seg_bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) return fail(TMPI_ERR_SYS, "mmap peer: %s", strerror(errno));
  H.base[peer] = (char*)p;
  return TMPI_OK;
}

int tmpi_shm_ready(void) { return H.live ? 1 : 0; }
size_t tmpi_shm_capacity(void) { return H.live ? H.stage_bytes : 0; }
void* tmpi_shm_base(int peer) { return (H.live && peer >= 0 && peer < H.world) ? H.base[peer] : nullptr; }

int tmpi_shm_destroy(void) {
  tmpi_sync_all();
  std::lock_guard<std::mutex> lk(g_mu);
  if (!H.live) return TMPI_OK;
  for (int r = 0; r < H.world; ++r) if (H.base[r]) munmap(H.base[r], H.seg_bytes);
  shm_unlink(H.my_name.c_str());
  H = Heap();
  return TMPI_OK;
}

int tmpi_shm_barrier(const int* members, int n, int me, int64_t timeout_ms) {
  auto m = vec(members, n);
  int64_t t = timeout_ms >= 0 ? timeout_ms : budget();
  return run_sync([=] { int st = check_group(m.data(), n, me); return st ? st : group_barrier(m.data(), n, me, t); });
}

int tmpi_shm_allreduce(const void* in, void* out, size_t n, int dtype, double scale,
                       const int* members, int nm, int me, int algo) {
  auto m = vec(members, nm);
  return run_sync([=] { return shm_allreduce_impl(in, out, n, dtype, scale, m, me, algo); });
}
uint64_t tmpi_shm_allreduce_async(const void* in, void* out, size_t n, int dtype, double scale,
                                  const int* members, int nm, int me, int algo) {
  auto m = vec(members, nm);
  return submit_ordered(kShmLane, [=] { return shm_allreduce_impl(in, out, n, dtype, scale, m, me, algo); });
}
int tmpi_shm_broadcast(void* buf, size_t n, int dtype, int root, const int* members, int nm, int me) {
  auto m = vec(members, nm);
  return run_sync([=] { return shm_broadcast_impl(buf, n, dtype, root, m, me); });
}
uint64_t tmpi_shm_broadcast_async(void* buf, size_t n, int dtype, int root, const int* members, int nm, int me) {
  auto m = vec(members, nm);
  return submit_ordered(kShmLane, [=] { return shm_broadcast_impl(buf, n, dtype, root, m, me); });
}
int tmpi_shm_reduce(const void* in, void* out, size_t n, int dtype, int root, const int* members, int nm, int me) {
  auto m = vec(members, nm);
  return run_sync([=] { return shm_reduce_impl(in, out, n, dtype, root, m, me); });
}
int tmpi_shm_allgather(const void* in, void* out, size_t n_in, const int64_t* counts, int dtype,
                       const int* members, int nm, int me) {
  auto m = vec(members, nm);
  std::vector<int64_t> c;
  if (counts) c.assign(counts, counts + nm);
  return run_sync([=] { return shm_allgather_impl(in, out, n_in, c, dtype, m, me); });
}

}  // extern "C"

// ---------------------------------------------------------------- host parameter server
// Shards live in the owner's arena behind a small lock word.  A client applies
// its update (or reads the shard) directly in the owner's memory while holding
// that lock, so updates to one shard are serialised as they are by the
// reference's server thread (lib/parameterserver.cpp:404-541,632-663) without
// any thread polling for messages.  Requests run on the parameter-server pool
// and complete a handle; when send's handle has completed the update is
// already applied at every owner.
namespace tmpi {
namespace {

struct ShardHeader { std::atomic<uint32_t> lock; uint32_t pad[15]; };  // 64 bytes

struct PsInstance {
  bool live = false;
  size_t n = 0; int dtype = 0;
  std::vector<int> members; int me = 0;
  size_t arena_off = 0;      // same offset in every member's arena
  size_t shard_cap = 0;      // bytes reserved per shard
};
std::vector<PsInstance> g_ps;

int lock_shard(ShardHeader* h, int64_t timeout_ms) {
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  int iter = 0;
  for (;;) {
    uint32_t exp = 0;
    if (h->lock.compare_exchange_weak(exp, 1, std::memory_order_acquire)) return TMPI_OK;
    spin_pause(iter++);
    if ((iter & 1023) == 0 && Clock::now() > deadline)
      return fail(TMPI_ERR_TIMEOUT, "parameter server: shard lock not released within %lld ms", (long long)timeout_ms);
  }
}
void unlock_shard(ShardHeader* h) { h->lock.store(0, std::memory_order_release); }

template <typename T>
void apply_rule(T* shard, const T* upd, size_t n, int rule) {
  if (rule == 0) { for (size_t i = 0; i < n; ++i) shard[i] = from_acc<T>(0.0); }
  else if (rule == 1) { memcpy(shard, upd, n * sizeof(T)); }
  else { for (size_t i = 0; i < n; ++i) shard[i] = from_acc<T>(to_acc<T>(shard[i]) + to_acc<T>(upd[i])); }
}

int apply_rule_typed(int dtype, void* shard, const void* upd, size_t n, int rule) {
  switch (dtype) {
    case TMPI_F32: apply_rule((float*)shard, (const float*)upd, n, rule); return TMPI_OK;
    case TMPI_F64: apply_rule((double*)shard, (const double*)upd, n, rule); return TMPI_OK;
    case TMPI_BF16: apply_rule((__nv_bfloat16*)shard, (const __nv_bfloat16*)upd, n, rule); return TMPI_OK;
    case TMPI_F16: apply_rule((__half*)shard, (const __half*)upd, n, rule); return TMPI_OK;
    case TMPI_I32: apply_rule((int32_t*)shard, (const int32_t*)upd, n, rule); return TMPI_OK;
    case TMPI_I64: apply_rule((int64_t*)shard, (const int64_t*)upd, n, rule); return TMPI_OK;
  }
  return fail(TMPI_ERR_UNSUPPORTED, "parameter server: dtype %d", dtype);
}

}  // namespace
}  // namespace tmpi

extern "C" {

int tmpi_ps_shard_range(size_t n, int size, int rank, size_t* begin, size_t* end) {
  if (size < 1 || rank < 0 || rank >= size) return fail(TMPI_ERR_INVALID, "bad shard request");
  shm_shard(n, size, rank, begin, end);
  return TMPI_OK;
}

// Collective over `members` (the caller brackets it with barriers).  Returns the instance id.
int tmpi_shm_ps_init(const void* data, size_t n, int dtype, const int* members, int nm, int me) {
  std::lock_guard<std::mutex> lk(g_mu);
  int st = check_group(members, nm, me);
  if (st) return -st;
  size_t es = dtype_size(dtype);
  size_t cap = ((n + nm - 1) / nm) * es;
  cap = (cap + 63) & ~size_t(63);
  size_t need = sizeof(ShardHeader) + cap;
  if (H.arena_used + need > H.arena_bytes)
    return -fail(TMPI_ERR_STATE, "parameter server arena full (%zu of %zu bytes used, %zu more needed)",
                 H.arena_used, H.arena_bytes, need);
  PsInstance inst;
  inst.live = true; inst.n = n; inst.dtype = dtype;
  inst.members.assign(members, members + nm); inst.me = me;
  inst.arena_off = H.arena_used; inst.shard_cap = cap;
  H.arena_used += need;
  char* mine = arena(H.rank) + inst.arena_off;
  new (mine) ShardHeader();
  ((ShardHeader*)mine)->lock.store(0);
  size_t b, e; shm_shard(n, nm, me, &b, &e);
  memcpy(mine + sizeof(ShardHeader), (const char*)data + b * es, (e - b) * es);
  g_ps.push_back(inst);
  return (int)g_ps.size() - 1;
}

int tmpi_shm_ps_free(int id) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (id < 0 || id >= (int)g_ps.size()) return fail(TMPI_ERR_INVALID, "no parameter server %d", id);
  g_ps[id].live = false;
  bool any = false;
  for (auto& p : g_ps) any = any || p.live;
  if (!any) { g_ps.clear(); H.arena_used = 0; }
  return TMPI_OK;
}

int tmpi_shm_ps_free_all(void) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_ps.clear(); H.arena_used = 0;
  return TMPI_OK;
}

static int ps_get(int id, PsInstance* out) {
  std::lock_guard<std::mutex> lk(g_mu);
  if (id < 0 || id >= (int)g_ps.size() || !g_ps[id].live) return fail(TMPI_ERR_INVALID, "no parameter server %d", id);
  *out = g_ps[id];
  return TMPI_OK;
}

uint64_t tmpi_shm_ps_send(int id, const void* data, int rule) {
  PsInstance inst;
  int st = ps_get(id, &inst);
  if (st) return make_ready_handle(st);
  if (rule < 0 || rule > 2) return make_ready_handle(fail(TMPI_ERR_INVALID, "unknown update rule %d", rule));
  return submit(POOL_PS, [inst, data, rule] {
    size_t es = dtype_size(inst.dtype);
    int N = (int)inst.members.size();
    int64_t tmo = budget();
    // start at my own shard and walk round so that clients spread over owners
    for (int k = 0; k < N; ++k) {
      int i = (inst.me + k) % N;
      size_t b, e; shm_shard(inst.n, N, i, &b, &e);
      char* s = arena(inst.members[i]) + inst.arena_off;
      ShardHeader* h = (ShardHeader*)s;
      int st = lock_shard(h, tmo);
      if (st) return st;
      st = apply_rule_typed(inst.dtype, s + sizeof(ShardHeader), (const char*)data + b * es, e - b, rule);
      unlock_shard(h);
      if (st) return st;
    }
    return (int)TMPI_OK;
  });
}

uint64_t tmpi_shm_ps_receive(int id, void* data) {
  PsInstance inst;
  int st = ps_get(id, &inst);
  if (st) return make_ready_handle(st);
  return submit(POOL_PS, [inst, data] {
    size_t es = dtype_size(inst.dtype);
    int N = (int)inst.members.size();
    int64_t tmo = budget();
    for (int k = 0; k < N; ++k) {
      int i = (inst.me + k) % N;
      size_t b, e; shm_shard(inst.n, N, i, &b, &e);
      char* s = arena(inst.members[i]) + inst.arena_off;
      ShardHeader* h = (ShardHeader*)s;
      int st = lock_shard(h, tmo);
      if (st) return st;
      memcpy((char*)data + b * es, s + sizeof(ShardHeader), (e - b) * es);
      unlock_shard(h);
    }
    return (int)TMPI_OK;
  });
}

}  // extern "C"
