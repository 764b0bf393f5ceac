// CUDA symmetric heap: one slab per rank, mapped by every peer once.
//
// Every buffer that takes part in a device collective lives at the same offset
// in every rank's slab, so a kernel needs only the table of slab bases to reach
// a peer's copy.  This replaces the reference's per-tensor machinery - an IPC
// handle exchange keyed by each tensor's base pointer, storage retention so that
// keys cannot be recycled, per-collective IPC event matrices
// (lib/resources.cpp:840-1163, lib/torch_mpi_cuda.cpp:27-89) - with one exchange
// at start-up.
//
// Layout of a slab:  [control: flags, 1 MiB][one-shot slots][bounce buffers][arena].
// Backend 0 allocates with cudaMalloc and shares with cudaIpc handles; backend 1
// (cuda_vmm.cpp) uses the virtual-memory API so that the slabs can also be bound
// to an NVLink multicast object (NVLS).  An *emulated* heap puts all ranks' slabs
// on one device in one process, for exercising the multi-rank kernels on a
// single GPU with cooperative launches.
#include <chrono>
#include <algorithm>
#include "cuda_state.h"
#include <algorithm>
#include <cstring>

namespace tmpi {

static CudaHeap g_heap;
CudaHeap& heap() { return g_heap; }

int cuda_fail(cudaError_t e, const char* what) {
  return fail(TMPI_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define CK(call)                                          \
  do {                                                    \
    cudaError_t e__ = (call);                             \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call); \
  } while (0)

static size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int layout_heap(CudaHeap& h, size_t arena_bytes) {
  h.slot_bytes = round_up((size_t)tunable("oneshot_max_bytes"), 256);
  h.bounce_bytes = round_up((size_t)tunable("staging_bytes"), 4096);
  h.slots_off = kControlBytes;
  size_t slots = (size_t)kHeapLanes * 2 * h.world * h.slot_bytes;
  h.bounce_off = round_up(h.slots_off + slots, 4096);
  h.arena_off = round_up(h.bounce_off + 2 * h.bounce_bytes, 1 << 16);
  h.arena_cursor = h.arena_off;
  h.total_bytes = round_up(h.arena_off + arena_bytes, (size_t)2 << 20);
  // the one-shot kernel addresses slot (parity * world + writer) of a lane: the last lane's last slot must
  // end before the bounce buffers, and a lane's region must end where the next lane's begins
  if (oneshot_slots_off(h, kHeapLanes - 1) + (size_t)2 * h.world * h.slot_bytes > h.bounce_off)
    return fail(TMPI_ERR_STATE, "heap layout: one-shot slots overlap the bounce buffers");
  return TMPI_OK;
}

// Steady-state budget, or the start-up budget while the grace period after the heap's creation runs.
int64_t device_wait_budget_ms() {
  int64_t b = tunable("device_wait_budget_ms");
  const CudaHeap& h = heap();
  const auto age = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - h.created).count();
  if (age < tunable("device_wait_startup_grace_ms")) b = std::max<int64_t>(b, tunable("device_wait_startup_budget_ms"));
  return b;
}

int setup_common(CudaHeap& h) {
  h.created = std::chrono::steady_clock::now();
  CK(cudaHostAlloc((void**)&h.status_host, sizeof(int) * 4 * kHeapLanes, cudaHostAllocMapped));
  memset(h.status_host, 0, sizeof(int) * 4 * kHeapLanes);
  CK(cudaHostGetDevicePointer((void**)&h.status_dev, h.status_host, 0));
  int lo = 0, hi = 0;
  CK(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  for (int l = 0; l < kHeapLanes; ++l) CK(cudaStreamCreateWithPriority(&h.lane_stream[l], cudaStreamNonBlocking, hi));
  memset(h.epoch, 0, sizeof(h.epoch));
  return TMPI_OK;
}

int fill_peers(Peers* P, const int* members, int n, int me, int lane) {
  CudaHeap& h = heap();
  if (!h.live) return fail(TMPI_ERR_STATE, "CUDA heap not created");
  if (n < 1 || n > kMaxPeers || me < 0 || me >= n) return fail(TMPI_ERR_INVALID, "bad group (%d members, me %d)", n, me);
  if (lane < 0 || lane >= kHeapLanes) return fail(TMPI_ERR_INVALID, "bad lane %d", lane);
  if (!h.emulated && members[me] != h.rank)
    return fail(TMPI_ERR_INVALID, "members[me]=%d is not this rank (%d)", members[me], h.rank);
  memset(P, 0, sizeof(*P));
  const int mine = members[me];
  for (int i = 0; i < n; ++i) {
    int r = members[i];
    if (r < 0 || r >= h.world || !h.base[r]) return fail(TMPI_ERR_STATE, "peer %d is not mapped", r);
    P->base[i] = h.base[r];
    P->rank_of[i] = r;
    P->epoch[i] = h.epoch[lane][mine][r];
  }
  P->n = n; P->me = me; P->lane = lane;
  P->status = h.status_dev + 4 * lane;
  P->budget_ns = (unsigned long long)device_wait_budget_ms() * 1000000ull;
  P->mc_base = h.mc_base;
  P->heap_bytes = h.total_bytes;
  return TMPI_OK;
}

void advance_epochs(const int* members, int n, int me, int lane, int barriers) {
  CudaHeap& h = heap();
  const int mine = members[me];
  for (int i = 0; i < n; ++i) h.epoch[lane][mine][members[i]] += (uint32_t)barriers;
}

int grid_for(size_t items, int threads, const char* cap_name) {
  int cap = (int)tunable(cap_name);
  if (cap < 1) cap = 1;
  if (cap > kMaxBlocks) cap = kMaxBlocks;
  size_t want = (items + threads - 1) / threads;
  if (want < 1) want = 1;
  return (int)std::min<size_t>(want, (size_t)cap);
}

}  // namespace tmpi

using namespace tmpi;

extern "C" {

int tmpi_has_cuda(void) {
  int n = 0;
  return (cudaGetDeviceCount(&n) == cudaSuccess && n > 0) ? 1 : 0;
}

int tmpi_cuda_set_device(int device) {
  CK(cudaSetDevice(device));
  return TMPI_OK;
}

int tmpi_cuda_heap_create(size_t bytes, int rank, int world, int backend) {
  CudaHeap& h = heap();
  if (h.live) return fail(TMPI_ERR_STATE, "CUDA heap already created");
  if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world)
    return fail(TMPI_ERR_INVALID, "bad rank/world %d/%d (at most %d ranks per heap)", rank, world, kMaxPeers);
  h.rank = rank; h.world = world; h.backend = backend; h.emulated = false;
  CK(cudaGetDevice(&h.device));
  int st = layout_heap(h, bytes);
  if (st) return st;
  st = setup_common(h);
  if (st) return st;
  if (backend == 1) {
    st = vmm_create(h);
    if (st) return st;
  } else {
    void* p = nullptr;
    CK(cudaMalloc(&p, h.total_bytes));
    h.base[rank] = (char*)p;
  }
  CK(cudaMemset(h.base[rank], 0, h.arena_off));   // flags, slots and bounce start at zero
  CK(cudaDeviceSynchronize());
  h.imported[rank] = true;
  h.live = true;
  return TMPI_OK;
}

int tmpi_cuda_heap_create_emulated(size_t bytes, int world) {
  CudaHeap& h = heap();
  if (h.live) return fail(TMPI_ERR_STATE, "CUDA heap already created");
  if (world < 1 || world > 8) return fail(TMPI_ERR_INVALID, "emulation supports 1..8 ranks");
  h.rank = 0; h.world = world; h.backend = 0; h.emulated = true;
  CK(cudaGetDevice(&h.device));
  int st = layout_heap(h, bytes);
  if (st) return st;
  st = setup_common(h);
  if (st) return st;
  for (int r = 0; r < world; ++r) {
    void* p = nullptr;
    CK(cudaMalloc(&p, h.total_bytes));
    CK(cudaMemset(p, 0, h.arena_off));
    h.base[r] = (char*)p; h.imported[r] = true;
  }
  CK(cudaDeviceSynchronize());
  h.live = true;
  return TMPI_OK;
}

int tmpi_cuda_heap_export(void* out, int cap) {
  CudaHeap& h = heap();
  if (!h.live || h.emulated) return -fail(TMPI_ERR_STATE, "no exportable heap");
  if (h.backend == 1) return vmm_export(h, out, cap);
  if (cap < (int)sizeof(cudaIpcMemHandle_t)) return -fail(TMPI_ERR_INVALID, "export buffer too small");
  cudaIpcMemHandle_t hd;
  cudaError_t e = cudaIpcGetMemHandle(&hd, h.base[h.rank]);
  if (e != cudaSuccess) return -cuda_fail(e, "cudaIpcGetMemHandle");
  memcpy(out, &hd, sizeof(hd));
  return (int)sizeof(hd);
}

int tmpi_cuda_heap_import(int peer, const void* blob, int len) {
  CudaHeap& h = heap();
  if (!h.live || h.emulated) return fail(TMPI_ERR_STATE, "no heap to import into");
  if (peer < 0 || peer >= h.world) return fail(TMPI_ERR_INVALID, "bad peer %d", peer);
  if (peer == h.rank || h.imported[peer]) return TMPI_OK;
  if (h.backend == 1) return vmm_import(h, peer, blob, len);
  if (len != (int)sizeof(cudaIpcMemHandle_t)) return fail(TMPI_ERR_INVALID, "bad IPC handle length %d", len);
  cudaIpcMemHandle_t hd;
  memcpy(&hd, blob, sizeof(hd));
  void* p = nullptr;
  CK(cudaIpcOpenMemHandle(&p, hd, cudaIpcMemLazyEnablePeerAccess));
  h.base[peer] = (char*)p;
  h.imported[peer] = true;
  return TMPI_OK;
}

int tmpi_cuda_heap_finish(void) {
  CudaHeap& h = heap();
  for (int r = 0; r < h.world; ++r)
    if (!h.imported[r]) return fail(TMPI_ERR_STATE, "peer %d was never imported", r);
  return TMPI_OK;
}

int tmpi_cuda_heap_destroy(void) {
  CudaHeap& h = heap();
  if (!h.live) return TMPI_OK;
  tmpi_sync_all();
  cudaDeviceSynchronize();
  if (h.backend == 1) {
    vmm_destroy(h);
  } else if (h.emulated) {
    for (int r = 0; r < h.world; ++r) if (h.base[r]) cudaFree(h.base[r]);
  } else {
    for (int r = 0; r < h.world; ++r)
      if (r != h.rank && h.base[r]) cudaIpcCloseMemHandle(h.base[r]);
    cudaFree(h.base[h.rank]);
  }
  for (int l = 0; l < kHeapLanes; ++l) if (h.lane_stream[l]) cudaStreamDestroy(h.lane_stream[l]);
  if (h.status_host) cudaFreeHost(h.status_host);
  h.live = false; h.emulated = false; h.mc_base = nullptr; h.mc_bound = false;
  h.status_host = h.status_dev = nullptr;
  memset(h.base, 0, sizeof(h.base));
  memset(h.imported, 0, sizeof(h.imported));
  memset(h.lane_stream, 0, sizeof(h.lane_stream));
  return TMPI_OK;
}

void* tmpi_cuda_heap_base(int peer) {
  CudaHeap& h = heap();
  return (h.live && peer >= 0 && peer < h.world) ? h.base[peer] : nullptr;
}
void* tmpi_cuda_heap_mc_base(void) { return heap().live ? heap().mc_base : nullptr; }
size_t tmpi_cuda_heap_capacity(void) { return heap().live ? heap().total_bytes - heap().arena_off : 0; }
// 1 when the library was built with recording bounds checks on peer accesses (-DTMPI_DEBUG_BOUNDS)
int tmpi_debug_bounds_build(void) {
#ifdef TMPI_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}
int tmpi_cuda_heap_world(void) { return heap().live ? heap().world : 0; }
int tmpi_cuda_heap_layout(size_t* out, int n) {
  const CudaHeap& h = heap();
  if (!h.live) return fail(TMPI_ERR_STATE, "CUDA heap not created");
  const size_t v[6] = {h.slots_off, h.slot_bytes, h.bounce_off, h.bounce_bytes, h.arena_off, h.total_bytes};
  for (int i = 0; i < n && i < 6; ++i) out[i] = v[i];
  return TMPI_OK;
}
int tmpi_cuda_heap_rank(void) { return heap().live ? heap().rank : -1; }

size_t tmpi_cuda_heap_alloc(size_t bytes, size_t align) {
  CudaHeap& h = heap();
  if (!h.live) { fail(TMPI_ERR_STATE, "CUDA heap not created"); return (size_t)-1; }
  if (align < 256) align = 256;
  std::lock_guard<std::mutex> lk(h.mu);
  size_t off = round_up(h.arena_cursor, align);
  if (off + bytes > h.total_bytes) {
    fail(TMPI_ERR_STATE, "symmetric heap exhausted: %zu bytes requested, %zu of %zu free (raise the heap_bytes tunable)",
         bytes, h.total_bytes - h.arena_cursor, h.total_bytes - h.arena_off);
    return (size_t)-1;
  }
  h.arena_cursor = off + bytes;
  return off;
}

// Moves the allocation cursor back to `cursor` (an offset returned earlier by alloc, or 0 for empty).
int tmpi_cuda_heap_reset_allocator(size_t cursor) {
  CudaHeap& h = heap();
  if (!h.live) return fail(TMPI_ERR_STATE, "CUDA heap not created");
  std::lock_guard<std::mutex> lk(h.mu);
  if (cursor == 0) cursor = h.arena_off;
  if (cursor < h.arena_off || cursor > h.total_bytes) return fail(TMPI_ERR_INVALID, "bad cursor");
  h.arena_cursor = cursor;
  return TMPI_OK;
}

int tmpi_cuda_collective_status(int lane, int* code, int* where, int* peer) {
  CudaHeap& h = heap();
  if (!h.live || lane < 0 || lane >= kHeapLanes) return fail(TMPI_ERR_STATE, "no heap / bad lane");
  volatile int* s = h.status_host + 4 * lane;
  *code = s[0]; *where = s[1]; *peer = s[2];
  if (s[0]) { s[0] = 0; s[1] = 0; s[2] = 0; s[3] = 0; }
  return TMPI_OK;
}

}  // extern "C"
