// State of the CUDA symmetric heap, shared by the runtime's CUDA translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <chrono>
#include <mutex>
#include <vector>
#include "common.h"
#include "../kernels/flags.cuh"
#include "../kernels/launch.h"

namespace tmpi {

constexpr int kHeapLanes = 4;          // 0 sync/user stream, 1 async pool, 2 fused optimizer, 3 parameter server
constexpr int LANE_SYNC = 0, LANE_ASYNC = 1, LANE_OPT = 2, LANE_PS = 3;

struct CudaHeap {
  bool live = false;
  bool emulated = false;             // all ranks on this device, in this process
  int backend = 0;                   // 0 cudaMalloc + cudaIpc, 1 VMM (+ multicast)
  int rank = 0, world = 1, device = 0;
  size_t total_bytes = 0;            // whole mapping per rank
  size_t slot_bytes = 0;             // one-shot slot
  size_t slots_off = 0;              // [lane][parity][writer] slots
  size_t bounce_off = 0;             // [lane 0..1] bounce buffers
  size_t bounce_bytes = 0;
  size_t arena_off = 0;              // user allocations start here
  size_t arena_cursor = 0;
  char* base[kMaxPeers] = {};
  bool imported[kMaxPeers] = {};
  char* mc_base = nullptr;
  uint32_t epoch[kMaxLanes][kMaxPeers][kMaxPeers] = {};   // [lane][a][b]: barriers done between heap ranks a and b
                                                          // (a real rank only uses row a == its own rank)
  int* status_host = nullptr;        // mapped pinned, kHeapLanes * 4 ints
  int* status_dev = nullptr;
  cudaStream_t lane_stream[kHeapLanes] = {};
  // VMM bookkeeping
  CUmemGenericAllocationHandle mem_handle = 0;
  CUmemGenericAllocationHandle peer_handles[kMaxPeers] = {};
  CUmemGenericAllocationHandle mc_handle = 0;
  bool mc_bound = false;
  int export_fd = -1, mc_export_fd = -1;
  std::chrono::steady_clock::time_point created{};   // start of the start-up grace period of device waits
  std::mutex mu;                     // arena + epochs of lanes driven from several threads
};

CudaHeap& heap();

int cuda_fail(cudaError_t e, const char* what);
int cu_fail(CUresult r, const char* what);

// one-shot slot offset helpers
inline size_t oneshot_slots_off(const CudaHeap& h, int lane) {
  return h.slots_off + (size_t)lane * 2 * h.world * h.slot_bytes;
}
inline size_t bounce_off(const CudaHeap& h, int lane) { return h.bounce_off + (size_t)lane * h.bounce_bytes; }

// Fills P for the given members (heap ranks) as seen from member index `me` (heap rank members[me]).
// In emulation every rank of the group gets its own Peers with the same epochs.
int fill_peers(Peers* P, const int* members, int n, int me, int lane);
// Advances the pair epochs of `lane` for these members by `barriers`.
void advance_epochs(const int* members, int n, int me, int lane, int barriers);

int64_t device_wait_budget_ms();
int grid_for(size_t work_items, int threads, const char* cap_name = "comm_max_ctas");

// VMM / multicast backend (cuda_vmm.cpp)
int vmm_create(CudaHeap& h);
int vmm_export(CudaHeap& h, void* out, int cap);
int vmm_import(CudaHeap& h, int peer, const void* blob, int len);
int vmm_destroy(CudaHeap& h);

}  // namespace tmpi
