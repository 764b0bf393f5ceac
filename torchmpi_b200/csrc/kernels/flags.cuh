// Cross-GPU signalling for kernels that read and write peer memory.
//
// Every rank's symmetric heap starts with a control region holding one 32-bit
// flag per (lane, block, writer rank).  A block of rank r announces "I am at
// point k" to peer p by storing an epoch value into p's flag [lane][block][r]
// with release order at system scope, and waits for p by polling its own flag
// [lane][block][p] with acquire order.  Epochs only grow, so flags are never
// reset; they are counted per pair of ranks by the host (both ends of a pair
// have issued the same collectives involving each other, in the same order on a
// lane), which lets sub-groups of the heap run collectives independently.
//
// Every wait is bounded: after `budget_ns` without the expected value the block
// records {code, where, peer, epoch} in a host-mapped status word, raises a
// block-wide abort flag, stops touching peer memory and returns normally.  The
// host turns the status into an error.  Nothing here traps or spins for ever.
//
// The reference synchronises its copy-engine ring with IPC events plus one
// host MPI_Barrier per step (lib/detail/collectives_cuda.cpp:274-385); here the
// whole collective is one kernel and the host is not involved.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "vec.cuh"

namespace tmpi {

constexpr int kMaxPeers = 16;        // ranks per heap
constexpr int kMaxLanes = 8;
constexpr int kMaxBlocks = 256;      // CTAs per collective kernel
constexpr size_t kFlagBytes = size_t(kMaxLanes) * kMaxBlocks * kMaxPeers * sizeof(uint32_t);
constexpr size_t kControlBytes = 1 << 20;   // flags + spare, start of every heap

enum { ST_OK = 0, ST_TIMEOUT = 3 };

// The ranks taking part in one launch, seen from one of them.
struct Peers {
  char* base[kMaxPeers];        // heap base of member i as mapped in this process
  uint32_t epoch[kMaxPeers];    // pair epoch with member i before this launch
  int rank_of[kMaxPeers];       // heap rank of member i
  int n;                        // members
  int me;                       // my index among the members
  int lane;
  int* status;                  // host-mapped int[4]; status[0] != 0 after a failure
  unsigned long long budget_ns;
  char* mc_base;                // multicast mapping of the heap (nullptr when absent)
  size_t heap_bytes;            // bytes of every member's mapping (debug bounds checks)
};

__device__ __forceinline__ uint32_t* flag_ptr(char* heap_base, int lane, int block, int writer) {
  return reinterpret_cast<uint32_t*>(heap_base) + ((size_t)lane * kMaxBlocks + block) * kMaxPeers + writer;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Polls *p until it has reached `want` (wrap-safe) or the budget is spent.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t want, unsigned long long budget_ns) {
  if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
  unsigned long long t0 = global_ns();
  unsigned sleep_ns = 32;
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
      __nanosleep(sleep_ns);
    }
    if (sleep_ns < 1024) sleep_ns *= 2;
    if (global_ns() - t0 > budget_ns) return false;
  }
}

__device__ __forceinline__ void report(const Peers& P, int code, int where, int peer, uint32_t epoch) {
  if (P.status && atomicCAS(P.status, 0, code) == 0) {
    P.status[1] = where; P.status[2] = peer; P.status[3] = (int)epoch;
    __threadfence_system();
  }
}

#ifdef TMPI_DEBUG_BOUNDS
// Kernel entry in the debug build: publishes the address ranges that peer accesses of this launch may touch
// (every thread writes the same values; a block-wide barrier follows in the caller).
__device__ __forceinline__ void dbg_enter(const Peers& P, const void* local0, size_t len0, const void* local1, size_t len1) {
  if (threadIdx.x == 0) {
    int k = 0;
    for (int i = 0; i < P.n; ++i) { g_dbg.lo[k] = P.base[i]; g_dbg.len[k++] = P.heap_bytes; }
    g_dbg.lo[k] = P.mc_base; g_dbg.len[k++] = P.heap_bytes;
    g_dbg.lo[k] = (const char*)local0; g_dbg.len[k++] = len0;
    g_dbg.lo[k] = (const char*)local1; g_dbg.len[k++] = len1;
    g_dbg.status = P.status;
    g_dbg.n = k;
    __threadfence();
  }
}
#define TMPI_DBG_ENTER(P, l0, n0, l1, n1) dbg_enter((P), (l0), (n0), (l1), (n1))
#else
#define TMPI_DBG_ENTER(P, l0, n0, l1, n1)
#endif

// Barrier number k (1-based within the launch) of this block with the same block of every peer.
// All threads of the block must call it.  Returns false when a wait ran out: the caller must
// then skip every further access to peer memory.
__device__ __forceinline__ bool peer_barrier(const Peers& P, uint32_t k, int where, int* s_abort) {
  __threadfence_system();
  __syncthreads();
  int t = threadIdx.x;
  if (t < P.n && t != P.me && *s_abort == 0) {
    uint32_t e = P.epoch[t] + k;
    st_release_sys(flag_ptr(P.base[t], P.lane, blockIdx.x, P.rank_of[P.me]), e);
    if (!wait_flag(flag_ptr(P.base[P.me], P.lane, blockIdx.x, P.rank_of[t]), e, P.budget_ns)) {
      report(P, ST_TIMEOUT, where, P.rank_of[t], e);
      atomicExch(s_abort, 1);
    }
  }
  __syncthreads();
  return *s_abort == 0;
}

}  // namespace tmpi
