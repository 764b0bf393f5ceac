// Pieces shared by the fused tensor-parallel GEMM kernels (single-CTA and CTA-pair variants): the
// argument block, bulk-copy wrappers and the copy-engine body of the all-gather.
#pragma once
#include "gemm_core.cuh"
#include "flags.cuh"
#include "vec.cuh"

namespace tmpi {
namespace gemm {

struct FusedArgs {
  Peers P;
  size_t sym_off;              // ag: offset of every rank's A shard; rs: offset of the slot array [R][rows][N]
  __nv_bfloat16* local;        // ag: local full-A buffer; rs: local output [rows_per_rank, N]
  uint32_t* ready;             // ag: one flag per M-tile (local memory)
  uint32_t ready_value;
  unsigned int* grid_counter;  // rs: monotonically growing arrival counter (local memory)
  unsigned int grid_target;
  int rows_per_rank;
  int n_comm;
};

constexpr int COPY_BYTES = 32768, COPY_STAGES = 6;

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(sm100::smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(sm100::smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(sm100::smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// ------------------------------------------------------------------ all-gather -> GEMM
// Copy-engine body of one comm CTA (all threads enter; one thread drives the copies).
//
// The CTA's tiles (128 rows = tile_bytes contiguous bytes each, own shard first, then the peers in
// ring order) are cut into 32 KB pieces numbered q = 0, 1, ...; piece q uses ring stage q % 6 and
// mbarrier parity (q / 6) & 1.  Steady state of iteration k: piece k has landed -> start its store
// -> wait until all stores but the newest are complete -> publish the tiles they finish ->
// start the load of piece k + 4 (its stage was last used by piece k - 2, whose store is complete).
// Four loads (128 KB) and up to two stores are in flight per CTA.
template <typename Sh>
__device__ void ag_comm(const FusedArgs& g, const Problem& p, unsigned char* tiles, Sh* sh, int* s_abort) {
  const Peers& P = g.P;
  const int R = P.n;
  const int tiles_per_rank = g.rows_per_rank / BM;
  const size_t tile_bytes = (size_t)BM * p.K * 2;
  const int ppt = (int)(tile_bytes / COPY_BYTES);               // pieces per tile (K % 128 == 0 on the host side)
  const int b = blockIdx.x;
  const int cnt = b < tiles_per_rank ? (tiles_per_rank - b + g.n_comm - 1) / g.n_comm : 0;   // my tiles per shard
  const int total = cnt * R * ppt;
  if (!peer_barrier(P, 1, 200, s_abort)) return;                // every rank's shard is ready to be read
  if (threadIdx.x == 0 && total > 0) {
    uint64_t* bars = sh->full;                                   // six contiguous barriers (full[] then empty[])
    auto src_of = [&](int q, const char** sp, char** dp, int* m_tile) {
      const int u = q / ppt, pi = q % ppt;
      // peers in ring order first; my own shard last (the GEMM reads it in place, the copy only completes A_full)
      const int src = (P.me + 1 + u / cnt) % R, c = b + (u % cnt) * g.n_comm;
      *m_tile = src * tiles_per_rank + c;
      *sp = P.base[src] + g.sym_off + (size_t)c * tile_bytes + (size_t)pi * COPY_BYTES;
      *dp = (char*)g.local + (size_t)(*m_tile) * tile_bytes + (size_t)pi * COPY_BYTES;
    };
    auto load = [&](int q) {
      const char* sp; char* dp; int mt;
      src_of(q, &sp, &dp, &mt);
      const int st = q % COPY_STAGES;
      sm100::mbar_expect_tx(&bars[st], COPY_BYTES);
      bulk_load(tiles + (size_t)st * COPY_BYTES, sp, COPY_BYTES, &bars[st]);
    };
    auto publish = [&](int q) {                                  // piece q is complete in local memory
      if (q % ppt != ppt - 1) return;
      const char* sp; char* dp; int mt;
      src_of(q, &sp, &dp, &mt);
      sm100::fence_proxy_async();
      __threadfence();
      st_release_gpu(&g.ready[mt], g.ready_value);
    };
    bool ok = true;
    for (int q = 0; q < 4 && q < total; ++q) load(q);
    for (int k = 0; k < total; ++k) {
      const int st = k % COPY_STAGES;
      if (!sm100::mbar_wait(&bars[st], (uint32_t)((k / COPY_STAGES) & 1), kWaitBudgetNs)) { ok = false; break; }
      const char* sp; char* dp; int mt;
      src_of(k, &sp, &dp, &mt);
      bulk_store(dp, tiles + (size_t)st * COPY_BYTES, COPY_BYTES);
      bulk_commit();
      asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); // stores of pieces <= k - 1 are complete
      if (k >= 1) publish(k - 1);
      if (k + 4 < total) load(k + 4);                           // its stage was last used by piece k - 2
    }
    bulk_wait_all();
    if (ok) {
      publish(total - 1);
    } else {
      fail(sh, p, 10);
      atomicExch(s_abort, 1);
    }
  }
  peer_barrier(P, 2, 201, s_abort);                              // nobody still reads my shard
}


// out[i] = sum over r of slots[r][i], added in rank order (every rank computes the same bits), for the
// reduce-scatter tail.  RC is the rank count when it is known at compile time (0: run-time loop); all
// loads of an iteration are issued before the first add, RC x U 16-byte loads per thread in flight -
// with one load in flight the pass ran at a seventh of the memory bandwidth.
template <int RC>
__device__ __forceinline__ void slot_sum_t(const __nv_bfloat16* __restrict__ slots, size_t slot_elems, int R,
                                           __nv_bfloat16* __restrict__ out, size_t t0, size_t stride) {
  using P8 = Pack<__nv_bfloat16, 8>;
  constexpr int U = RC == 0 ? 4 : (RC >= 4 ? 2 : 4);
  const size_t nv = slot_elems / 8;
  size_t i = t0;
  for (; i + (U - 1) * stride < nv; i += U * stride) {
    Acc<__nv_bfloat16, 8> acc[U];
    if constexpr (RC > 0) {
      P8 x[RC][U];
#pragma unroll
      for (int r = 0; r < RC; ++r)
#pragma unroll
        for (int u = 0; u < U; ++u) x[r][u] = ld_pack_peer<__nv_bfloat16, 8>(slots + (size_t)r * slot_elems + (i + u * stride) * 8);
#pragma unroll
      for (int u = 0; u < U; ++u) {
        acc[u].set(x[0][u]);
#pragma unroll
        for (int r = 1; r < RC; ++r) acc[u].add(x[r][u]);
      }
    } else {
      for (int r = 0; r < R; ++r) {
        P8 x[U];
#pragma unroll
        for (int u = 0; u < U; ++u) x[u] = ld_pack_peer<__nv_bfloat16, 8>(slots + (size_t)r * slot_elems + (i + u * stride) * 8);
#pragma unroll
        for (int u = 0; u < U; ++u) { if (r == 0) acc[u].set(x[u]); else acc[u].add(x[u]); }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) st_pack<__nv_bfloat16, 8>(out + (i + u * stride) * 8, acc[u].pack(1.0f));
  }
  for (; i < nv; i += stride) {
    Acc<__nv_bfloat16, 8> acc;
    for (int r = 0; r < R; ++r) {
      P8 x = ld_pack_peer<__nv_bfloat16, 8>(slots + (size_t)r * slot_elems + i * 8);
      if (r == 0) acc.set(x); else acc.add(x);
    }
    st_pack<__nv_bfloat16, 8>(out + i * 8, acc.pack(1.0f));
  }
}

__device__ __forceinline__ void slot_sum(const __nv_bfloat16* slots, size_t slot_elems, int R, __nv_bfloat16* out,
                                         size_t t0, size_t stride) {
  switch (R) {
    case 2: slot_sum_t<2>(slots, slot_elems, R, out, t0, stride); break;
    case 4: slot_sum_t<4>(slots, slot_elems, R, out, t0, stride); break;
    case 8: slot_sum_t<8>(slots, slot_elems, R, out, t0, stride); break;
    default: slot_sum_t<0>(slots, slot_elems, R, out, t0, stride); break;
  }
}

}  // namespace gemm
}  // namespace tmpi
