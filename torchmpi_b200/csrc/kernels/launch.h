// Host-side interface of the collective kernels (implemented in collectives.cu, ar_sgd.cu, ps.cu).
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include "flags.cuh"

namespace tmpi {

enum CollOp {
  OP_AR_ONESHOT = 0,    // push inputs into every peer's slot, one barrier, local sum
  OP_AR_TWOSHOT,        // reduce own shard from all peers, write it to all peers
  OP_AR_NVLS,           // multimem.ld_reduce own shard, multimem.st it
  OP_AR_RING,           // in-kernel chunked ring (comparison variant)
  OP_BCAST_PULL,        // every non-root reads the root's buffer
  OP_BCAST_CHUNKED,     // scatter from root, then all-gather among peers
  OP_BCAST_MC,          // root stores through the multicast mapping
  OP_REDUCE,            // root reads and sums every peer's buffer
  OP_ALLGATHER,         // everybody reads every peer's chunk
  OP_REDUCE_SCATTER,    // everybody sums its own slice of every peer's buffer
  OP_BARRIER,
  OP_AR_TWOSHOT_ANY,    // two-shot on tensors outside the heap: scatter-push, local reduce, gather-pull
  OP_BCAST_ANY,         // broadcast of a tensor outside the heap: root pushes into scratch, peers copy out
  OP_BCAST_SCATTER_MC,  // member m reads chunk m from the root and stores it through the multicast mapping
  OP_BCAST_SCATTER_PUSH,  // each non-root member reads its chunk from the root and stores it into the other non-root members
  OP_COUNT
};

struct CollArgs {
  Peers P;
  const void* in;          // local input pointer (one-shot) or nullptr
  void* out;               // local output pointer (one-shot, reduce, allgather, reduce_scatter)
  size_t in_off;           // byte offset of the symmetric source buffer (or of the one-shot slots)
  size_t out_off;          // byte offset of the symmetric destination buffer
  size_t n;                // elements
  size_t aux;              // one-shot: bytes per slot
  size_t cnt[kMaxPeers];   // allgather: elements contributed by member i
  float scale;
  int root;
};

struct CollArgsPack {      // single-GPU emulation: all ranks in one cooperative launch
  CollArgs r[8];
};

// Number of peer barriers the op performs (the host advances pair epochs by this much).
int barriers_used(int op, int nmembers);

// Launches the kernel of `op` for element type `dtype`.  nranks == 1: the real thing, args[0] is
// this rank.  nranks > 1: emulation, one cooperative launch with gridDim.y == nranks.
// `vec` selects 16-byte packs (1) or single elements (0).
cudaError_t launch_collective(int op, int dtype, const CollArgs* args, int nranks, int vec,
                              int grid, int threads, cudaStream_t stream);

struct SgdArgs {
  Peers P;
  size_t grad_off, weight_off;   // symmetric byte offsets
  float* master;                 // this rank's shard (nullptr: none)
  float* momentum;               // this rank's shard (nullptr: none)
  size_t n;                      // elements in the bucket
  float lr, momentum_coef, dampening, weight_decay, grad_scale;
  int nesterov, first_step, zero_grads, use_nvls;
};
struct SgdArgsPack { SgdArgs r[8]; };
int sgd_barriers_used(int nmembers);
cudaError_t launch_allreduce_sgd(int grad_dtype, int weight_dtype, const SgdArgs* args, int nranks,
                                 int grid, int threads, cudaStream_t stream);

struct PsArgs {
  Peers P;
  size_t shard_off;        // symmetric byte offset of the shard storage
  void* data;              // local tensor
  size_t n;                // elements of the whole tensor
  int rule;                // 0 zero, 1 copy, 2 add; -1 = pull
};
cudaError_t launch_ps(int dtype, const PsArgs* args, int grid, int threads, cudaStream_t stream);

cudaError_t launch_wait_probe(const Peers& P, cudaStream_t stream);

}  // namespace tmpi
