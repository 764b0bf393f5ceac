// Flat C ABI of libtorchmpi_b200.so.
//
// Python binds these symbols with ctypes (torchmpi_b200/_lib.py).  The layer
// plays the role of the reference's extern "C" surface (lib/c_api.h:11-174)
// but is shaped for one process per GPU on an NVSwitch host: tensors are
// passed as raw device/host pointers plus element counts, CUDA streams as
// opaque handles, and every entry point returns a status code (0 = ok)
// instead of aborting; tmpi_last_error() gives the message.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---------------------------------------------------------------- status
enum {
  TMPI_OK = 0,
  TMPI_ERR_INVALID = 1,      // bad argument
  TMPI_ERR_CUDA = 2,         // a CUDA runtime / driver call failed
  TMPI_ERR_TIMEOUT = 3,      // a bounded wait (host or device) ran out
  TMPI_ERR_STATE = 4,        // wrong call order / missing resource
  TMPI_ERR_UNSUPPORTED = 5,
  TMPI_ERR_SYS = 6,          // an OS call failed
};
const char* tmpi_last_error(void);
int tmpi_version(void);
int tmpi_has_cuda(void);  // 1 when a CUDA device answers in this process

// ---------------------------------------------------------------- dtypes
enum {
  TMPI_U8 = 0, TMPI_I8 = 1, TMPI_I16 = 2, TMPI_I32 = 3, TMPI_I64 = 4,
  TMPI_F16 = 5, TMPI_BF16 = 6, TMPI_F32 = 7, TMPI_F64 = 8,
};
size_t tmpi_dtype_size(int dtype);

// ---------------------------------------------------------------- tunables
// Same names and defaults as the reference's constants (lib/constants.cpp:130-155),
// plus the knobs of the B200 data plane.  Unknown names return TMPI_ERR_INVALID.
int tmpi_set_tunable(const char* name, int64_t value);
int tmpi_get_tunable(const char* name, int64_t* value);
int tmpi_num_tunables(void);
const char* tmpi_tunable_name(int index);
int tmpi_freeze_tunables(void);  // later sets fail with TMPI_ERR_STATE

// ---------------------------------------------------------------- communicator stack
// The control plane (key exchange) lives in Python on a store; the split
// itself, the level stack, the cursor and the collective span live here.
int tmpi_comm_reset(int world_rank, int world_size);
// keys: parent_size blocks of 1024 bytes (NUL padded), in parent order.
// parent_members: world ranks of the parent communicator in parent order.
// Returns the new level index (>= 0) or a negative status.
int tmpi_comm_push(const char* keys, const int* parent_members, int parent_size,
                   const char* my_key);
int tmpi_comm_num_levels(void);
int tmpi_comm_set(int level);                 // cursor -> (level, intra)
int tmpi_comm_set_typed(int level, int inter);
int tmpi_comm_level(void);
int tmpi_comm_is_inter(void);
int tmpi_comm_set_span(int begin, int end);
int tmpi_comm_get_span(int* begin, int* end);
int tmpi_comm_is_cartesian(int level);
// members of the intra (inter = 0) or inter (inter = 1) group of a level, as
// world ranks in group-rank order.  Returns the group size; fills at most cap.
int tmpi_comm_members(int level, int inter, int* out, int cap);
int tmpi_comm_rank_in(int level, int inter);
int tmpi_comm_key(int level, char* out, int cap);
// members of the communicator under the cursor (level 0 is always intra)
int tmpi_comm_current_members(int* out, int cap);
int tmpi_comm_group_of(int level, int world_rank, int* out, int cap);   // members of that rank's group at `level` (0: none)
int tmpi_comm_names(char* out, int cap);
int tmpi_comm_has_inter_collective(int level);
int tmpi_comm_has_intra_collective(int level);
int tmpi_comm_pop_to(int num_levels);          // drop levels above (tests)

// ---------------------------------------------------------------- ring plan
// Reduce-scatter / all-gather schedule of a chunked ring (one int pair per
// step and chunk): out[(step * total_chunks + c) * 2 + {0,1}] =
// {sender ring index, receiver ring index}.  phase 0 = reduce, 1 = broadcast.
int tmpi_ring_plan(int total_chunks, int size, int phase, int* out, int cap);
// chunk owned by `ring_index` to send / receive at `step` (-1 = none)
int tmpi_ring_send_chunk(int ring_index, int size, int step, int phase);
int tmpi_ring_recv_chunk(int ring_index, int size, int step, int phase);

// ---------------------------------------------------------------- handles
// An asynchronous operation is named by a 64-bit id.  wait frees the handle.
// timeout_ms < 0 waits for ever (bounded by the deadlock heuristic tunable).
int tmpi_handle_wait(uint64_t handle, int64_t timeout_ms);
int tmpi_handle_done(uint64_t handle);        // 1 done, 0 running, <0 unknown
// device-side wait: make `stream` wait for the handle's completion event
int tmpi_handle_stream_wait(uint64_t handle, void* stream);
int tmpi_sync_all(void);                       // drain both pools
int tmpi_handles_in_flight(void);
uint64_t tmpi_test_lost_handle(void);   // fault injection: a handle that never completes (a dropped request)
// test helpers: a host task that sleeps, then completes with `status`
uint64_t tmpi_test_sleep_task(int pool, int ms, int status);

// ---------------------------------------------------------------- host symmetric heap (POSIX shm)
// CPU ranks of one host map each other's segments; the same one-sided
// algorithms as the GPU data plane run on host threads.
int tmpi_shm_create(const char* name, size_t bytes, int rank, int world, void** base);
int tmpi_shm_attach(int peer, const char* name);
int tmpi_shm_ready(void);
int tmpi_shm_destroy(void);
size_t tmpi_shm_capacity(void);               // payload bytes per rank
void* tmpi_shm_base(int peer);
// members: heap ranks taking part, in group order; me = my index in members.
// `in`/`out` are ordinary host pointers; the heap is the bounce buffer.
int tmpi_shm_allreduce(const void* in, void* out, size_t n, int dtype, double scale,
                       const int* members, int nmembers, int me, int algo);
int tmpi_shm_broadcast(void* buf, size_t n, int dtype, int root,
                       const int* members, int nmembers, int me);
int tmpi_shm_reduce(const void* in, void* out, size_t n, int dtype, int root,
                    const int* members, int nmembers, int me);
int tmpi_shm_allgather(const void* in, void* out, size_t n_in, const int64_t* counts, int dtype,
                       const int* members, int nmembers, int me);
int tmpi_shm_barrier(const int* members, int nmembers, int me, int64_t timeout_ms);
uint64_t tmpi_shm_allreduce_async(const void* in, void* out, size_t n, int dtype, double scale,
                                  const int* members, int nmembers, int me, int algo);
uint64_t tmpi_shm_broadcast_async(void* buf, size_t n, int dtype, int root,
                                  const int* members, int nmembers, int me);

// ---------------------------------------------------------------- host parameter server (shm shards)
// One instance per tensor; shards live in the owner's heap segment; clients
// push/pull one-sidedly under a per-shard lock.  rule: 0 zero, 1 copy, 2 add.
int tmpi_ps_shard_range(size_t n, int size, int rank, size_t* begin, size_t* end);
int tmpi_shm_ps_init(const void* data, size_t n, int dtype,
                     const int* members, int nmembers, int me);   // returns instance id
int tmpi_shm_ps_free(int instance);
int tmpi_shm_ps_free_all(void);
uint64_t tmpi_shm_ps_send(int instance, const void* data, int rule);
uint64_t tmpi_shm_ps_receive(int instance, void* data);

// ---------------------------------------------------------------- CUDA symmetric heap
// backend 0: cudaMalloc + cudaIpc handles; backend 1: VMM + NVLS multicast.
int tmpi_cuda_set_device(int device);
int tmpi_cuda_heap_create(size_t bytes, int rank, int world, int backend);
int tmpi_cuda_heap_export(void* out, int cap);           // bytes to publish to peers
int tmpi_cuda_heap_import(int peer, const void* blob, int len);
int tmpi_cuda_heap_finish(void);                          // after all imports
int tmpi_cuda_heap_mc_export(void* out, int cap);         // rank 0 of the heap: multicast blob
int tmpi_cuda_heap_mc_import(const void* blob, int len);
int tmpi_cuda_heap_mc_bind(void);                         // after every rank added its device
int tmpi_cuda_heap_destroy(void);
void* tmpi_cuda_heap_base(int peer);
void* tmpi_cuda_heap_mc_base(void);                       // NULL when no multicast
size_t tmpi_cuda_heap_capacity(void);
size_t tmpi_cuda_heap_alloc(size_t bytes, size_t align);  // symmetric offset; (size_t)-1 on failure
int tmpi_cuda_heap_reset_allocator(size_t keep_bytes);
int tmpi_cuda_heap_world(void);
int tmpi_debug_bounds_build(void);                       // 1: peer accesses are bounds-checked and recorded (debug build)
// out[0..n): slots_off, slot_bytes, bounce_off, bounce_bytes, arena_off, total_bytes (per-rank mapping)
int tmpi_cuda_heap_layout(size_t* out, int n);
int tmpi_cuda_heap_rank(void);
// single-process emulation for tests on one GPU: `world` heaps on one device
int tmpi_cuda_heap_create_emulated(size_t bytes, int world);

// ---------------------------------------------------------------- CUDA collectives
// All buffers named by *offset* live in the symmetric heap; pointers are
// ordinary device pointers.  members/me select a sub-group of the heap's ranks.
// algo: 0 auto, 1 one-shot, 2 two-shot, 3 nvls, 4 ring.
// Every call is enqueued on `stream` and returns at once.
typedef struct {
  const int* members; int nmembers; int me; int lane;
} tmpi_group_t;

int tmpi_cuda_allreduce(const void* in, void* out, size_t n, int dtype, double scale,
                        const tmpi_group_t* g, int algo, void* stream);
int tmpi_cuda_allreduce_heap(size_t in_off, size_t out_off, size_t n, int dtype, double scale,
                             const tmpi_group_t* g, int algo, void* stream);
int tmpi_cuda_broadcast(void* buf, size_t n, int dtype, int root,
                        const tmpi_group_t* g, void* stream);
int tmpi_cuda_broadcast_heap(size_t off, size_t n, int dtype, int root,
                             const tmpi_group_t* g, int algo, void* stream);
int tmpi_cuda_reduce(const void* in, void* out, size_t n, int dtype, int root,
                     const tmpi_group_t* g, void* stream);
int tmpi_cuda_allgather(const void* in, void* out, size_t n_in, int dtype,
                        const tmpi_group_t* g, void* stream);
int tmpi_cuda_allgatherv(const void* in, void* out, size_t n_in, const int64_t* counts,
                         int dtype, const tmpi_group_t* g, void* stream);
int tmpi_cuda_reduce_scatter(const void* in, void* out, size_t n_out, int dtype, double scale,
                             const tmpi_group_t* g, void* stream);
int tmpi_cuda_barrier(const tmpi_group_t* g, void* stream);
// asynchronous flavours: a pool thread owning a comm stream launches the
// kernel after `stream`'s current work and returns a handle.
uint64_t tmpi_cuda_allreduce_async(const void* in, void* out, size_t n, int dtype, double scale,
                                   const tmpi_group_t* g, int algo, void* stream);
uint64_t tmpi_cuda_broadcast_async(void* buf, size_t n, int dtype, int root,
                                   const tmpi_group_t* g, void* stream);
// device status word of the last collective on `lane` (0 ok); clears it
int tmpi_cuda_collective_status(int lane, int* code, int* where, int* peer);
int tmpi_cuda_set_wait_budget_ms(int64_t ms);
// test helper: run a wait on a flag that nobody sets, return the status code
int tmpi_cuda_test_wait_timeout(int64_t budget_ms, void* stream);

// fused gradient allreduce + SGD(momentum) step over a flat bucket in the heap.
typedef struct {
  size_t grad_off;      // heap offset of the gradient bucket (grad_dtype)
  size_t weight_off;    // heap offset of the working weights (weight_dtype)
  void* master;         // fp32 master shard of this rank (NULL: weights are the master)
  void* momentum;       // fp32 momentum shard of this rank (NULL: no momentum)
  size_t n;             // elements in the bucket (multiple of 8 * nmembers)
  int grad_dtype, weight_dtype;
  float lr, momentum_coef, dampening, weight_decay, grad_scale;
  int nesterov, first_step, zero_grads;
} tmpi_sgd_bucket_t;
int tmpi_cuda_allreduce_sgd(const tmpi_sgd_bucket_t* b, const tmpi_group_t* g, int algo, void* stream);

// ---------------------------------------------------------------- CUDA parameter server
int tmpi_cuda_ps_push(size_t shard_off, const void* data, size_t n, int dtype, int rule,
                      const tmpi_group_t* g, void* stream);
int tmpi_cuda_ps_pull(size_t shard_off, void* data, size_t n, int dtype,
                      const tmpi_group_t* g, void* stream);
uint64_t tmpi_cuda_ps_push_async(size_t shard_off, const void* data, size_t n, int dtype, int rule,
                                 const tmpi_group_t* g, void* stream);
uint64_t tmpi_cuda_ps_pull_async(size_t shard_off, void* data, size_t n, int dtype,
                                 const tmpi_group_t* g, void* stream);

// ---------------------------------------------------------------- single-GPU hot ops
int tmpi_sgd_momentum(void* weight, int weight_dtype, const void* grad, int grad_dtype,
                      void* master, void* momentum, size_t n, float lr, float momentum_coef,
                      float dampening, float weight_decay, float grad_scale, int nesterov,
                      int first_step, int zero_grads, void* stream);
// scratch: tmpi_xent_scratch_bytes(rows) bytes, zeroed once before the first call
size_t tmpi_xent_scratch_bytes(int rows);
int tmpi_xent_fwd_bwd(const void* logits, int dtype, const int64_t* labels, int rows, int cols,
                      float* loss_sum, void* dlogits, float grad_scale, void* scratch, void* stream);
// the same with a row pitch `ld` (elements) for logits and dlogits; dlogits columns cols..ld-1 are zeroed
int tmpi_xent_fwd_bwd_ld(const void* logits, int dtype, const int64_t* labels, int rows, int cols, int ld,
                      float* loss_sum, void* dlogits, float grad_scale, void* scratch, void* stream);
int tmpi_absmean_var(const void* x, int dtype, size_t n, double* out2, void* scratch, void* stream);
size_t tmpi_absmean_var_scratch_bytes(void);
int tmpi_easgd_elastic(void* local, const void* center, void* delta, size_t n, int dtype,
                       float alpha, void* stream);
int tmpi_downpour_accum(void* accum, const void* grad, size_t n, int dtype, float scale,
                        int zero_first, void* stream);
// bias gradient of a linear layer: db[c] = sum_r dz[r, c]; with z given, dz = dy * gelu'(z) is computed and
// written in the same pass (channels a multiple of 1024 for 16-bit types, 512 for fp32)
size_t tmpi_bias_grad_scratch_bytes(int channels);
int tmpi_bias_grad(const void* dy, const void* z, void* dz, void* db, int rows, int channels, int dtype,
                   void* scratch, void* stream);
// y = gelu(z), erf form, n elements (a multiple of 16 bytes, pointers 16-byte aligned)
int tmpi_gelu_fwd(const void* z, void* y, size_t n, int dtype, void* stream);
// layer normalisation over the last dimension of [rows, channels]; x, y, gamma, beta share the dtype;
// mean / rstd ([rows], fp32) are written by forward and read by backward
int tmpi_layernorm_supported(int channels, int dtype);
size_t tmpi_layernorm_scratch_bytes(int channels);
int tmpi_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd,
                       int rows, int channels, float eps, int dtype, void* stream);
int tmpi_layernorm_bwd(const void* x, const void* dy, const void* gamma, const float* mean, const float* rstd,
                       void* dx, void* dgamma, void* dbeta, int rows, int channels, int dtype, void* scratch,
                       void* stream);
int tmpi_bn_relu_fwd(const void* x, const void* residual, void* y, const float* gamma,
                     const float* beta, float* running_mean, float* running_var,
                     float* save_mean, float* save_invstd, int64_t rows, int channels,
                     float eps, float momentum, int relu, int training, int dtype,
                     void* mask_bits, void* scratch, void* stream);
int tmpi_bn_relu_bwd(const void* x, const void* y, const void* dy, void* dx, void* dresidual,
                     const float* gamma, const float* beta, const float* save_mean, const float* save_invstd,
                     float* dgamma, float* dbeta, int64_t rows, int channels, int relu, int dtype,
                     const void* mask_bits, void* scratch, void* stream);
int tmpi_bn_relu_bwd_acc(const void* x, const void* y, const void* dy, void* dx, void* dresidual, const float* gamma,
                         const float* beta, const float* save_mean, const float* save_invstd, float* dgamma, float* dbeta,
                         int64_t rows, int channels, int relu, int dtype, const void* mask_bits, void* scratch,
                         float* acc_gamma, float* acc_beta, void* stream);
size_t tmpi_bn_scratch_bytes(int channels);
// training forward of the same stage when the producer of x already left `partial_rows` rows of partial
// sums, [row][2][channels] floats, in `partials` (the statistics pass is skipped)
int tmpi_bn_relu_fwd_partials(const void* x, const void* residual, void* y, const float* gamma, const float* beta,
                              float* running_mean, float* running_var, float* save_mean, float* save_invstd, int64_t rows,
                              int channels, float eps, float momentum, int relu, int dtype, void* mask_bits,
                              void* partials, int partial_rows, void* stream);

// ---------------------------------------------------------------- convolutions as implicit GEMMs (conv_gemm.cu)
// bf16, channels-last, dense; x [N, H, W, Cin], w [Cout, R, S, Cin] (a channels-last Conv2d weight as it lies),
// y [N, Ho, Wo, Cout]; Cin and Cout multiples of 64, square filters.
int tmpi_conv_max_ctas(void);
int tmpi_conv_fwd(const void* x, const void* w, void* y, int N, int H, int W, int Cin, int Cout, int R, int S, int stride,
                  int pad, float* stats, int* stat_rows, void* stream);
int tmpi_conv_dgrad(const void* dy, const void* w, void* dx, const void* add, int N, int H, int W, int Cin, int Cout, int R,
                    int S, int stride, int pad, void* stream);
size_t tmpi_conv_wgrad_workspace_bytes(int N, int H, int W, int Cin, int Cout, int R, int S, int stride, int pad);
int tmpi_conv_wgrad(const void* dy, const void* x, void* dw, int N, int H, int W, int Cin, int Cout, int R, int S,
                    int stride, int pad, void* workspace, size_t workspace_bytes, int accumulate, void* stream);
int tmpi_conv_status(void);
// causal self-attention forward, head size 64, bf16: q, k, v as [B * T, H * 64] matrices with one row pitch (the column
// blocks of a fused QKV projection), out [B * T, ld_out], lse [B, H, T] fp32 (optional); T a multiple of 128
int tmpi_attention_fwd(const void* q, const void* k, const void* v, int64_t ld_qkv, void* out, int64_t ld_out, float* lse,
                       int B, int T, int H, float scale, void* stream);
// gradients: o and dout [B * T, H * 64] with their own pitches, lse from the forward, delta [B, H, T] scratch, dq_acc a
// fp32 [B * T, H * 64] buffer (cleared by the call) that receives dQ, dq (optional: dq_acc rounded) / dk / dv bf16 [B * T, ld_dkv]
int tmpi_attention_bwd(const void* q, const void* k, const void* v, int64_t ld_qkv, const void* o, int64_t ld_o,
                       const void* dout, int64_t ld_do, const float* lse, float* delta, float* dq_acc, void* dq, void* dk,
                       void* dv, int64_t ld_dkv, int B, int T, int H, float scale, void* stream);
int tmpi_attention_bwd_status(void);
void tmpi_attention_bwd_set_trace(void* device_buffer);   // tuning aid, as for the forward
int tmpi_attention_ctas_per_sm(void);
void tmpi_attention_set_v_stages(int n);              // tuning aid: 1 or 2 V buffers per CTA
void tmpi_attention_set_trace(void* device_buffer);   // tuning aid: phase time stamps of one CTA
int tmpi_attention_status(void);
// C[M, N] (+)= A^T B for A [K, M], B [K, N] with a long K and a small output (split over K; same kernel family)
size_t tmpi_gemm_tn_splitk_workspace_bytes(int M, int N, int64_t K);
int tmpi_gemm_bf16_tn_splitk(const void* A, const void* B, void* C, int M, int N, int64_t K, int64_t lda, int64_t ldb,
                             void* workspace, size_t workspace_bytes, int accumulate, void* stream);
// batch-norm + ReLU + max-pool (3x3, stride 2, pad 1) as one stage; y, idx: [N, (H-1)/2+1, (W-1)/2+1, C]
int tmpi_bn_relu_pool_fwd(const void* x, void* y, void* idx, const float* gamma, const float* beta,
                          float* running_mean, float* running_var, float* save_mean, float* save_invstd,
                          int N, int H, int W, int channels, float eps, float momentum, int training,
                          int dtype, void* scratch, void* stream);
int tmpi_bn_relu_pool_bwd(const void* x, const void* dy, const void* idx, void* dx, const float* gamma,
                          const float* beta, const float* save_mean, const float* save_invstd,
                          float* dgamma, float* dbeta, int N, int H, int W, int channels, int dtype,
                          void* scratch, void* stream);
// channels-last max pooling; idx holds one byte per output element (position inside the window)
int tmpi_maxpool_fwd(const void* x, void* y, void* idx, int N, int H, int W, int C, int OH, int OW,
                     int k, int s, int p, int dtype, void* stream);
int tmpi_maxpool_bwd(const void* dy, const void* idx, void* dx, int N, int H, int W, int C, int OH, int OW,
                     int k, int s, int p, int dtype, void* stream);

// Patch matrix of a 7x7 / stride 2 / pad 3 convolution over a channels-last input with 3 channels:
// col[N*OH*OW, tmpi_stem_patch_width()] in (kh, kw, c) order, zero padded (the stem as a GEMM).
int tmpi_stem_im2col(const void* x, void* col, int N, int H, int W, int dtype, void* stream);
int tmpi_stem_patch_width(void);

// ---------------------------------------------------------------- tcgen05 GEMM family
// C[M,N] = act(A[M,K] * B[N,K]^T (+ bias)), bf16 in, fp32 accumulate in TMEM.
int tmpi_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                   int epilogue, void* stream);
// explicit row pitches (elements, multiples of 8) of A, B, C as stored; M, N >= 256
int tmpi_gemm_bf16_ex(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                      int64_t lda, int64_t ldb, int64_t ldc, int epilogue, void* stream);

// ---------------------------------------------------------------- tracing
// ring buffer of (op, algo, bytes, microseconds) records per process
int tmpi_trace_enable(int on);
int tmpi_trace_record(const char* op, const char* algo, uint64_t bytes, double us);
int tmpi_trace_dump(char* out, int cap);  // JSON lines
int tmpi_trace_clear(void);

#ifdef __cplusplus
}
#endif
