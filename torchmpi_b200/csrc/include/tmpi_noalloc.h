// An entry point for callers that must not allocate GPU memory.
//
// This has no counterpart in the reference (facebookarchive/TorchMPI has no loss kernel and no
// allocation-free call of any kind); it is an addition of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits.  Examples: a step callback of a
// host framework that forbids allocation once training has started; a latency-critical loop that
// may not enter the driver's allocator (cudaMalloc can synchronise the whole device); a process
// whose GPU memory has all been handed to another memory pool, so that one more cudaMalloc may
// simply fail.  Such a caller cannot provide the scratch buffer that tmpi_xent_fwd_bwd asks for
// without allocating it first.
//
// tmpi_xent_fwd_bwd_noalloc computes exactly what tmpi_xent_fwd_bwd computes (softmax
// cross-entropy over [rows, cols] logits: the summed loss in loss_sum[0] and, if dlogits is not
// NULL, (softmax - onehot) * grad_scale), but takes no scratch argument: its scratch is an array
// compiled into the library's device image.  The call performs no cudaMalloc, cudaFree or any
// other allocating routine; the caller still passes the input and output buffers.
//
// Limits and rules:
//  * rows <= TMPI_XENT_NOALLOC_MAX_ROWS; more rows are rejected with TMPI_ERR_INVALID and a
//    message (use tmpi_xent_fwd_bwd with your own scratch then).  cols is not limited.
//  * The array costs 256 + 4 * TMPI_XENT_NOALLOC_MAX_ROWS bytes (about 64 KiB) on every GPU
//    that loads the library, until the process exits.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current) and remembers it.  Make that first call during set-up, before any
//    stream capture begins.
//  * All calls on a device share the array.  Calls whose kernels may run at the same time on one
//    device (different streams) race on it: serialise them, e.g. by using one stream.
#pragma once
#include <stdint.h>

#define TMPI_XENT_NOALLOC_MAX_ROWS 16384

#ifdef __cplusplus
extern "C" {
#endif

int tmpi_xent_fwd_bwd_noalloc(const void* logits, int dtype, const int64_t* labels, int rows, int cols,
                              float* loss_sum, void* dlogits, float grad_scale, void* stream);

#ifdef __cplusplus
}
#endif
