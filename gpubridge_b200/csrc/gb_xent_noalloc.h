/* Fused cross-entropy for callers that must not allocate.
 *
 * This entry point has no counterpart in the reference project; it exists for embedders of
 * this library.
 *
 * Who needs it.  gb_xent_fwd_bwd() asks its caller for scratch memory (one float per row and
 * a counter).  Some callers have nowhere to get it from: code that runs inside somebody
 * else's memory pool and may not call cudaMalloc behind its back (a plugin of an inference
 * server, an operator registered into a framework that owns all device memory), code on a
 * path where an allocation could synchronise the device or fail at a bad moment (a step that
 * has to keep a latency bound, an out-of-memory handler), and bare C programs that link the
 * library without torch and do not want an allocator of their own.  For them the scratch
 * is a fixed array inside the library.
 *
 * What it does.  Same arguments and same results as gb_xent_fwd_bwd(), minus the two scratch
 * pointers: `logits` ([rows, ld] row-major, bf16 when dtype is 1, fp32 when 0, 16-byte
 * aligned, ld a multiple of 8 resp. 4) is overwritten with the gradient of the mean loss,
 * the mean loss goes to `loss_out` (device memory), `targets` are int64 class indices.  The
 * caller still owns inputs and outputs.  The call itself never calls cudaMalloc, cudaFree or
 * any routine that allocates.
 *
 * Limits and rules.
 *  - rows <= GB_XENT_NOALLOC_MAX_ROWS (65536).  More rows are refused with
 *    GB_XENT_NOALLOC_TOO_MANY_ROWS before anything is launched; gb_xent_noalloc_error()
 *    turns any return code into text.  Every GPU that loads the library holds the array
 *    (256 KiB + 256 bytes) until the process exits.
 *  - The first call on a device looks the array's address up (cudaGetSymbolAddress, with that
 *    device current) and keeps it; make that first call before you start capturing a stream,
 *    with the device you will run on already current.
 *  - All calls on one device share the one array, and it keeps what the last call left in it.
 *    The counter in it is cleared on the stream at the start of every call.  Two calls that
 *    overlap on the GPU (different streams, no ordering between them) race on the array and
 *    give wrong losses: order them on one stream or with events.
 */
#ifndef GB_XENT_NOALLOC_H
#define GB_XENT_NOALLOC_H

#include <cuda_runtime.h>
#include <stddef.h>

#define GB_XENT_NOALLOC_MAX_ROWS 65536
#define GB_XENT_NOALLOC_TOO_MANY_ROWS (-2)

#ifdef __cplusplus
extern "C" {
#endif

/* The existing entry point: scratch supplied by the caller. */
int gb_xent_fwd_bwd(void* logits, int dtype, const long long* targets, size_t rows, size_t vocab,
                    size_t ld, float* row_loss, unsigned int* counter, float* loss_out,
                    cudaStream_t stream);

/* The same computation with the scratch inside the library.  Returns 0, a cudaError_t, or
 * GB_XENT_NOALLOC_TOO_MANY_ROWS. */
int gb_xent_fwd_bwd_noalloc(void* logits, int dtype, const long long* targets, size_t rows,
                            size_t vocab, size_t ld, float* loss_out, cudaStream_t stream);

const char* gb_xent_noalloc_error(int code);

#ifdef __cplusplus
}
#endif
#endif
