/* Column sums (bias gradient) without any allocation.
 *
 * This entry point has no counterpart in the reference: the reference has no
 * model kernels at all, and its own kernels take scratch that a hook allocated
 * with cudaMalloc at communicator creation.
 *
 * Who needs it.  Some programs that load this library may not allocate device
 * memory at the moment they call in: a serving process whose whole HBM was
 * handed to another allocator at start-up (a later cudaMalloc simply fails), or
 * a latency-critical loop that cannot afford the device-wide synchronisation
 * cudaMalloc / cudaFree imply.  The regular entry point, piccl_ops_colsum, makes
 * the caller pass a workspace; this variant keeps its workspace in a fixed
 * array inside the library image instead, so the caller passes only input and
 * output.
 *
 *   out[c] (+)= sum over r < rows of x[r, c]        x: bf16 [rows, C] row-major, out: bf16 [C]
 *
 * Limits and rules
 *  - C must be a multiple of 8 and at most PICCL_OPS_COLSUM_NOALLOC_MAX_COLS (16384); rows >= 1 (any
 *    number: the rows are folded into at most 64 partial sums).  Anything else is rejected with
 *    a message on stderr and a negative return value; nothing is launched.
 *  - x must be 16-byte aligned (it is read 8 bf16 at a time); a view that starts at an odd element
 *    offset is refused (-7), not faulted on.  out needs only the alignment of a bf16.
 *  - The workspace is 64 x 16384 floats = 4 MiB.  Every GPU that loads the library holds it until
 *    the process exits, used or not.  With CUDA's default lazy module loading the GPU only sets the
 *    array up when the library's code is first used on that device, i.e. at the FIRST CALL: make
 *    that call before the rest of the device memory is handed to another allocator and before the
 *    latency-critical loop starts, or run with CUDA_MODULE_LOADING=EAGER; otherwise the first call
 *    can fail with -5 / -6 or take unusually long.
 *  - The first call on a device looks up the device address of the workspace (that device must be
 *    current, as for every call).  Make that first call outside any stream capture.
 *  - All calls on one device share the one workspace and it keeps what the last call left there.
 *    Nothing in it has to start at zero (every partial sum that is read was written by the same
 *    call), but two calls that overlap on the GPU (different streams, no ordering between them)
 *    race on it and both results are undefined.  Order them with events or use one stream.
 *  - No cudaMalloc, cudaFree or allocating library routine is called by this function, on the first call or later.
 *
 * Returns 0 after the launches were issued on `stream`;
 *   -1 bad C (not a multiple of 8, or < 8)     -2 C above the maximum     -3 rows < 1
 *   -4 null pointer                            -5 the workspace address could not be obtained
 *   -6 launch failure (the CUDA error is printed)     -7 x is not 16-byte aligned
 */
#ifndef PICCL_OPS_COLSUM_NOALLOC_H
#define PICCL_OPS_COLSUM_NOALLOC_H

#define PICCL_OPS_COLSUM_NOALLOC_MAX_COLS 16384
#define PICCL_OPS_COLSUM_NOALLOC_MAX_PARTS 64

#ifdef __cplusplus
extern "C" {
#endif

int piccl_ops_colsum_noalloc(const void* x, void* out, int rows, int C, int accumulate, void* stream);

#ifdef __cplusplus
}
#endif
#endif
