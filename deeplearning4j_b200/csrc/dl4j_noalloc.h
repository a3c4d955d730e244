// Entry points of this library that perform no device or host allocation of their own.
//
// There is no counterpart to this header in the reference project; it exists for embedders of this
// library whose call sites are not allowed to allocate:
//   * a host runtime that carved up all device memory ahead of time (a fixed arena / workspace plan,
//     in the spirit of ND4J workspaces) and treats any allocation inside the training loop as a bug;
//   * code running where an allocation would stall everything else, because cudaMalloc / cudaFree
//     synchronise the whole device and serialise against work on other streams;
//   * plain C callers that have no tensor allocator to ask for a temporary buffer.
// Such callers hand in every input and output buffer; the only working memory the routine needs lives
// in a fixed-size device array that is part of the library image itself.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Limits of dl4j_layer_norm_bwd_noalloc.  The scratch array is sized for exactly these.
#define DL4J_NOALLOC_LN_MAX_C 1024      /* widest normalised axis (elements)                     */
#define DL4J_NOALLOC_LN_MAX_BLOCKS 296  /* thread blocks that may park partial sums in scratch   */
#define DL4J_NOALLOC_LN_MAX_ROWS 2147483647LL

// Layer-norm backward over a [rows, C] activation (same math as dl4j_layer_norm_bwd):
//   dx    = rstd * (dy*gain - mean_C(dy*gain) - xhat * mean_C(dy*gain*xhat)),  xhat = (x - mean) * rstd
//   dgain = sum_rows dy * xhat,   dbias = sum_rows dy
// Unlike dl4j_layer_norm_bwd, which adds into dgain / dbias with floating-point atomics, this variant
// parks one partial sum per thread block in scratch memory and lets the last block to finish add them
// up in block order, so the parameter gradients are bit-reproducible from call to call.
//   accumulate == 0: dgain / dbias are overwritten;  accumulate != 0: the sums are added to their contents.
//   dtype: 0 = float16, 1 = bfloat16, 2 = float32 (dy, x, dx; the codes every entry point of the library uses); gain, mean, rstd, dgain, dbias are float32.
//   dgain and dbias may be null (that gradient is then skipped).
//   Alignment: dy, x, dx and gain must start on a 16-byte boundary (they are moved with 16-byte vector accesses; with
//   C % 8 == 0 every row then keeps that alignment); mean, rstd, dgain and dbias on a 4-byte boundary.  A pointer that
//   breaks this is rejected with -6 before anything is launched.
//   `stream` must belong to the device that is current at the call: the scratch address is looked up for the current
//   device, and a stream of another device is not supported.
//
// Memory: the routine allocates nothing (no cudaMalloc / cudaFree, no allocating library call).  Its
// scratch (256 B of counters + DL4J_NOALLOC_LN_MAX_BLOCKS * 2 * DL4J_NOALLOC_LN_MAX_C floats, about
// 2.3 MiB) is a file-scope __device__ array.  The first call on each device looks up that array's
// device address (cudaGetSymbolAddress, with that device current); this one-time set-up may load the
// module, so make the first call per device before any stream capture begins.
// The counter block has to be zero when the kernel starts: the call clears it on `stream` ahead of the
// launch, and the kernel leaves it zero again.  The partial sums need no clearing.
// All calls on one device share the one scratch array: calls that may overlap in time (different
// streams, or several host threads) race on it and must be serialised by the caller.
//
// Returns 0 on success; -6 for sizes beyond the limits above (C % 8 != 0, C > DL4J_NOALLOC_LN_MAX_C,
// rows < 1), a bad dtype, a null or misaligned pointer -- a one-line reason is written to stderr; a positive value
// is a cudaError_t from set-up or launch.
int dl4j_layer_norm_bwd_noalloc(const void* dy, const void* x, const float* gain, const float* mean, const float* rstd,
                                void* dx, float* dgain, float* dbias, long long rows, int C, int dtype, int accumulate,
                                void* stream);

#ifdef __cplusplus
}
#endif
