// Allocation-free entry point of liboslo_b200_cuda.  This has no counterpart in the reference library
// (EleutherAI/oslo): there every kernel wrapper allocates its work buffers through the PyTorch allocator.
//
// Why it exists.  Some callers of these kernels are not allowed to allocate device memory at the moment
// of the call: code that runs inside a region where cudaMalloc is forbidden or would deadlock (a stream
// being captured, a callback on a CUDA stream, a collective's critical section), and C or C++ hosts that
// link this library without PyTorch and its caching allocator and have handed all of the GPU's memory to
// their own pools already.  The ordinary column-sum entry point, oslo_colsum, needs a scratch buffer of
// parts x H floats that such a caller would have to obtain somewhere.
//
// What it does.  oslo_colsum_noalloc computes out[c] = sum over rows of x[r, c] with the same two kernels
// as oslo_colsum, but keeps the per-block partial sums in a fixed array that is part of the library image
// (OSLO_COLSUM_NOALLOC_MAX_SCRATCH_FLOATS floats = 8 MiB, resident on every GPU that loads the library until
// the process exits).  The caller passes only the input and the output.  It calls no cudaMalloc, cudaFree
// or any routine that allocates, PyTorch's included.
//
// Rules of use.
//   * Limit: H (the number of columns) must not exceed OSLO_COLSUM_NOALLOC_MAX_SCRATCH_FLOATS; larger inputs are
//     refused with OSLO_NOALLOC_ERR_TOO_LARGE and a message on stderr.  When parts x H would not fit, fewer row
//     partitions are used, which only costs speed.  H must be a multiple of 4 (fp32) or 8 (fp16 / bf16), and
//     x and out must be 16-byte aligned, as for oslo_colsum; a misaligned or null pointer is refused with
//     OSLO_NOALLOC_ERR_ARGUMENT before anything is launched.
//   * First call on a device: the first call made while a given device is current looks up the device address
//     of the array and the SM count for that device and remembers them.  Make that first call outside any
//     stream capture; later calls on the device only launch kernels.
//   * One array for everybody: all calls on a device share the array, and it keeps whatever the last call
//     left in it.  Every cell a call reads is written by that same call first, so nothing needs clearing, but
//     two calls whose kernels overlap in time on one GPU (different streams) race on it.  Serialise them: use
//     one stream, or order the streams with events.
//   * The call is asynchronous on `stream`, like the other entry points; the result is ready when the stream
//     reaches that point.
#pragma once

#define OSLO_COLSUM_NOALLOC_MAX_SCRATCH_FLOATS (1LL << 21)

#define OSLO_NOALLOC_ERR_ARGUMENT (-1)   /* bad dtype code, H not a multiple of the vector width, or x / out null or not 16-byte aligned */
#define OSLO_NOALLOC_ERR_LAUNCH (-2)     /* a kernel launch failed */
#define OSLO_NOALLOC_ERR_TOO_LARGE (-10) /* H exceeds the built-in scratch */
#define OSLO_NOALLOC_ERR_SETUP (-11)     /* the one-time look-up of the scratch address failed */
#define OSLO_NOALLOC_ERR_DEVICE (-12)    /* no current device, or a device ordinal >= 64 */

#ifdef __cplusplus
extern "C" {
#endif

// x: [rows, H] row-major, out: [H]; dtype 0 = fp32, 1 = fp16, 2 = bf16 (input and output alike).
// stream: a cudaStream_t (0 for the default stream).  Returns 0 or one of the codes above.
int oslo_colsum_noalloc(const void* x, void* out, long long rows, int H, int dtype, void* stream);

// The size of the built-in scratch array, in floats.
long long oslo_colsum_noalloc_max_scratch_floats(void);

#ifdef __cplusplus
}
#endif
