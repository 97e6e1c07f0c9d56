// Column sum without any allocation, for callers that cannot allocate.
//
// This entry point has no counterpart in the reference: it is an addition of this library.
//
// The regular column-sum (`_C.colsum`, used for bias gradients) asks torch's caching allocator for a buffer of
// per-slice partial sums on every call.  Some callers cannot do that: code that runs while the process must not
// touch any allocator (a memory-accounting pass that compares allocator statistics before and after, a hook that
// runs inside an allocator callback, a host program that links this library without torch and owns all device
// memory itself).  For them this variant keeps the partial sums in a fixed array inside the library's device
// image, so a call only launches two kernels on the stream it is given.
//
//   out[j] (+)= sum over r < rows of a[r * lda + j],   j < n,  `a` bf16 on the device, `out` fp32 on the device.
//
// Limits and rules:
//   * `a` and `out` must be 4-byte aligned (`a` is read two bf16 values at a time): a bf16 view that starts on an odd
//     element is refused with SSB_COLSUM_STATIC_E_BAD_ARG and nothing is launched.
//   * n must be even, at most SSB_COLSUM_STATIC_MAX_N (8192); lda must be even and >= n; rows >= 1.  Larger sizes
//     are refused with SSB_COLSUM_STATIC_E_TOO_LARGE and nothing is launched.  The array holds
//     128 x 8192 floats = 4 MiB per device.
//   * The first call on each device looks up the array's address on that device (with that device current).
//     That lookup is not a stream operation, so make the first call on a device before you begin capturing
//     a stream on it.  Later calls on that device only launch kernels.
//   * Every call on a device uses the same array.  Nothing in it has to be zero when a call starts: the first
//     kernel writes every partial sum the second one reads.  Two calls that may run at the same time on one
//     device (different streams, or different host threads on different streams) race on the array; order them
//     on one stream or with events.
//   * The call makes `a`'s device current neither for you nor for itself: call it with the device that owns
//     `a` and `out` current.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define SSB_COLSUM_STATIC_MAX_N 8192
#define SSB_COLSUM_STATIC_MAX_SLICES 128

#define SSB_COLSUM_STATIC_OK 0
#define SSB_COLSUM_STATIC_E_BAD_ARG 1     /* null or misaligned pointer, rows < 1, n < 2, odd n or lda, lda < n */
#define SSB_COLSUM_STATIC_E_TOO_LARGE 2   /* n > SSB_COLSUM_STATIC_MAX_N */
#define SSB_COLSUM_STATIC_E_SETUP 3       /* the address lookup of the scratch array failed on this device */
#define SSB_COLSUM_STATIC_E_LAUNCH 4      /* a kernel launch was rejected */

// `stream` is a cudaStream_t (null = the default stream).  Returns one of the codes above.
int ssb_colsum_bf16_static(const void* a, long long lda, float* out, int accumulate, int rows, int n, void* stream);

// A short description of a return code of ssb_colsum_bf16_static (static storage, never null).
const char* ssb_colsum_static_strerror(int code);

#ifdef __cplusplus
}
#endif
