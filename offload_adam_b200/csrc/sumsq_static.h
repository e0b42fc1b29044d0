// Squared L2 norm of a bf16 buffer without any allocation, as a plain C symbol.
//
// This entry point has no counterpart in the reference optimizer.  It exists for hosts
// that may not allocate device memory at the moment they need a gradient norm: a
// process whose own pool already owns the whole GPU (a serving engine, a trainer whose
// caching allocator is capped at the device size), where a driver allocation can fail
// outright or force a device-wide synchronisation in the middle of a step, and callers
// that are not linked against PyTorch at all and therefore cannot borrow its allocator.
//
// The reduction needs a little global memory of its own (one partial sum per thread
// block and a ticket counter).  Here that scratch is a fixed array compiled into the
// library image, so the caller passes only the input and the output.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest input the fixed scratch can serve: 65536 blocks of 8192 elements.
#define OAB_SUMSQ_STATIC_MAX_ELEMS (65536LL * 8192LL)

// Return codes.
#define OAB_STATIC_OK 0
#define OAB_STATIC_BAD_ARGUMENT 1   // null pointer or negative length
#define OAB_STATIC_TOO_LARGE 2      // n > OAB_SUMSQ_STATIC_MAX_ELEMS
#define OAB_STATIC_CUDA_ERROR 3     // a CUDA call failed; see the message

// *out = sum_i float(x[i])^2 over n bfloat16 values, accumulated in fp32 in a fixed
// order (the result is reproducible for a given n).
//
//   x       device pointer to n bfloat16 values (any alignment; 32-byte aligned
//           buffers take the vector path)
//   n       0 <= n <= OAB_SUMSQ_STATIC_MAX_ELEMS; larger inputs are refused with
//           OAB_STATIC_TOO_LARGE and nothing is launched
//   out     device pointer to one float, overwritten
//   stream  cudaStream_t on which the work is enqueued (NULL: default stream).  It has
//           to belong to the device that is current in the calling thread, which is also
//           the device x and out live on: with a stream of another device the memset or
//           the launch fails and the call returns OAB_STATIC_CUDA_ERROR
//   err     optional buffer that receives a readable message on failure
//   err_len size of that buffer in bytes
//
// The call enqueues a 4-byte memset and one kernel on `stream` and returns without
// waiting.  It performs no device or host allocation of any kind.
//
// The first call made on a device looks up the address of the built-in scratch array
// (one cudaGetSymbolAddress while that device is current) and remembers it; make that
// first call outside any stream capture.
//
// All calls on a device share the one scratch array (256 KiB + a counter, resident in
// every GPU that loads the library until the process exits).  It still holds what the
// previous call left there: the counter is cleared at the start of each call, the
// partial sums are overwritten before they are read.  Two calls whose kernels can
// overlap on the GPU (different streams without an ordering between them) race on the
// array and give wrong sums; order them on one stream or with events.
int oab_sumsq_bf16_static(const void* x, long long n, float* out, void* stream, char* err,
                          int err_len);

#ifdef __cplusplus
}
#endif
