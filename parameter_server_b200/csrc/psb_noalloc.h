// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference implementation; it exists
// for embedders of this library, not for parity.
//
// Who needs it: code that must not (or cannot) obtain device memory at call time.
// Examples are a solver running as a plug-in inside a host application that has
// handed all of HBM to its own pool and forbids foreign cudaMalloc calls, a
// monitoring hook that computes the objective from inside a latency-critical
// serving loop where cudaMalloc's device-wide synchronisation is unacceptable,
// and C or Fortran callers that link only against this .so and have no allocator
// (torch's or any other) to borrow scratch space from.
//
// What it is: psb_reduce_sum (reduce_kernels.cu) with its scratch space moved
// into a fixed array that lives in the library's device image.  Every GPU that
// loads the library holds that array (8448 bytes) until the process exits.
#pragma once
#include <cstddef>
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest input accepted, in elements (2^31 floats = 8 GiB).  Larger inputs are
// rejected with cudaErrorInvalidValue and a message on stderr.
#define PSB_REDUCE_STATIC_MAX_ELEMS (1ull << 31)

// out[0] = Σ term_op(x[i]) for i < n, accumulated in fp64 in a fixed order.
//   x      device pointer, n floats (caller-owned input)
//   op     0 Σlog(1+1/x)  1 Σ|x| over finite non-zero x  2 #{x != 0, not NaN}  3 Σlog(1+e^-x)  4 Σmax(0,1-x)²
//   out    device pointer to one double (caller-owned output)
//   stream stream to launch on
// Returns 0 or a cudaError_t value.
//
// The function calls no cudaMalloc/cudaFree and no allocating library routine.
// * Every call asks the runtime for the device address of the built-in scratch
//   array (cudaGetSymbolAddress, with the caller's device current).  The first
//   such call on a device makes the runtime load the library's device image
//   there: make it during start-up, before any stream capture begins on that
//   device.  Later calls are answered from the runtime's tables.  Nothing is
//   remembered inside this library, so a cudaDeviceReset between calls is safe
//   (the array's contents are lost, which no call depends on).
// * All calls on one device share the one scratch array.  The word that must be
//   zero at launch is cleared on `stream` before every launch, but two calls
//   whose kernels overlap on the GPU (different streams, no dependency) race on
//   the partial sums and give wrong results: serialise them.
int psb_reduce_sum_static(const float* x, size_t n, int op, double* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
