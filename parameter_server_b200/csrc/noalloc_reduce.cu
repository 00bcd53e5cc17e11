// psb_reduce_sum_static: the deterministic sum reduction with built-in scratch space,
// for callers that cannot allocate device memory (see psb_noalloc.h).
#include <cstdio>

#include "psb_noalloc.h"
#include "reduce_kernels.cuh"

using namespace psb;

namespace {

// Scratch of the reduction: partial sums + ticket word (layout in reduce_kernels.cuh).
// In host code this name is only a handle for cudaGetSymbolAddress — it is NOT a device
// address and must never be passed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[kReduceScratchBytes];

// Device address of g_static_scratch on the current device.  Asked for on every call: after
// the first call on a device the runtime answers from its own tables (no device work), and
// an address remembered here would go stale if the application reset the device.
cudaError_t scratch_address(void** addr) { return cudaGetSymbolAddress(addr, g_static_scratch); }

}  // namespace

extern "C" int psb_reduce_sum_static(const float* x, size_t n, int op, double* out, cudaStream_t stream) {
  if (n > PSB_REDUCE_STATIC_MAX_ELEMS) {
    std::fprintf(stderr, "psb_reduce_sum_static: n = %zu exceeds the maximum of %llu elements\n", n,
                 (unsigned long long)PSB_REDUCE_STATIC_MAX_ELEMS);
    return (int)cudaErrorInvalidValue;
  }
  if (op < 0 || op > 4 || out == nullptr || (x == nullptr && n != 0)) {
    std::fprintf(stderr, "psb_reduce_sum_static: invalid argument (op = %d)\n", op);
    return (int)cudaErrorInvalidValue;
  }
  void* base = nullptr;
  cudaError_t e = scratch_address(&base);
  if (e != cudaSuccess) return (int)e;
  double* partial = reinterpret_cast<double*>(base);
  unsigned* ticket = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(base) + 8 * (size_t)kReduceMaxBlocks);
  // the array keeps whatever the previous call (or a failed one) left: the ticket must start at 0
  e = cudaMemsetAsync(ticket, 0, sizeof(unsigned), stream);
  if (e != cudaSuccess) return (int)e;
  reduce_sum_kernel<<<reduce_grid(n), kReduceThreads, 0, stream>>>(x, n, op, partial, ticket, out);
  return (int)cudaGetLastError();
}
