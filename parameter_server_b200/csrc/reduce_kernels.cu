// C entry point of the deterministic sum reductions used for objective values:
// DARLIN's Σ log(1+1/dual) (src/linear_method/darling.cc:506), the λ₁‖w‖₁ penalty
// and nnz(w) over weights with NaN-encoded filtered keys
// (src/linear_method/darling.cc:542-552), and the logistic loss
// (src/linear_method/loss.h:73-79).
#include "reduce_kernels.cuh"

using namespace psb;

extern "C" {

// scratch: device memory of at least psb_reduce_scratch_bytes() bytes whose ticket word
// (see reduce_kernels.cuh) is zero; the kernel leaves it zero.  out: one device double.
size_t psb_reduce_scratch_bytes() { return kReduceScratchBytes; }

int psb_reduce_sum(const float* x, size_t n, int op, void* scratch, size_t scratch_bytes, double* out,
                   cudaStream_t stream) {
  if (scratch_bytes < kReduceScratchBytes || op < 0 || op > 4) return (int)cudaErrorInvalidValue;
  double* partial = reinterpret_cast<double*>(scratch);
  unsigned* ticket = reinterpret_cast<unsigned*>(reinterpret_cast<char*>(scratch) + 8 * (size_t)kReduceMaxBlocks);
  reduce_sum_kernel<<<reduce_grid(n), kReduceThreads, 0, stream>>>(x, n, op, partial, ticket, out);
  return (int)cudaGetLastError();
}

}  // extern "C"
