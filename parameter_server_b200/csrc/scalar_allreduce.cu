// All-reduce of a handful of scalars over the GPUs of the box without a collective library: the per-pass
// progress merge of the batch solvers (objective terms, non-zero count, active keys: sums; KKT violation: max —
// LinearMethod::mergeProgress, src/linear_method/linear_method.cc:106-120) and the per-step statistics.
//
// Every rank writes its values into its own copy of a symmetric buffer, raises a flag on every peer (release,
// system scope) and waits (bounded) for all peers' flags.  Then it reads the result:
//   * with a multicast mapping of the buffer (NVLink SHARP): ONE `multimem.ld_reduce` per value — the switch
//     reads all ranks' copies and returns their sum (or maximum) — fp64 sums, u32 maxima;
//   * without: one peer load per rank and value, added in rank order.
// Both give every rank the same fp64 result up to the order of the additions; the solvers only compare and
// print these values.  Two buffers alternate by call parity, so a rank may enter the next call while a slower
// one still reads the previous results.
#include "psb_common.cuh"

namespace psb {

constexpr int kMaxScalars = 32;

struct ScalarPeers {
  double* sums[PSB_MAX_RANKS];        // rank r: [2][kMaxScalars] values to be added
  uint32_t* maxs[PSB_MAX_RANKS];      // rank r: [2][kMaxScalars] non-negative floats as bit patterns (their order)
  uint64_t* flags[PSB_MAX_RANKS];     // rank r: [sender] = sequence number of the sender's last call
  const double* mc_sums;              // multicast address of `sums`, or nullptr
  const uint32_t* mc_maxs;            // multicast address of `maxs`, or nullptr
  int rank, world;
  uint64_t timeout_ns;
};

__global__ void k_scalar_allreduce(ScalarPeers P, const double* in_sum, int nsum, const float* in_max, int nmax, uint64_t seq,
                                   double* out_sum, float* out_max, uint32_t* status) {
  const int par = (int)(seq & 1);
  const int t = threadIdx.x;
  if (t < nsum) P.sums[P.rank][par * kMaxScalars + t] = in_sum[t];
  if (t < nmax) P.maxs[P.rank][par * kMaxScalars + t] = __float_as_uint(fmaxf(in_max[t], 0.f));
  __syncthreads();
  if (t < P.world) {
    __threadfence_system();
    st_release_sys_u64(P.flags[t] + P.rank, seq << 32);
    bool ok;
    wait_epoch_ge(P.flags[P.rank] + t, (uint32_t)seq, P.timeout_ns, &ok);
    if (!ok) set_status(status, kWaitTimeout, (uint32_t)t, 21);
  }
  __syncthreads();
  if (t < nsum) {
    double v = 0.0;
    if (P.mc_sums != nullptr) {
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.f64 %0, [%1];" : "=d"(v) : "l"(P.mc_sums + par * kMaxScalars + t) : "memory");
    } else {
      for (int r = 0; r < P.world; ++r) {
        unsigned long long b;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(b) : "l"(P.sums[r] + par * kMaxScalars + t) : "memory");
        v += __longlong_as_double((long long)b);
      }
    }
    out_sum[t] = v;
  }
  if (t < nmax) {
    uint32_t v = 0u;
    if (P.mc_maxs != nullptr) {
      asm volatile("multimem.ld_reduce.relaxed.sys.global.max.u32 %0, [%1];" : "=r"(v) : "l"(P.mc_maxs + par * kMaxScalars + t) : "memory");
    } else {
      for (int r = 0; r < P.world; ++r) v = max(v, ld_relaxed_sys_u32(P.maxs[r] + par * kMaxScalars + t));
    }
    out_max[t] = __uint_as_float(v);
  }
}

}  // namespace psb

using namespace psb;

extern "C" int psb_scalar_allreduce(const ScalarPeers* P, const double* in_sum, int nsum, const float* in_max, int nmax,
                                    uint64_t seq, double* out_sum, float* out_max, uint32_t* status, cudaStream_t s) {
  if (nsum < 0 || nmax < 0 || nsum > kMaxScalars || nmax > kMaxScalars || P->world > kMaxScalars) return (int)cudaErrorInvalidValue;
  k_scalar_allreduce<<<1, 64, 0, s>>>(*P, in_sum, nsum, in_max, nmax, seq, out_sum, out_max, status);
  return (int)cudaGetLastError();
}
