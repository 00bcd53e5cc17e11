// Sparse fully connected layer: Y = act(X·W) for a row-major sparse X (a minibatch of examples with a few
// features each) and a dense model W stored one row per input feature — an embedding-bag sum.  Role of
// SparseFullyConnectedLayer (src/neural_network/sparse_fully_connected_layer.h:31-88), which keeps one
// vector per feature key and adds the vectors of an example's features.
//
//   forward   Y[i,:]  = act( Σ_{j ∈ row i} x_ij · W[j,:] )        one warp per example, lanes over the outputs
//   backward  Wg[j,:] += x_ij · Z[i,:]   with Z = dY ∘ act'(Y)     vector reductions into the feature's row
// X carries no gradient (it is the data).
#include "psb_common.cuh"

namespace psb {

enum SpfcAct : int { kSpIdentity = 0, kSpRelu = 1, kSpScaledTanh = 2, kSpSigmoid = 3 };

__device__ __forceinline__ float spfc_act(float x, int act) {
  switch (act) {
    case kSpRelu: return fmaxf(x, 0.f);
    case kSpScaledTanh: return 1.7159f * tanhf(0.6666667f * x);
    case kSpSigmoid: return 1.f / (1.f + __expf(-x));
    default: return x;
  }
}
// derivative of the activation expressed through its output y
__device__ __forceinline__ float spfc_act_grad(float y, int act) {
  switch (act) {
    case kSpRelu: return y > 0.f ? 1.f : 0.f;
    case kSpScaledTanh: { const float t = y / 1.7159f; return 1.7159f * 0.6666667f * (1.f - t * t); }
    case kSpSigmoid: return y * (1.f - y);
    default: return 1.f;
  }
}

// out_dim is a multiple of 4: a lane owns float4 pieces of the output row
__global__ void k_spfc_forward(const int64_t* __restrict__ off, const int32_t* __restrict__ idx, const float* __restrict__ vals,
                               const float* __restrict__ W, float* __restrict__ Y, int rows, int in_dim, int out_dim, int act,
                               uint32_t* status) {
  const int lane = threadIdx.x & 31;
  const int64_t gwarp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int quads = out_dim >> 2;
  for (int64_t i = gwarp; i < rows; i += nwarps) {
    const int64_t b = off[i], e = off[i + 1];
    for (int q0 = 0; q0 < quads; q0 += 32) {
      const int q = q0 + lane;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int64_t p = b; p < e; ++p) {
        const int32_t j = idx[p];                      // same address for the whole warp: one broadcast load
        if (j < 0 || j >= in_dim) { if (lane == 0) set_status(status, kBadIndex, (uint32_t)j, 31); continue; }
        const float x = vals ? vals[p] : 1.f;
        if (q < quads) {
          const float4 w = __ldg(reinterpret_cast<const float4*>(W + (size_t)j * out_dim) + q);
          acc.x += x * w.x; acc.y += x * w.y; acc.z += x * w.z; acc.w += x * w.w;
        }
      }
      if (q < quads) {
        acc.x = spfc_act(acc.x, act); acc.y = spfc_act(acc.y, act); acc.z = spfc_act(acc.z, act); acc.w = spfc_act(acc.w, act);
        reinterpret_cast<float4*>(Y + (size_t)i * out_dim)[q] = acc;
      }
    }
  }
}

// Wg must be zero on entry
__global__ void k_spfc_backward(const int64_t* __restrict__ off, const int32_t* __restrict__ idx, const float* __restrict__ vals,
                                const float* __restrict__ Y, const float* __restrict__ dY, float* __restrict__ Wg, int rows,
                                int in_dim, int out_dim, int act) {
  const int lane = threadIdx.x & 31;
  const int64_t gwarp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int quads = out_dim >> 2;
  for (int64_t i = gwarp; i < rows; i += nwarps) {
    const int64_t b = off[i], e = off[i + 1];
    for (int q0 = 0; q0 < quads; q0 += 32) {
      const int q = q0 + lane;
      float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      if (q < quads) {
        const float4 y = reinterpret_cast<const float4*>(Y + (size_t)i * out_dim)[q];
        const float4 g = reinterpret_cast<const float4*>(dY + (size_t)i * out_dim)[q];
        z = make_float4(g.x * spfc_act_grad(y.x, act), g.y * spfc_act_grad(y.y, act), g.z * spfc_act_grad(y.z, act),
                        g.w * spfc_act_grad(y.w, act));
      }
      for (int64_t p = b; p < e; ++p) {
        const int32_t j = idx[p];
        if (j < 0 || j >= in_dim || q >= quads) continue;
        const float x = vals ? vals[p] : 1.f;
        float* dst = Wg + (size_t)j * out_dim + 4 * (size_t)q;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(x * z.x), "f"(x * z.y), "f"(x * z.z),
                     "f"(x * z.w) : "memory");
      }
    }
  }
}

}  // namespace psb

using namespace psb;

extern "C" {
int psb_spfc_forward(const int64_t* off, const int32_t* idx, const float* vals, const float* W, float* Y, int rows, int in_dim,
                     int out_dim, int act, uint32_t* status, cudaStream_t s) {
  if (out_dim <= 0 || (out_dim & 3) || rows < 0) return (int)cudaErrorInvalidValue;
  const int64_t blocks = ((int64_t)rows * 32 + 255) / 256;
  k_spfc_forward<<<(int)(blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks)), 256, 0, s>>>(off, idx, vals, W, Y, rows, in_dim,
                                                                                           out_dim, act, status);
  return (int)cudaGetLastError();
}
int psb_spfc_backward(const int64_t* off, const int32_t* idx, const float* vals, const float* Y, const float* dY, float* Wg, int rows,
                      int in_dim, int out_dim, int act, cudaStream_t s) {
  if (out_dim <= 0 || (out_dim & 3) || rows < 0) return (int)cudaErrorInvalidValue;
  const int64_t blocks = ((int64_t)rows * 32 + 255) / 256;
  k_spfc_backward<<<(int)(blocks < 1 ? 1 : (blocks > 148 * 8 ? 148 * 8 : blocks)), 256, 0, s>>>(off, idx, vals, Y, dY, Wg, rows, in_dim,
                                                                                            out_dim, act);
  return (int)cudaGetLastError();
}
}
