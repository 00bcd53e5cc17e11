// Plain batch solver (no darling{} section): block gradient / diagonal curvature, the learners' block update
// and the margin update as stand-alone kernels over a column-major rows shard, for the loss family of the
// reference (src/linear_method/loss.h:66-104: LogitLoss, SquareHingeLoss), the penalties
// (src/linear_method/penalty.h:15-50) and the learners (src/linear_method/learner/proximal_gradient.h:20-53,
// gradient_descent.h:19-24).  Every rank keeps the whole weight vector; the block's (G,U) sums of the ranks
// are added between the first and the second kernel by the caller.
//
// A row's state is the pair {y_i, m_i = y_i·(Xw)_i}; both losses are functions of the margin m.
#include "psb_common.cuh"

namespace psb {

enum BatchLoss : int { kLossLogit = 0, kLossSquareHinge = 1 };
enum BatchLearner : int { kProxGradient = 0, kGradientDescent = 1 };

struct BatchShard {
  const int64_t* col_ptr;   // cols+1 offsets (column-major)
  const uint32_t* row_idx;  // nnz
  const float* vals;        // nnz or nullptr (binary features)
  const uint32_t* col_of;   // nnz: column of every non-zero
  float2* ym;               // rows: {y, margin}
};

// d loss / d (Xw)_i (already multiplied by y where the chain rule asks for it) and the curvature d²/d(Xw)²
__device__ __forceinline__ void loss_coefs(int kind, float y, float m, float* g, float* h) {
  if (kind == kLossLogit) {
    const float tau = 1.f / (1.f + __expf(m));
    *g = -y * tau;
    *h = tau * (1.f - tau);
  } else {
    // max(0, 1 − m)²: gradient −2·y·(1 − m) where m < 1 (the reference's formula has the indicator inverted
    // and lacks the (1 − m) factor, src/linear_method/loss.h:102), curvature 2 there
    const bool act = m < 1.f;
    *g = act ? -2.f * y * (1.f - m) : 0.f;
    *h = act ? 2.f : 0.f;
  }
}

// (G_j, U_j) += Σ_i {g_i·x_ij, h_i·x_ij²} over the non-zeros of columns [c0, c1); gu is indexed by j − c0
__global__ void k_batch_block_grad(BatchShard D, int kind, int64_t c0, int64_t c1, float2* gu) {
  const int64_t p0 = D.col_ptr[c0], p1 = D.col_ptr[c1];
  const int lane = threadIdx.x & 31;
  const int64_t gwarp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t base = p0 + gwarp * 32; base < p1; base += nwarps * 32) {
    const int64_t e = base + lane;
    const bool valid = e < p1;
    int64_t j = -1;
    float g = 0.f, u = 0.f;
    if (valid) {
      j = (int64_t)D.col_of[e];
      const float2 ym = D.ym[D.row_idx[e]];
      const float v = D.vals ? D.vals[e] : 1.f;
      float gi, hi;
      loss_coefs(kind, ym.x, ym.y, &gi, &hi);
      g = gi * v;
      u = hi * v * v;
    }
    // segmented sum over runs of equal j (the non-zeros of a column are contiguous)
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int64_t oj = __shfl_down_sync(0xffffffffu, j, off);
      const float og = __shfl_down_sync(0xffffffffu, g, off);
      const float ou = __shfl_down_sync(0xffffffffu, u, off);
      if (lane + off < 32 && oj == j) { g += og; u += ou; }
    }
    const int64_t pj = __shfl_up_sync(0xffffffffu, j, 1);
    if (valid && (lane == 0 || pj != j))
      asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(gu + (j - c0)), "f"(g), "f"(u) : "memory");
  }
}

// Block update of the learners: w ← w + d, d kept for the margin update.
//   proximal gradient, L1:  the soft-thresholded Newton step of src/linear_method/learner/proximal_gradient.h
//   proximal gradient, L2:  d = −(G + 2λw) / (U/η + 2λ)
//   gradient descent:       d = −η·(G + ∂penalty)
// Steps are clipped to [−5, 5].
__global__ void k_batch_block_update(const float2* gu, float* w, float* d_out, int64_t n, int learner, int pnorm, float eta,
                                     float lam) {
  for (int64_t k = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; k < n; k += (int64_t)gridDim.x * blockDim.x) {
    const float G = gu[k].x, U = gu[k].y, wk = w[k];
    float d;
    if (learner == kGradientDescent) {
      d = -eta * (G + (pnorm == 2 ? 2.f * lam * wk : 0.f));
    } else if (pnorm == 1) {
      const float u = U / eta + 1e-10f, gp = G + lam, gn = G - lam;
      d = gp <= u * wk ? -gp / u : (gn >= u * wk ? -gn / u : -wk);
      d = fminf(5.f, fmaxf(-5.f, d));
    } else {
      const float u = U / eta + 2.f * lam + 1e-10f;
      d = fminf(5.f, fmaxf(-5.f, -(G + 2.f * lam * wk) / u));
    }
    w[k] = wk + d;
    d_out[k] = d;
  }
}

// m_i += y_i·x_ij·d_j over the non-zeros of columns [c0, c1); d is indexed by j − c0
__global__ void k_batch_block_margin(BatchShard D, int64_t c0, int64_t c1, const float* d) {
  const int64_t p0 = D.col_ptr[c0], p1 = D.col_ptr[c1];
  for (int64_t e = p0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < p1; e += (int64_t)gridDim.x * blockDim.x) {
    const float dj = d[(int64_t)D.col_of[e] - c0];
    if (dj != 0.f) {
      const uint32_t i = D.row_idx[e];
      atomicAdd(&D.ym[i].y, D.ym[i].x * (D.vals ? D.vals[e] : 1.f) * dj);
    }
  }
}

}  // namespace psb

using namespace psb;

static inline int bgrid(int64_t n) {
  int64_t b = (n + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return (int)b;
}

extern "C" {
int psb_batch_block_grad(const BatchShard* D, int kind, int64_t c0, int64_t c1, void* gu, int64_t nnz_hint, cudaStream_t s) {
  k_batch_block_grad<<<bgrid(nnz_hint), 256, 0, s>>>(*D, kind, c0, c1, (float2*)gu);
  return (int)cudaGetLastError();
}
int psb_batch_block_update(const void* gu, float* w, float* d_out, int64_t n, int learner, int pnorm, float eta, float lam,
                           cudaStream_t s) {
  k_batch_block_update<<<bgrid(n), 256, 0, s>>>((const float2*)gu, w, d_out, n, learner, pnorm, eta, lam);
  return (int)cudaGetLastError();
}
int psb_batch_block_margin(const BatchShard* D, int64_t c0, int64_t c1, const float* d, int64_t nnz_hint, cudaStream_t s) {
  k_batch_block_margin<<<bgrid(nnz_hint), 256, 0, s>>>(*D, c0, c1, d);
  return (int)cudaGetLastError();
}
}
