// Dense layer GEMM on the 5th-generation tensor cores: D[M,N] = act(A[M,K] · B[N,K]ᵀ), fp32 in
// memory, TF32 multiply, fp32 accumulate in tensor memory (TMEM).
//
// One CTA (128 threads) per 128x128 output tile:
//   warp 0, one lane   TMA producer: cp.async.bulk.tensor 2-D tiles of A and B (128 rows x 32 floats =
//                      one 128-byte swizzle row each) into a 4-stage shared-memory ring, completion on
//                      the stage's "full" mbarrier
//   warp 1, one lane   MMA issuer: tcgen05.mma.cta_group::1.kind::tf32, four K=8 steps per stage, the
//                      accumulator lives in 128 TMEM columns; tcgen05.commit releases the stage
//                      ("empty" mbarrier) and finally signals "accumulator complete"
//   all 4 warps        epilogue: tcgen05.ld 32 lanes x 32 columns per warp and step, activation, store
// Both operands are K-major (row-major with K contiguous), which is how the layers keep their data:
// activations [batch, features] and weights [out, in]; the transposed products of the backward
// pass go through the tiled transpose kernel first.  No multicast is used anywhere.
//
// This is the framework's replacement of the Eigen GEMMs of the reference's fully connected
// layer (src/neural_network/fully_connected_layer.h:27-65); the activation functions are those
// of src/neural_network/activation_function.h:39-99.
//
// Every mbarrier wait is bounded.  If one runs out, the CTA records it in the status word, stops
// issuing work, waits a bounded time for copies in flight, frees its TMEM and returns.
#include <cuda.h>

#include "psb_common.cuh"

namespace psb {

constexpr int kBM = 128, kBN = 128, kBK = 32;       // tile; kBK floats = 128 bytes = swizzle span
constexpr int kStages = 4;
constexpr int kUmmaK = 8;                            // K per tcgen05.mma for tf32
constexpr uint32_t kStageBytesA = kBM * kBK * 4, kStageBytesB = kBN * kBK * 4;
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kWaitLimit = 4u * 1000u * 1000u;   // polls of try_wait before giving up

enum Activation : int { kActIdentity = 0, kActRelu = 1, kActScaledTanh = 2, kActSigmoid = 3 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bounded wait for the phase with the given parity; false when the limit is hit
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t addr = smem_u32(bar);
  for (uint32_t i = 0; i < kWaitLimit; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(addr), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, groups of 8 rows
// (1024 bytes) are the swizzle atoms.  start address >> 4 in bits 0-13, stride byte offset
// (1024 >> 4) in bits 32-45, descriptor version 1 in bits 46-47, layout type 2 (128B swizzle)
// in bits 61-63; the leading byte offset is not used for swizzled K-major tiles.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// instruction descriptor for kind::tf32: D fp32 (1 at bits 4-5), A and B tf32 (2 at bits 7-9 and
// 10-12), both K-major (bits 15, 16 = 0), N >> 3 at bits 17-22, M >> 4 at bits 24-28
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case kActRelu: return fmaxf(x, 0.f);
    case kActScaledTanh: return 1.7159f * tanhf(0.6666667f * x);
    case kActSigmoid: return 1.f / (1.f + __expf(-x));
    default: return x;
  }
}

struct __align__(1024) GemmSmem {
  float a[kStages][kBM * kBK];
  float b[kStages][kBN * kBK];
  uint64_t full[kStages], empty[kStages], acc_full;
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

__global__ void __launch_bounds__(128, 1)
gemm_tf32_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                         float* __restrict__ out, int M, int N, int K, int ldo, int act, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmem& s = *reinterpret_cast<GemmSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * kBM, n0 = blockIdx.y * kBN;
  const int nkb = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
    mbar_init(&s.acc_full, 1);
    s.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {   // one warp allocates the accumulator columns
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s.tmem_base;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer
    for (int kb = 0; kb < nkb; ++kb) {
      const int st = kb % kStages;
      if (kb >= kStages && !mbar_wait(&s.empty[st], ((kb / kStages) - 1) & 1)) { s.abort_flag = 1; break; }
      if (s.abort_flag) break;
      mbar_expect_tx(&s.full[st], kStageBytesA + kStageBytesB);
      tma_load_2d(s.a[st], &map_a, &s.full[st], kb * kBK, m0);
      tma_load_2d(s.b[st], &map_b, &s.full[st], kb * kBK, n0);
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    constexpr uint32_t idesc = make_idesc(kBM, kBN);
    for (int kb = 0; kb < nkb; ++kb) {
      const int st = kb % kStages;
      if (!mbar_wait(&s.full[st], (kb / kStages) & 1)) { s.abort_flag = 1; break; }
      if (s.abort_flag) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t da = make_smem_desc(smem_u32(s.a[st]));
      const uint64_t db = make_smem_desc(smem_u32(s.b[st]));
#pragma unroll
      for (int k = 0; k < kBK / kUmmaK; ++k) {
        const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
        const uint64_t adv = (uint64_t)((k * kUmmaK * 4) >> 4);   // 32 bytes per K step inside the swizzle row
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem), "l"(da + adv), "l"(db + adv), "r"(idesc), "r"(accumulate) : "memory");
      }
      // release the stage once the MMAs that read it have completed
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s.empty[st])) : "memory");
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s.acc_full)) : "memory");
  }
  __syncwarp();

  // ---------------- epilogue (all four warps; warp w owns TMEM lanes 32w .. 32w+31)
  int ok = 1;
  if (lane == 0) {
    ok = mbar_wait(&s.acc_full, 0) ? 1 : 0;
    if (!ok) s.abort_flag = 1;
    if (s.abort_flag) ok = 0;
  }
  ok = __shfl_sync(0xffffffffu, ok, 0);   // warp-uniform: the TMEM loads below are warp-collective
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (ok) {
    const int row = m0 + warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < kBN; c0 += 32) {
      uint32_t r[32];
      const uint32_t taddr = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
      asm volatile(
          "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
          "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
          "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
          : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
            "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
            "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
            "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
          : "r"(taddr) : "memory");
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      if (row < M) {
        float* dst = out + (size_t)row * ldo + n0 + c0;
        const int ncol = N - (n0 + c0);
        if (ncol >= 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float4 v;
            v.x = apply_act(__uint_as_float(r[j]), act);
            v.y = apply_act(__uint_as_float(r[j + 1]), act);
            v.z = apply_act(__uint_as_float(r[j + 2]), act);
            v.w = apply_act(__uint_as_float(r[j + 3]), act);
            *reinterpret_cast<float4*>(dst + j) = v;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (j < ncol) dst[j] = apply_act(__uint_as_float(r[j]), act);
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s.abort_flag) {
    if (threadIdx.x == 0) set_status(status, kWaitTimeout, blockIdx.x, 100 + blockIdx.y);
    // give copies that may still be in flight a bounded time to land before the shared memory goes away
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ------------------------------------------------------------------ persistent variant for large problems
// One CTA per SM walks a list of 128x256 output tiles.  Six warps: warp 0 (one lane) TMA producer,
// warp 1 (one lane) MMA issuer, warps 2-5 epilogue (warp w reads TMEM lanes 32·(w mod 4) ...).  The
// accumulator is double-buffered in TMEM (2 x 256 columns): while the epilogue warps drain tile i, the
// tensor core already works on tile i+1.  The shared-memory ring runs across tile boundaries.
constexpr int kPBN = 256;
constexpr int kPStages = 4;
constexpr uint32_t kPStageBytesB = kPBN * kBK * 4;
constexpr int kPThreads = 192;

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct __align__(1024) GemmSmemP {
  float a[kPStages][kBM * kBK];
  float b[kPStages][kPBN * kBK];
  uint64_t full[kPStages], empty[kPStages], tfull[2], tempty[2];
  uint32_t tmem_base;
  volatile uint32_t abort_flag;
};

__global__ void __launch_bounds__(kPThreads, 1)
gemm_tf32_persistent_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                            float* __restrict__ out, int M, int N, int K, int ldo, int act, uint32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  GemmSmemP& s = *reinterpret_cast<GemmSmemP*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nbm = (M + kBM - 1) / kBM, nbn = (N + kPBN - 1) / kPBN;
  const int ntiles = nbm * nbn;
  const int nkb = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int i = 0; i < kPStages; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&s.tfull[i], 1); mbar_init(&s.tempty[i], 4); }
    s.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s.tmem_base)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s.tmem_base;

  if (warp == 0 && lane == 0) {
    // ---------------- TMA producer: tiles are walked m-fastest so that concurrent CTAs share a B panel
    uint32_t g = 0;
    for (int t = blockIdx.x; t < ntiles && !s.abort_flag; t += gridDim.x) {
      const int m0 = (t % nbm) * kBM, n0 = (t / nbm) * kPBN;
      for (int kb = 0; kb < nkb; ++kb, ++g) {
        const int st = g % kPStages;
        if (g >= (uint32_t)kPStages && !mbar_wait(&s.empty[st], ((g / kPStages) - 1) & 1)) { s.abort_flag = 1; break; }
        if (s.abort_flag) break;
        mbar_expect_tx(&s.full[st], kStageBytesA + kPStageBytesB);
        tma_load_2d(s.a[st], &map_a, &s.full[st], kb * kBK, m0);
        tma_load_2d(s.b[st], &map_b, &s.full[st], kb * kBK, n0);
      }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer
    constexpr uint32_t idesc = make_idesc(kBM, kPBN);
    uint32_t g = 0, it = 0;
    for (int t = blockIdx.x; t < ntiles && !s.abort_flag; t += gridDim.x, ++it) {
      const uint32_t acc = it & 1u;
      if (it >= 2 && !mbar_wait(&s.tempty[acc], ((it >> 1) - 1) & 1)) { s.abort_flag = 1; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t d_tmem = tmem + acc * (uint32_t)kPBN;
      for (int kb = 0; kb < nkb; ++kb, ++g) {
        const int st = g % kPStages;
        if (!mbar_wait(&s.full[st], (g / kPStages) & 1)) { s.abort_flag = 1; break; }
        if (s.abort_flag) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t da = make_smem_desc(smem_u32(s.a[st]));
        const uint64_t db = make_smem_desc(smem_u32(s.b[st]));
#pragma unroll
        for (int k = 0; k < kBK / kUmmaK; ++k) {
          const uint32_t accumulate = (kb > 0 || k > 0) ? 1u : 0u;
          const uint64_t adv = (uint64_t)((k * kUmmaK * 4) >> 4);
          asm volatile(
              "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
              "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
              ::"r"(d_tmem), "l"(da + adv), "l"(db + adv), "r"(idesc), "r"(accumulate) : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s.empty[st])) : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&s.tfull[acc])) : "memory");
    }
  } else if (warp >= 2) {
    // ---------------- epilogue warps
    const int q = warp & 3;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
      const uint32_t acc = it & 1u;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(&s.tfull[acc], (it >> 1) & 1) ? 1 : 0;
        if (!ok) s.abort_flag = 1;
        if (s.abort_flag) ok = 0;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int m0 = (t % nbm) * kBM, n0 = (t / nbm) * kPBN;
      const int row = m0 + q * 32 + lane;
#pragma unroll 1
      for (int c0 = 0; c0 < kPBN; c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16) + acc * (uint32_t)kPBN + (uint32_t)c0;
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
            "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
              "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
              "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
            : "r"(taddr) : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (c0 + 32 >= kPBN) {
          // last chunk is in registers: hand the accumulator back to the MMA warp before the stores
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(&s.tempty[acc]);
        }
        if (row < M && n0 + c0 < N) {
          float* dst = out + (size_t)row * ldo + n0 + c0;
          const int ncol = N - (n0 + c0);
          if (ncol >= 32 && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              float4 v;
              v.x = apply_act(__uint_as_float(r[j]), act);
              v.y = apply_act(__uint_as_float(r[j + 1]), act);
              v.z = apply_act(__uint_as_float(r[j + 2]), act);
              v.w = apply_act(__uint_as_float(r[j + 3]), act);
              *reinterpret_cast<float4*>(dst + j) = v;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ncol) dst[j] = apply_act(__uint_as_float(r[j]), act);
          }
        }
      }
    }
  }
  __syncwarp();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (s.abort_flag) {
    if (threadIdx.x == 0) set_status(status, kWaitTimeout, blockIdx.x, 200);
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

// ------------------------------------------------------------------ elementwise / layout kernels of the NN app
// tiled transpose out[c][r] = in[r][c]   (src/base/dense_matrix.h:87-104)
__global__ void k_transpose(const float* __restrict__ in, float* __restrict__ out, int rows, int cols) {
  __shared__ float tile[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y)
    if (r0 + j < rows && c < cols) tile[j][threadIdx.x] = in[(size_t)(r0 + j) * cols + c];
  __syncthreads();
  const int r = blockIdx.y * 32 + threadIdx.x, c0 = blockIdx.x * 32;
  for (int j = threadIdx.y; j < 32; j += blockDim.y)
    if (c0 + j < cols && r < rows) out[(size_t)(c0 + j) * rows + r] = tile[threadIdx.x][j];
}
// z = g ∘ act'(y) with act' expressed through the activation output y
__global__ void k_act_backward(const float* __restrict__ g, const float* __restrict__ y, float* __restrict__ z, size_t n, int act) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float yv = y[i];
    float d = 1.f;
    if (act == kActRelu) d = yv > 0.f ? 1.f : 0.f;
    else if (act == kActScaledTanh) { const float t = yv / 1.7159f; d = 1.7159f * 0.6666667f * (1.f - t * t); }
    else if (act == kActSigmoid) d = yv * (1.f - yv);
    z[i] = g[i] * d;
  }
}
// logistic loss layer: loss += Σ log(1+e^{-x y}); grad = -y/(1+e^{x y})   (src/neural_network/loss_layer.h:39-58)
__global__ void k_logistic_loss(const float* __restrict__ x, const float* __restrict__ y, float* __restrict__ grad, size_t n, double* loss) {
  double acc = 0.0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float m = x[i] * y[i];
    acc += (double)log1pexp(-m);
    if (grad) grad[i] = -y[i] / (1.f + __expf(m));
  }
  acc = warp_sum_d(acc);
  if ((threadIdx.x & 31) == 0 && acc != 0.0) atomicAdd(loss, acc);
}
// SGD: w -= α g / (β + sqrt(t));  AdaGrad: h += g², w -= α g / (β + sqrt(h))   (src/neural_network/sgd_solver.h:11-36)
__global__ void k_sgd_update(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ h, size_t n, float alpha, float beta,
                             float iter, int adagrad) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float gv = g[i];
    float denom;
    if (adagrad) { const float hv = h[i] + gv * gv; h[i] = hv; denom = beta + sqrtf(hv); }
    else denom = beta + sqrtf(iter);
    w[i] -= alpha * gv / denom;
  }
}
// per-column mean-centre and scale to norm sqrt(rows)   (src/neural_network/data_layer.h:25-31)
__global__ void k_col_normalize(float* __restrict__ x, int rows, int cols) {
  const int c = blockIdx.x;
  __shared__ double sh[64];
  double s = 0.0;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) s += x[(size_t)r * cols + c];
  s = warp_sum_d(s);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) { double t = 0; for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += sh[i]; sh[32] = t / rows; }
  __syncthreads();
  const float mean = (float)sh[32];
  double q = 0.0;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) { const float d = x[(size_t)r * cols + c] - mean; q += (double)d * d; }
  q = warp_sum_d(q);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = q;
  __syncthreads();
  if (threadIdx.x == 0) { double t = 0; for (int i = 0; i < (int)(blockDim.x >> 5); ++i) t += sh[i]; sh[33] = t; }
  __syncthreads();
  const float nrm = (float)sqrt(sh[33]);
  const float scale = nrm > 0.f ? sqrtf((float)rows) / nrm : 0.f;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) x[(size_t)r * cols + c] = (x[(size_t)r * cols + c] - mean) * scale;
}

}  // namespace psb

using namespace psb;

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}
// 2-D map over a row-major [rows, k] fp32 matrix with row stride ld (floats), box = 128 rows x 32 floats, 128B swizzle
int make_map(CUtensorMap* map, const float* base, int rows, int k, int ld, int box_rows = kBM) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
inline int egrid(size_t n) { size_t b = (n + 255) / 256; if (b < 1) b = 1; if (b > 148 * 8) b = 148 * 8; return (int)b; }

}  // namespace

extern "C" {

// out[M,N] (row stride ldo) = act(a[M,K] (row stride lda) · b[N,K]ᵀ (row stride ldb)).
// Requirements: a, b 16-byte aligned; lda, ldb multiples of 4 floats.  Returns 0, a CUDA error, or
// -1 when tensor maps cannot be created (no driver entry point).
int psb_gemm_tn_tf32(const float* a, const float* b, float* out, int M, int N, int K, int lda, int ldb, int ldo, int act,
                     uint32_t* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 3) || (ldb & 3) || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return (int)cudaErrorInvalidValue;
  CUtensorMap ma, mb;
  int r = make_map(&ma, a, M, K, lda);
  if (r) return r;
  // large problems: persistent kernel with 128x256 tiles and a double-buffered accumulator
  static int sms = 0;
  if (sms == 0) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev); }
  const long tiles_p = (long)((M + kBM - 1) / kBM) * ((N + kPBN - 1) / kPBN);
  if (tiles_p >= sms) {
    r = make_map(&mb, b, N, K, ldb, kPBN);
    if (r) return r;
    const size_t smem_p = sizeof(GemmSmemP) + 1024;
    static bool attr_p = false;
    if (!attr_p) {
      cudaError_t e = cudaFuncSetAttribute(gemm_tf32_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_p);
      if (e != cudaSuccess) return (int)e;
      attr_p = true;
    }
    const int grid = (int)(tiles_p < sms ? tiles_p : sms);
    gemm_tf32_persistent_kernel<<<grid, kPThreads, smem_p, stream>>>(ma, mb, out, M, N, K, ldo, act, status);
    return (int)cudaGetLastError();
  }
  r = make_map(&mb, b, N, K, ldb);
  if (r) return r;
  const size_t smem = sizeof(GemmSmem) + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tf32_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  dim3 grid((M + kBM - 1) / kBM, (N + kBN - 1) / kBN);
  gemm_tf32_tcgen05_kernel<<<grid, 128, smem, stream>>>(ma, mb, out, M, N, K, ldo, act, status);
  return (int)cudaGetLastError();
}
int psb_transpose(const float* in, float* out, int rows, int cols, cudaStream_t s) {
  dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
  k_transpose<<<grid, block, 0, s>>>(in, out, rows, cols);
  return (int)cudaGetLastError();
}
int psb_act_backward(const float* g, const float* y, float* z, size_t n, int act, cudaStream_t s) {
  k_act_backward<<<egrid(n), 256, 0, s>>>(g, y, z, n, act);
  return (int)cudaGetLastError();
}
int psb_logistic_loss(const float* x, const float* y, float* grad, size_t n, double* loss, cudaStream_t s) {
  k_logistic_loss<<<egrid(n), 256, 0, s>>>(x, y, grad, n, loss);
  return (int)cudaGetLastError();
}
int psb_sgd_update(float* w, const float* g, float* h, size_t n, float alpha, float beta, float iter, int adagrad, cudaStream_t s) {
  k_sgd_update<<<egrid(n), 256, 0, s>>>(w, g, h, n, alpha, beta, iter, adagrad);
  return (int)cudaGetLastError();
}
int psb_col_normalize(float* x, int rows, int cols, cudaStream_t s) {
  k_col_normalize<<<cols, 256, 0, s>>>(x, rows, cols);
  return (int)cudaGetLastError();
}

}  // extern "C"
