// Key-range sharded key→value vector on peer memory: the device form of KVVector
// (src/parameter/kv_vector.h) and of the push / pull message pair of SharedParameter
// (src/parameter/shared_parameter.h:14-26, 90-149).
//
// Every rank (server) holds the sorted keys of its key range and k fp32 values per key in
// peer-addressable buffers.  A worker resolves its keys once — owner by key range, slot by binary
// search in the owner's key array, read over NVLink — which is the steady state of the
// reference's key cache (src/system/remote_node.cc:96-184): afterwards pushes and pulls carry
// values only.
//   pull  out[i, :]            = vals[owner_i][slot_i, :]      plain peer loads (16-byte vectors when k % 4 == 0)
//   push  vals[owner_i][slot_i, :] += in[i, :]                 red.add (v4 / v2 / scalar) on peer memory:
//                                                              the sum over workers happens at the owner
// Unknown keys resolve to slot -1: pulls return zeros for them and pushes skip them.
#include "psb_common.cuh"

namespace psb {

struct KvPeers {
  const uint64_t* keys[PSB_MAX_RANKS];   // sorted unique keys of every shard
  float* vals[PSB_MAX_RANKS];            // [nkeys, k]
  int64_t nkeys[PSB_MAX_RANKS];
  KeySeps seps;
  int k;
  int pad;
};

__global__ void k_kv_resolve(KvPeers P, const uint64_t* __restrict__ q, size_t n, int32_t* __restrict__ owner, int32_t* __restrict__ slot) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t key = q[i];
    const int o = route_owner(P.seps, key);
    const uint64_t* k = P.keys[o];
    int64_t lo = 0, hi = P.nkeys[o];
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (ld_relaxed_sys_u64(k + mid) < key) lo = mid + 1; else hi = mid;
    }
    owner[i] = o;
    slot[i] = (lo < P.nkeys[o] && ld_relaxed_sys_u64(k + lo) == key) ? (int32_t)lo : -1;
  }
}

// one thread per (row, 4-float chunk) when k % 4 == 0, otherwise one thread per element
__global__ void k_kv_pull(KvPeers P, const int32_t* __restrict__ owner, const int32_t* __restrict__ slot, size_t n, float* __restrict__ out) {
  const int k = P.k;
  if ((k & 3) == 0) {
    const int chunks = k >> 2;
    const size_t total = n * (size_t)chunks;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
      const size_t i = t / chunks;
      const int c = (int)(t % chunks);
      const int32_t s = slot[i];
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s >= 0) {
        const float4* src = reinterpret_cast<const float4*>(P.vals[owner[i]] + (size_t)s * k) + c;
        asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(src) : "memory");
      }
      reinterpret_cast<float4*>(out + i * (size_t)k)[c] = v;
    }
  } else {
    const size_t total = n * (size_t)k;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
      const size_t i = t / k;
      const int c = (int)(t % k);
      const int32_t s = slot[i];
      out[t] = s >= 0 ? ld_relaxed_sys_f32(P.vals[owner[i]] + (size_t)s * k + c) : 0.f;
    }
  }
}

__global__ void k_kv_push(KvPeers P, const int32_t* __restrict__ owner, const int32_t* __restrict__ slot, size_t n, const float* __restrict__ in) {
  const int k = P.k;
  if ((k & 3) == 0) {
    const int chunks = k >> 2;
    const size_t total = n * (size_t)chunks;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
      const size_t i = t / chunks;
      const int c = (int)(t % chunks);
      const int32_t s = slot[i];
      if (s < 0) continue;
      const float4 v = reinterpret_cast<const float4*>(in + i * (size_t)k)[c];
      float* dst = P.vals[owner[i]] + (size_t)s * k + 4 * c;
      asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
    }
  } else {
    const size_t total = n * (size_t)k;
    for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
      const size_t i = t / k;
      const int32_t s = slot[i];
      if (s >= 0) red_add_sys_f32(P.vals[owner[i]] + (size_t)s * k + (t % k), in[t]);
    }
  }
  __threadfence_system();
}

// baseline helpers: gather / scatter-add on local memory only (used with all_to_all exchanges)
__global__ void k_rows_gather(const float* __restrict__ vals, const int32_t* __restrict__ slot, size_t n, int k, float* __restrict__ out) {
  const size_t total = n * (size_t)k;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int32_t s = slot[t / k];
    out[t] = s >= 0 ? vals[(size_t)s * k + (t % k)] : 0.f;
  }
}
__global__ void k_rows_scatter_add(float* __restrict__ vals, const int32_t* __restrict__ slot, size_t n, int k, const float* __restrict__ in) {
  const size_t total = n * (size_t)k;
  for (size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (size_t)gridDim.x * blockDim.x) {
    const int32_t s = slot[t / k];
    if (s >= 0) atomicAdd(&vals[(size_t)s * k + (t % k)], in[t]);
  }
}

}  // namespace psb

using namespace psb;

namespace {
inline int kgrid(size_t n) { size_t b = (n + 255) / 256; if (b < 1) b = 1; if (b > 148 * 16) b = 148 * 16; return (int)b; }
}

extern "C" {

int psb_kv_resolve(const KvPeers* P, const uint64_t* q, size_t n, int32_t* owner, int32_t* slot, cudaStream_t s) {
  k_kv_resolve<<<kgrid(n), 256, 0, s>>>(*P, q, n, owner, slot);
  return (int)cudaGetLastError();
}
int psb_kv_pull(const KvPeers* P, const int32_t* owner, const int32_t* slot, size_t n, float* out, cudaStream_t s) {
  k_kv_pull<<<kgrid(n * (size_t)((P->k & 3) ? P->k : P->k / 4)), 256, 0, s>>>(*P, owner, slot, n, out);
  return (int)cudaGetLastError();
}
int psb_kv_push(const KvPeers* P, const int32_t* owner, const int32_t* slot, size_t n, const float* in, cudaStream_t s) {
  k_kv_push<<<kgrid(n * (size_t)((P->k & 3) ? P->k : P->k / 4)), 256, 0, s>>>(*P, owner, slot, n, in);
  return (int)cudaGetLastError();
}
int psb_rows_gather(const float* vals, const int32_t* slot, size_t n, int k, float* out, cudaStream_t s) {
  k_rows_gather<<<kgrid(n * (size_t)k), 256, 0, s>>>(vals, slot, n, k, out);
  return (int)cudaGetLastError();
}
int psb_rows_scatter_add(float* vals, const int32_t* slot, size_t n, int k, const float* in, cudaStream_t s) {
  k_rows_scatter_add<<<kgrid(n * (size_t)k), 256, 0, s>>>(vals, slot, n, k, in);
  return (int)cudaGetLastError();
}

}  // extern "C"
