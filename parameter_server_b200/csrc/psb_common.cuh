// Shared device-side primitives for the sm_100a kernels of this library:
// system-scope loads/stores used on peer (NVLink) memory, bounded flag waits,
// the 64-bit mixer used by every hash table, warp helpers and the status word.
//
// Conventions
//  * A "rank" is one GPU that hosts worker r and server (key-range shard) r.
//  * Cross-GPU waits never spin forever: they give up after `timeout_ns`
//    (and an iteration cap), record {code, peer, phase} in the status word and
//    let the kernel run to its end so that the context stays usable.
//  * kEmptyKey (2^64-1) is never a valid key; the reference's key space
//    Range::all() = [0, 2^64-1) excludes it as well (src/base/range.h:75-78).
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <cooperative_groups.h>

namespace cg = cooperative_groups;

#define PSB_MAX_RANKS 8
#define PSB_WARP 32

namespace psb {

constexpr uint64_t kEmptyKey = 0xFFFFFFFFFFFFFFFFull;

// status word layout (uint32_t[8], owned by the caller, zeroed by the caller)
enum StatusCode : uint32_t {
  kOk = 0,
  kWaitTimeout = 1,      // a bounded cross-GPU wait ran out
  kLocalTableFull = 2,   // per-minibatch dedup table overflow
  kShardTableFull = 3,   // owner hash table probe limit reached
  kInboxOverflow = 4,    // more records for one owner than the inbox holds
  kBadIndex = 5,         // an index failed its bounds check and was skipped
};

__device__ __forceinline__ void set_status(uint32_t* status, uint32_t code, uint32_t a, uint32_t b) {
  if (atomicCAS(&status[0], 0u, code) == 0u) {
    status[1] = a;
    status[2] = b;
  }
}

__device__ __forceinline__ uint64_t mix64(uint64_t x) {
  x ^= x >> 30; x *= 0xbf58476d1ce4e5b9ull;
  x ^= x >> 27; x *= 0x94d049bb133111ebull;
  x ^= x >> 31;
  return x;
}

// ---- system-scope memory operations (peer memory over NVLink / NVSwitch) ----
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t* p) {
  uint64_t v; asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
  uint32_t v; asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v; asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
  uint64_t v; asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" :: "l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_f32(float* p, float v) {
  asm volatile("st.relaxed.sys.global.f32 [%0], %1;" :: "l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void red_add_sys_f32(float* p, float v) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" :: "l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t;
}

// ---- L2 residency hints ----
// A minibatch step streams large arrays once (keys, slot maps, inbox records) next to hash
// tables that are probed at random many times.  Streams carry an evict-first policy so that
// they do not push the tables out of the 126 MB L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
  uint64_t p; asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p)); return p;
}
__device__ __forceinline__ uint64_t l2_evict_last_policy() {
  uint64_t p; asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p)); return p;
}
__device__ __forceinline__ uint64_t ld_stream_u64(const uint64_t* p, uint64_t pol) {
  uint64_t v; asm volatile("ld.global.L2::cache_hint.u64 %0, [%1], %2;" : "=l"(v) : "l"(p), "l"(pol)); return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const uint32_t* p, uint64_t pol) {
  uint32_t v; asm volatile("ld.global.L2::cache_hint.u32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol)); return v;
}
__device__ __forceinline__ float ld_stream_f32(const float* p, uint64_t pol) {
  float v; asm volatile("ld.global.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(pol)); return v;
}
__device__ __forceinline__ void st_stream_u32(uint32_t* p, uint32_t v, uint64_t pol) {
  asm volatile("st.global.L2::cache_hint.u32 [%0], %1, %2;" :: "l"(p), "r"(v), "l"(pol) : "memory");
}

// Wait until (*flag >> 32) >= want_epoch, at most timeout_ns. Returns the flag
// value on success; on timeout sets *ok=false and returns the last value seen.
__device__ __forceinline__ uint64_t wait_epoch_ge(const uint64_t* flag, uint32_t want_epoch,
                                                  uint64_t timeout_ns, bool* ok) {
  const uint64_t t0 = globaltimer_ns();
  const uint64_t max_iters = timeout_ns / 32 + 1024;
  uint64_t v = 0;
  for (uint64_t it = 0; it < max_iters; ++it) {
    v = ld_acquire_sys_u64(flag);
    if ((uint32_t)(v >> 32) >= want_epoch) { *ok = true; return v; }
    if ((it & 63) == 63 && globaltimer_ns() - t0 > timeout_ns) break;
    __nanosleep(40);
  }
  *ok = false;
  return v;
}

// ---- key-range routing (≤ 8 separators, kept in kernel-parameter space) ----
struct KeySeps {
  uint64_t sep[PSB_MAX_RANKS + 1];  // owner s holds keys in [sep[s], sep[s+1])
  int world;
};
__device__ __forceinline__ int route_owner(const KeySeps& s, uint64_t key) {
  int o = 0;
#pragma unroll
  for (int i = 1; i < PSB_MAX_RANKS; ++i) o += (i < s.world && key >= s.sep[i]) ? 1 : 0;
  return o;
}

// ---- warp helpers ----
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- open-addressing u64 set/map probes ----
// insert-or-find in a local (same GPU) table; returns slot or ~0ull when the
// probe limit is hit.  Probing wraps inside the aligned chunk of (chunk_mask + 1) slots that
// holds the home slot h, so a key never leaves its home chunk (chunk_mask = mask: whole table).
// *inserted (optional) is set when this call created the entry.
__device__ __forceinline__ uint64_t table_find_or_insert(uint64_t* keys, uint64_t mask, uint64_t chunk_mask,
                                                        uint64_t h, uint64_t key, int max_probe,
                                                        bool* inserted = nullptr) {
  uint64_t slot = h & mask;
  const uint64_t base = slot & ~chunk_mask;
  for (int i = 0; i < max_probe; ++i) {
    uint64_t cur = keys[slot];
    if (cur == key) return slot;
    if (cur == kEmptyKey) {
      unsigned long long prev = atomicCAS(reinterpret_cast<unsigned long long*>(keys + slot),
                                          (unsigned long long)kEmptyKey, (unsigned long long)key);
      if (prev == kEmptyKey) { if (inserted != nullptr) *inserted = true; return slot; }
      if (prev == key) return slot;
    }
    slot = base | ((slot + 1) & chunk_mask);
  }
  return ~0ull;
}

// ---- count-min sketch probes (src/base/countmin.h:33-67) ----
// 32-bit hash of a 64-bit key; probe j of k looks at (h + j·rotr17(h)) mod width.
__device__ __forceinline__ uint32_t cm_hash(uint64_t key) {
  const uint32_t seed = 0xbc9f1d34u, m = 0xc6a4a793u;
  uint32_t h = seed ^ (8u * m);
  h += (uint32_t)key; h *= m; h ^= (h >> 16);
  h += (uint32_t)(key >> 32); h *= m; h ^= (h >> 16);
  return h;
}
__device__ __forceinline__ void cm_insert(uint32_t* table, uint32_t width, int k, uint64_t key, uint32_t c) {
  uint32_t h = cm_hash(key);
  const uint32_t d = (h >> 17) | (h << 15);
  for (int j = 0; j < k; ++j) { atomicAdd(&table[h % width], c); h += d; }
}
__device__ __forceinline__ uint32_t cm_query(const uint32_t* table, uint32_t width, int k, uint64_t key, uint32_t wrap_mask) {
  uint32_t h = cm_hash(key), r = 0xFFFFFFFFu;
  const uint32_t d = (h >> 17) | (h << 15);
  for (int j = 0; j < k; ++j) { r = min(r, __ldcg(table + h % width) & wrap_mask); h += d; }
  return r;
}

// numerically safe log(1+exp(x))
__device__ __forceinline__ float log1pexp(float x) {
  return x > 0.f ? x + log1pf(__expf(-x)) : log1pf(__expf(x));
}

}  // namespace psb
