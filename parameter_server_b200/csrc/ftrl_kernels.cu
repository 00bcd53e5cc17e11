// Online FTRL-proximal on key-range sharded device hash tables: the two fused
// communication+compute kernels of the product path, plus the same phases as
// stand-alone kernels for the unfused NCCL baseline.
//
// One rank = one GPU = worker r (streams minibatches) + server r (owns the keys
// of [sep[r], sep[r+1]) in an open-addressing table {key -> w, z, pos, neg}).
//
//   ftrl_pull_spmv  : de-duplicate the minibatch's keys into a per-minibatch table
//                     that is laid out by owner; every owner then reads "its" region
//                     of every worker's table with coalesced peer loads over NVLink,
//                     looks the keys up in its own shard (creating missing ones),
//                     remembers the shard slot of every request and stores the
//                     weights straight into the worker's weight array with coalesced
//                     peer stores; the worker runs the CSR SpMV X·w, the logistic
//                     loss and the per-row coefficient −y/(1+e^{y·Xw}) — one
//                     cooperative kernel.
//   ftrl_push_update: Xᵀ·coef and the pos/neg row counts per unique key into the
//                     worker's accumulator array; every owner reads its region of
//                     every worker's accumulators with coalesced peer loads and
//                     applies the FTRL update to the slots it remembered, worker by
//                     worker — one cooperative kernel.
//
// No key is hashed twice on the owner, no record is packed, routed or copied into an
// inbox: the per-minibatch table IS the message, and what crosses NVLink are whole
// 1024-slot chunks (8 bytes of key out, 4 bytes of weight back, 4 or 16 bytes of
// gradient out per slot).
//
// The arithmetic is the reference's server rule FTRLModel::setValue
// (src/linear_method/ftrl_model.h:81-112), the worker gradient of LogitLoss
// (src/linear_method/loss.h:73-88) and FTRL::countKeys
// (src/linear_method/ftrl.cc:154-174); the message flow replaces
// SharedParameter::push/pull (src/parameter/shared_parameter.h:14-26,90-149) and
// KVVector::getValue (src/parameter/kv_vector.h:215-227).
// The schedule is bulk-synchronous (one legal serialisation of the reference's
// eventual-consistency execution): pull(e) sees every update of step e-1.
#include <cstddef>
#include <cstdlib>

#include "psb_common.cuh"

namespace psb {

struct ShardState {  // per-key state as the update rule sees it
  float w;
  float z;
  uint32_t pos;  // rule 0: #positive rows seen; rule 1: bit pattern of Σg² (float)
  uint32_t neg;
};

// One slot of an owner's table: 32 bytes = one DRAM sector.  Key and weight sit in
// the same 16 bytes, so a lookup is ONE 16-byte load per probe; an update is a
// read-modify-write of the same sector.
struct __align__(32) ShardSlot {
  uint64_t key;      // offset 0: kEmptyKey when free
  float w;           // offset 8
  float z;           // offset 12
  uint32_t pos;      // offset 16
  uint32_t neg;      // offset 20
  uint64_t reserved; // offset 24
};
static_assert(sizeof(ShardSlot) == 32 && offsetof(ShardSlot, w) == 8 && offsetof(ShardSlot, pos) == 16, "ShardSlot layout");

struct FtrlHyper {
  float alpha, beta, l1, l2;
  int rule;  // 0 = count-based ‖g‖ estimate (reference), 1 = Σ g² (McMahan et al.)
  int pad;
  // Tail-feature filter (src/linear_method/ftrl.cc:99-106, src/parameter/frequency_filter.h:28-43):
  // the owner adds every pushed key's row count to its count-min sketch and updates (and creates)
  // a key only once the estimate exceeds tail_freq, so rare keys never enter the model.  The
  // reference filters on the pull path; here the counts travel with the push anyway, the sketch
  // is local to the owner, and a key without a table entry pulls as 0 — the same model, no extra
  // message.  Off when tail_freq == 0 or cm == nullptr.
  uint32_t* cm;
  uint32_t cm_width;
  int cm_k;
  uint32_t tail_freq;
  uint32_t pad2;
};

// The per-minibatch table of every rank is cut into one region of R = 2^region_log2 slots per
// owner: a key of owner o lives in region o at the top region_log2 bits of its hash (linear
// probing confined to an aligned chunk of kChunkSlots slots).  The shard tables index with the
// top bits of the same hash, so chunk c of region o on EVERY worker covers the same contiguous
// range of owner o's shard table: an owner block that takes chunk c walks all workers' requests
// for one narrow range of its table, and the same key sent by two workers is always in the
// same chunk (worker-by-worker order needs block-level barriers only).
constexpr int kChunkSlots = 1024;
constexpr uint32_t kBadSlot = 0xFFFFFFFFu;   // request slot is empty
constexpr uint32_t kAbsent = 0xFFFFFFFEu;    // key has no entry in the shard (and none was made)

struct FtrlPeers {
  KeySeps seps;
  int rank;
  int max_probe;
  uint64_t tab_mask;                       // shard capacity − 1
  ShardSlot* tab;                          // this rank's shard (only its owner touches it)
  uint64_t* lt_keys[PSB_MAX_RANKS];        // rank r: per-minibatch key table [world << region_log2]
  float* lt_w[PSB_MAX_RANKS];              // rank r: pulled weight per slot (written by the owners)
  void* lt_acc[PSB_MAX_RANKS];             // rank r: gradient accumulators, two buffers of float or float4 per slot
  uint64_t* ready[PSB_MAX_RANKS];          // rank o: [sender] pull sequence whose table is complete
  uint64_t* replied[PSB_MAX_RANKS];        // rank s: [owner]  pull sequence whose weights are written
  uint64_t* grads[PSB_MAX_RANKS];          // rank o: [sender] push sequence whose accumulators are complete
  uint32_t* in_slot;                       // owner: [sender << region_log2 | index] shard slot of the request
  uint64_t* in_keys;                       // owner: copy of the requested keys (tail filter only, else nullptr)
  uint64_t timeout_ns;
  uint32_t tab_shift;                      // 64 − log2(shard capacity): slot = mix64(key) >> tab_shift
  uint32_t region_log2;
};

struct Minibatch {
  const void* offsets;     // rows+1, int64 (or int32 when off32)
  const void* keys;        // nnz keys: uint64, or uint32 feature ids (key_mode 1, 2)
  const float* vals;       // nnz values or nullptr (binary features)
  const float* y;          // rows, ±1
  int64_t nnz;
  int rows;
  uint16_t off32;          // offsets are int32
  uint16_t key_mode;       // 0: uint64 keys; 1: uint32 ids, key = id; 2: uint32 ids, key = mix64(id)
};

__device__ __forceinline__ int64_t mb_offset(const Minibatch& M, int64_t r) {
  return M.off32 ? (int64_t) reinterpret_cast<const int32_t*>(M.offsets)[r] : reinterpret_cast<const int64_t*>(M.offsets)[r];
}

struct __align__(16) AccSlot {  // accumulator of one per-minibatch slot when row counts are tracked
  float g;    // gradient
  float pos;  // #positive rows containing the key (exact in fp32: a minibatch has < 2^24 rows)
  float neg;  // #negative rows containing the key
  float pad;
};

// One 16-byte vector reduction per non-zero instead of separate atomics on g and counts.
__device__ __forceinline__ void red_add_acc(AccSlot* p, float g, float pos, float neg) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(g), "f"(pos), "f"(neg), "f"(0.f) : "memory");
}

struct LocalScratch {
  uint64_t* lt_keys;   // this rank's per-minibatch table (all kEmptyKey between steps)
  float* lt_w;         // pulled weight per slot
  void* lt_acc;        // accumulators: [2][slots] float (soa) or AccSlot
  uint64_t lt_slots;   // world << region_log2
  uint32_t* slot_of;   // nnz: local slot of each non-zero
  float* coef;         // rows: −y/(1+e^{y·Xw})
  float* xw;           // rows: X·w (predictions)
  uint32_t* send_cnt;  // [PSB_MAX_RANKS] scratch of the unfused baseline
  uint32_t* recv_cnt;  // [PSB_MAX_RANKS] scratch of the unfused baseline
  double* stats;       // [0] Σloss [1] rows [2] ‖w‖₁ [3] ‖w‖₂² [4] nnz(w) [5] unique keys [6] table entries
  uint32_t* status;    // StatusCode etc.
  uint64_t* trace;     // optional [16]: globaltimer at phase boundaries of the last step (see kTrace*)
  // soa != 0: no pos/neg row counts are tracked, an accumulator is one float (the random
  // accesses of the gradient scatter then stay inside L2: a quarter of the footprint).
  uint32_t soa;
  uint32_t parity;     // which of the two accumulator buffers this step uses
};

template <bool kCounts>
__device__ __forceinline__ size_t acc_bytes() { return kCounts ? sizeof(AccSlot) : sizeof(float); }

// Streams (keys, slot map) are read or written once per phase; they carry an evict-first L2 policy so
// that the hash tables stay resident (gradient phase 200 -> 181 us with 16-byte accumulators, measured).
#define PSB_STREAM_POLICY(pol) const uint64_t pol = l2_evict_first_policy()
#define PSB_LD_U64(p, pol) ld_stream_u64((p), (pol))
#define PSB_LD_U32(p, pol) ld_stream_u32((p), (pol))
#define PSB_LD_F32(p, pol) ld_stream_f32((p), (pol))
#define PSB_ST_U32(p, v, pol) st_stream_u32((p), (v), (pol))

// trace slots: pull kernel 0 start, 1 localized, 2 all owners replied, 3 block-0 end;
//              push kernel 4 start, 5 gradients done, 6 flags sent and tables cleared, 8 applied
#define PSB_TRACE(L, gtid, i) do { if ((L).trace != nullptr && (gtid) == 0) (L).trace[i] = globaltimer_ns(); } while (0)

// Both tables index with the TOP bits of the same 64-bit hash (see FtrlPeers).
__device__ __forceinline__ uint64_t shard_hash(uint64_t key, uint32_t shift) { return mix64(key) >> shift; }

__device__ __forceinline__ uint64_t mb_key(const Minibatch& M, int64_t i, uint64_t pol) {
  if (M.key_mode == 0) return PSB_LD_U64(reinterpret_cast<const uint64_t*>(M.keys) + i, pol);
  const uint64_t id = PSB_LD_U32(reinterpret_cast<const uint32_t*>(M.keys) + i, pol);
  return M.key_mode == 2 ? mix64(id) : id;
}

// slot of `key` in a per-minibatch table: region of its owner, top bits of its hash inside
__device__ __forceinline__ uint64_t local_home(const FtrlPeers& P, uint64_t key) {
  const uint64_t o = (uint64_t)route_owner(P.seps, key);
  const uint64_t h = P.region_log2 ? (mix64(key) >> (64 - P.region_log2)) : 0ull;
  return (o << P.region_log2) | h;
}

// ------------------------------------------------------------------ phases
// De-duplication of the minibatch's keys is bound by memory latency, not by bandwidth: every key
// costs a streamed load of the key and then a dependent random read of the table.  The loop is
// therefore software-pipelined: while key i is resolved, the table read of the thread's next key
// and the load of the key after that are already in flight (the asm loads are issued in program
// order, their results are used one and two iterations later).  A table read that is stale by the
// time it is used only sends the key through the compare-and-swap path, which re-reads.
__device__ __forceinline__ uint64_t ld_table_u64(const uint64_t* p) {
  uint64_t v; asm volatile("ld.global.u64 %0, [%1];" : "=l"(v) : "l"(p)); return v;
}

__device__ __forceinline__ void phase_localize(const FtrlPeers& P, const Minibatch& M, const LocalScratch& L,
                                               size_t gtid, size_t gsz) {
  PSB_STREAM_POLICY(pol);
  const int64_t step = (int64_t)gsz;
  const uint64_t region = 1ull << P.region_log2;
  const uint64_t cmask = (region < (uint64_t)kChunkSlots ? region : (uint64_t)kChunkSlots) - 1;
  uint32_t fresh = 0;
  int64_t i = (int64_t)gtid;
  if (i < M.nnz) {
    uint64_t key0 = mb_key(M, i, pol);
    uint64_t key1 = i + step < M.nnz ? mb_key(M, i + step, pol) : kEmptyKey;
    uint64_t h0 = local_home(P, key0);
    uint64_t cur0 = ld_table_u64(L.lt_keys + h0);
    for (; i < M.nnz; i += step) {
      uint64_t key2 = kEmptyKey, h1 = 0, cur1 = 0;
      if (i + 2 * step < M.nnz) key2 = mb_key(M, i + 2 * step, pol);
      if (i + step < M.nnz) {
        h1 = local_home(P, key1);
        cur1 = ld_table_u64(L.lt_keys + h1);
      }
      uint32_t slot = (uint32_t)h0;
      if (cur0 != key0) {
        bool inserted = false;
        const uint64_t s = table_find_or_insert(L.lt_keys, ~0ull, cmask, h0, key0, P.max_probe, &inserted);
        if (s == ~0ull) {
          set_status(L.status, kLocalTableFull, 0, 0);
          slot = kBadSlot;
        } else {
          slot = (uint32_t)s;
          fresh += inserted ? 1u : 0u;
        }
      }
      PSB_ST_U32(L.slot_of + i, slot, pol);
      key0 = key1; h0 = h1; cur0 = cur1; key1 = key2;
    }
  }
  fresh = __reduce_add_sync(0xffffffffu, fresh);
  if ((threadIdx.x & 31) == 0 && fresh) atomicAdd(&L.stats[5], (double)fresh);
}

// ---- shard table probes (owner side, this GPU's own memory)
// weight of `key` and its slot; kAbsent when the key has no entry
__device__ __forceinline__ uint32_t shard_find(const ShardSlot* tab, uint64_t mask, uint32_t shift, uint64_t key,
                                               int max_probe, float* w) {
  uint64_t slot = shard_hash(key, shift) & mask;
  for (int i = 0; i < max_probe; ++i) {
    uint64_t k, wz;
    asm volatile("ld.global.v2.u64 {%0, %1}, [%2];" : "=l"(k), "=l"(wz) : "l"(tab + slot) : "memory");
    if (k == key) { *w = __uint_as_float((uint32_t)wz); return (uint32_t)slot; }
    if (k == kEmptyKey) break;
    slot = (slot + 1) & mask;
  }
  *w = 0.f;
  return kAbsent;
}

// slot of `key`, created when missing (w = z = n = 0: the same model as "absent"); kAbsent when the
// probe limit is reached
__device__ __forceinline__ uint32_t shard_find_or_insert(ShardSlot* tab, uint64_t mask, uint32_t shift, uint64_t key,
                                                         int max_probe, float* w, int* inserted) {
  uint64_t slot = shard_hash(key, shift) & mask;
  for (int i = 0; i < max_probe; ++i) {
    uint64_t k, wz;
    asm volatile("ld.global.v2.u64 {%0, %1}, [%2];" : "=l"(k), "=l"(wz) : "l"(tab + slot) : "memory");
    if (k == key) { *w = __uint_as_float((uint32_t)wz); return (uint32_t)slot; }
    if (k == kEmptyKey) {
      const unsigned long long prev = atomicCAS(reinterpret_cast<unsigned long long*>(&tab[slot].key),
                                                (unsigned long long)kEmptyKey, (unsigned long long)key);
      if (prev == kEmptyKey) { *w = 0.f; ++*inserted; return (uint32_t)slot; }
      if (prev == key) { *w = tab[slot].w; return (uint32_t)slot; }
    }
    slot = (slot + 1) & mask;
  }
  *w = 0.f;
  return kAbsent;
}

// One thread of a block waits (bounded) until flag's epoch reaches `want`; the block learns the outcome.
__device__ __forceinline__ bool block_wait_flag(const uint64_t* flag, uint32_t want, uint64_t timeout_ns, int* sh_ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    bool ok;
    wait_epoch_ge(flag, want, timeout_ns, &ok);
    *sh_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return *sh_ok != 0;
}

constexpr int kLookupItems = kChunkSlots / 256;   // slots per thread and chunk (blocks of 256 threads)

// Owner side of the pull.  A task is (sender s, chunk c of this owner's region in s's table).
// Tasks are numbered sender-major starting with this rank itself, so the blocks that serve
// different senders wait for different flags and a slow sender holds up only its own blocks.
// `insert`: create missing keys (training); off for predictions and under the tail filter.
__device__ __forceinline__ void phase_lookup(const FtrlPeers& P, const LocalScratch& L, uint32_t seq, bool insert,
                                             int* sh_ok) {
  const int world = P.seps.world;
  const uint64_t region = 1ull << P.region_log2;
  const uint32_t chunk = region < (uint64_t)kChunkSlots ? (uint32_t)region : (uint32_t)kChunkSlots;
  const uint32_t chunks = (uint32_t)(region / chunk);
  const uint32_t tasks = chunks * (uint32_t)world;
  int dins = 0;
  int have = -1;   // sender whose flag this block has seen
  bool have_ok = false;
  for (uint32_t t = blockIdx.x; t < tasks; t += gridDim.x) {
    const int s = (P.rank + (int)(t / chunks)) % world;
    const uint32_t c = t % chunks;
    if (s != have) {
      have_ok = s == P.rank ? true : block_wait_flag(P.ready[P.rank] + s, seq, P.timeout_ns, sh_ok);
      have = s;
      if (!have_ok && threadIdx.x == 0) set_status(L.status, kWaitTimeout, (uint32_t)s, 1);
    }
    const size_t in0 = ((size_t)s << P.region_log2) + (size_t)c * chunk;          // owner-side index
    const size_t lt0 = ((size_t)P.rank << P.region_log2) + (size_t)c * chunk;     // index in the sender's table
    const bool peer = s != P.rank;
    const uint64_t* rk = P.lt_keys[s] + lt0;
    float* rw = P.lt_w[s] + lt0;
    uint64_t key[kLookupItems];
#pragma unroll
    for (int k = 0; k < kLookupItems; ++k) {
      const uint32_t i = (uint32_t)k * 256u + threadIdx.x;
      key[k] = kEmptyKey;
      if (i < chunk && have_ok) key[k] = peer ? ld_relaxed_sys_u64(rk + i) : __ldcg(rk + i);
    }
#pragma unroll
    for (int k = 0; k < kLookupItems; ++k) {
      const uint32_t i = (uint32_t)k * 256u + threadIdx.x;
      if (i >= chunk) continue;
      uint32_t slot = kBadSlot;
      float w = 0.f;
      if (key[k] != kEmptyKey) {
        slot = insert ? shard_find_or_insert(P.tab, P.tab_mask, P.tab_shift, key[k], P.max_probe, &w, &dins)
                      : shard_find(P.tab, P.tab_mask, P.tab_shift, key[k], P.max_probe, &w);
        if (insert && slot == kAbsent) set_status(L.status, kShardTableFull, 0, 0);
      }
      P.in_slot[in0 + i] = slot;
      if (P.in_keys != nullptr) P.in_keys[in0 + i] = key[k];
      if (have_ok) {
        if (peer) st_relaxed_sys_f32(rw + i, w); else rw[i] = w;
      }
    }
  }
  dins = __reduce_add_sync(0xffffffffu, dins);
  if ((threadIdx.x & 31) == 0 && dins) atomicAdd(&L.stats[6], (double)dins);
}

// Rows are walked a warp at a time; a lane first issues the loads of up to kRowBatch of its
// non-zeros, then consumes them, so that several slot-map loads are in flight per lane.
constexpr int kRowBatch = 4;

__device__ __forceinline__ void phase_spmv_loss(const Minibatch& M, const LocalScratch& L, size_t gwarp,
                                                size_t nwarps, int lane) {
  double loss = 0.0;
  PSB_STREAM_POLICY(pol);
  for (int64_t row = (int64_t)gwarp; row < M.rows; row += (int64_t)nwarps) {
    const int64_t b = mb_offset(M, row), e = mb_offset(M, row + 1);
    float s = 0.f;
    for (int64_t i0 = b + lane; i0 < e; i0 += 32 * kRowBatch) {
      uint32_t sl[kRowBatch];
      float x[kRowBatch];
#pragma unroll
      for (int k = 0; k < kRowBatch; ++k) {
        const int64_t i = i0 + 32 * k;
        sl[k] = i < e ? PSB_LD_U32(L.slot_of + i, pol) : kBadSlot;
        x[k] = (M.vals != nullptr && i < e) ? PSB_LD_F32(M.vals + i, pol) : 1.f;
      }
#pragma unroll
      for (int k = 0; k < kRowBatch; ++k) {
        if (sl[k] != kBadSlot) s += x[k] * __ldcg(L.lt_w + sl[k]);   // written by other GPUs: not through L1
      }
    }
    s = warp_sum(s);
    if (lane == 0) {
      const float y = M.y[row];
      const float m = y * s;
      loss += (double)log1pexp(-m);
      L.coef[row] = -y / (1.f + __expf(m));
      L.xw[row] = s;
    }
  }
  if (lane == 0 && loss != 0.0) atomicAdd(&L.stats[0], loss);
}

// Block-local cache of gradient accumulators for frequently hit slots.  Under Zipf
// popularity a few keys receive a large share of all non-zeros; accumulating them in
// shared memory and flushing once per block removes the same-address serialisation of
// global atomics.  Entries are claimed first come, first served; a slot that finds its
// cache line taken by another slot falls back to the global atomic.
constexpr int kHotLog2 = 10;
constexpr int kHotEntries = 1 << kHotLog2;
struct HotCache {
  uint32_t slot[kHotEntries];
  float g[kHotEntries];
  unsigned long long cnt[kHotEntries];
};

template <bool kCounts>
__device__ __forceinline__ void phase_grad(const Minibatch& M, const LocalScratch& L, size_t gwarp,
                                           size_t nwarps, int lane, HotCache* hc) {
  float* accf = reinterpret_cast<float*>(L.lt_acc) + (size_t)L.parity * L.lt_slots;
  AccSlot* accv = reinterpret_cast<AccSlot*>(L.lt_acc) + (size_t)L.parity * L.lt_slots;
  for (int i = threadIdx.x; i < kHotEntries; i += blockDim.x) {
    hc->slot[i] = kBadSlot;
    hc->g[i] = 0.f;
    if (kCounts) hc->cnt[i] = 0ull;
  }
  __syncthreads();
  PSB_STREAM_POLICY(pol);
  for (int64_t row = (int64_t)gwarp; row < M.rows; row += (int64_t)nwarps) {
    const int64_t b = mb_offset(M, row), e = mb_offset(M, row + 1);
    const float c = L.coef[row];
    const bool is_pos = M.y[row] > 0.f;
    const unsigned long long inc = is_pos ? (1ull << 32) : 1ull;
    for (int64_t i0 = b + lane; i0 < e; i0 += 32 * kRowBatch) {
      uint32_t sls[kRowBatch];
      float x[kRowBatch];
#pragma unroll
      for (int k = 0; k < kRowBatch; ++k) {
        const int64_t i = i0 + 32 * k;
        sls[k] = i < e ? PSB_LD_U32(L.slot_of + i, pol) : kBadSlot;
        x[k] = (M.vals != nullptr && i < e) ? PSB_LD_F32(M.vals + i, pol) : 1.f;
      }
#pragma unroll
      for (int k = 0; k < kRowBatch; ++k) {
        const uint32_t sl = sls[k];
        if (sl == kBadSlot) continue;
        const float gv = c * x[k];
        const int h = (int)((sl * 2654435761u) >> (32 - kHotLog2));  // top bits
        uint32_t cur = hc->slot[h];
        if (cur == kBadSlot) {
          const uint32_t prev = atomicCAS(&hc->slot[h], kBadSlot, sl);
          cur = prev == kBadSlot ? sl : prev;
        }
        if (cur == sl) {
          atomicAdd(&hc->g[h], gv);
          if (kCounts) atomicAdd(&hc->cnt[h], inc);
        } else if (kCounts) {
          red_add_acc(accv + sl, gv, is_pos ? 1.f : 0.f, is_pos ? 0.f : 1.f);
        } else {
          atomicAdd(accf + sl, gv);
        }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < kHotEntries; i += blockDim.x) {
    const uint32_t sl = hc->slot[i];
    if (sl != kBadSlot) {
      if (kCounts) {
        const unsigned long long c = hc->cnt[i];
        red_add_acc(accv + sl, hc->g[i], (float)(uint32_t)(c >> 32), (float)(uint32_t)c);
      } else {
        atomicAdd(accf + sl, hc->g[i]);
      }
    }
  }
}

// Between the gradient phase and the owners' update a worker empties its key table for the next
// minibatch (every owner has finished reading it: the worker saw all `replied` flags before its
// SpMV) and zeroes the accumulator buffer of the NEXT step (the owners read that one during the
// previous step's update, which they finished before they replied to this step's pull).
template <bool kCounts>
__device__ __forceinline__ void phase_reset_tables(const LocalScratch& L, size_t gtid, size_t gsz) {
  uint4* k = reinterpret_cast<uint4*>(L.lt_keys);
  const uint4 empty = make_uint4(0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu, 0xFFFFFFFFu);
  for (size_t i = gtid; i < L.lt_slots / 2; i += gsz) k[i] = empty;
  if (L.lt_slots & 1) { if (gtid == 0) L.lt_keys[L.lt_slots - 1] = kEmptyKey; }
  const size_t bytes = L.lt_slots * acc_bytes<kCounts>();
  char* next = reinterpret_cast<char*>(L.lt_acc) + (size_t)(L.parity ^ 1u) * bytes;
  uint4* a = reinterpret_cast<uint4*>(next);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (size_t i = gtid; i < bytes / 16; i += gsz) a[i] = zero;
  for (size_t i = (bytes / 16) * 16 + gtid; i < bytes; i += gsz) next[i] = 0;
}

__device__ __forceinline__ float ftrl_sqrt_n(float pos, float neg) {
  const float all = pos + neg;
  return all == 0.f ? 0.f : sqrtf(pos * neg / all);
}

// The reference's per-key server update (src/linear_method/ftrl_model.h:88-110).
__device__ __forceinline__ void ftrl_update(ShardState& e, float g, uint32_t dpos, uint32_t dneg,
                                            const FtrlHyper& h, float& dn1, float& dn2, int& dnnz) {
  float sqrt_n, sqrt_n_new;
  if (h.rule == 0) {
    sqrt_n = ftrl_sqrt_n((float)e.pos, (float)e.neg);
    e.pos += dpos;
    e.neg += dneg;
    sqrt_n_new = ftrl_sqrt_n((float)e.pos, (float)e.neg);
  } else {
    float n = __uint_as_float(e.pos);
    sqrt_n = sqrtf(n);
    n += g * g;
    sqrt_n_new = sqrtf(n);
    e.pos = __float_as_uint(n);
    e.neg += dpos + dneg;
  }
  const float sigma = (sqrt_n_new - sqrt_n) / h.alpha;
  e.z += g - sigma * e.w;
  const float l2 = h.l2 + (h.beta + sqrt_n_new) / h.alpha;
  const float w_old = e.w;
  const float az = fabsf(e.z) - h.l1;
  const float w = az > 0.f ? -copysignf(az, e.z) / l2 : 0.f;
  e.w = w;
  dn1 += fabsf(w) - fabsf(w_old);
  dn2 += w * w - w_old * w_old;
  dnnz += (w != 0.f && w_old == 0.f) - (w == 0.f && w_old != 0.f);
}

__device__ __forceinline__ bool tail_filter_on(const FtrlHyper& h) { return h.tail_freq != 0u && h.cm != nullptr; }

struct ApplyAcc {  // per-thread deltas of the model statistics, flushed once per kernel
  float dn1 = 0.f, dn2 = 0.f;
  int dnnz = 0, dins = 0;
};

__device__ __forceinline__ void apply_flush(ApplyAcc& a, double* stats) {
  const float dn1 = warp_sum(a.dn1), dn2 = warp_sum(a.dn2);
  const int dnnz = __reduce_add_sync(0xffffffffu, a.dnnz), dins = __reduce_add_sync(0xffffffffu, a.dins);
  if ((threadIdx.x & 31) == 0) {
    if (dn1 != 0.f) atomicAdd(stats + 2, (double)dn1);
    if (dn2 != 0.f) atomicAdd(stats + 3, (double)dn2);
    if (dnnz != 0) atomicAdd(stats + 4, (double)dnnz);
    if (dins != 0) atomicAdd(stats + 6, (double)dins);
  }
  a = ApplyAcc();
}

__device__ __forceinline__ void apply_slot(ShardSlot* tab, uint32_t slot, float g, uint32_t dpos, uint32_t dneg,
                                           const FtrlHyper& h, ApplyAcc& acc) {
  const float2 wz = *reinterpret_cast<const float2*>(&tab[slot].w);
  const uint2 pn = *reinterpret_cast<const uint2*>(&tab[slot].pos);
  ShardState e;
  e.w = wz.x; e.z = wz.y; e.pos = pn.x; e.neg = pn.y;
  ftrl_update(e, g, dpos, dneg, h, acc.dn1, acc.dn2, acc.dnnz);
  *reinterpret_cast<float2*>(&tab[slot].w) = make_float2(e.w, e.z);
  *reinterpret_cast<uint2*>(&tab[slot].pos) = make_uint2(e.pos, e.neg);
}

// gradient (and row counts) of request `i` of a chunk, from the sender's accumulators
template <bool kCounts>
__device__ __forceinline__ void load_acc(const void* base, size_t i, bool peer, float* g, uint32_t* dpos, uint32_t* dneg) {
  if (kCounts) {
    const AccSlot* p = reinterpret_cast<const AccSlot*>(base) + i;
    float4 v;
    if (peer)
      asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
    else
      v = __ldcg(reinterpret_cast<const float4*>(p));
    *g = v.x; *dpos = (uint32_t)v.y; *dneg = (uint32_t)v.z;
  } else {
    const float* p = reinterpret_cast<const float*>(base) + i;
    *g = peer ? ld_relaxed_sys_f32(p) : __ldcg(p);
    *dpos = 0u; *dneg = 0u;
  }
}

// Owner side of the push: chunk c of every sender, sender by sender in rank order (the reference
// applies each worker's push separately; the order only matters per key, and a key is in the
// same chunk on every sender).  The shard slots were resolved by the pull of the same step.
template <bool kCounts>
__device__ __forceinline__ void phase_apply_chunks(const FtrlPeers& P, const LocalScratch& L, const FtrlHyper& H,
                                                   uint32_t seq, ApplyAcc& acc, int* sh_ok) {
  const int world = P.seps.world;
  const uint64_t region = 1ull << P.region_log2;
  const uint32_t chunk = region < (uint64_t)kChunkSlots ? (uint32_t)region : (uint32_t)kChunkSlots;
  const uint32_t chunks = (uint32_t)(region / chunk);
  const size_t abytes = L.lt_slots * acc_bytes<kCounts>();
  uint32_t arrived = 0, failed = 0;   // bit s: this block has seen sender s's flag / its wait ran out
  for (uint32_t c = blockIdx.x; c < chunks; c += gridDim.x) {
    for (int s = 0; s < world; ++s) {
      if (!((arrived | failed) >> s & 1u)) {
        const bool ok = s == P.rank ? true : block_wait_flag(P.grads[P.rank] + s, seq, P.timeout_ns, sh_ok);
        if (ok) arrived |= 1u << s; else failed |= 1u << s;
        if (!ok && threadIdx.x == 0) set_status(L.status, kWaitTimeout, (uint32_t)s, 2);
      }
      if (failed >> s & 1u) continue;   // a sender that never arrived is skipped
      const size_t in0 = ((size_t)s << P.region_log2) + (size_t)c * chunk;
      const size_t lt0 = ((size_t)P.rank << P.region_log2) + (size_t)c * chunk;
      const bool peer = s != P.rank;
      const char* abase = reinterpret_cast<const char*>(P.lt_acc[s]) + (size_t)L.parity * abytes;
      uint32_t slot[kLookupItems];
#pragma unroll
      for (int k = 0; k < kLookupItems; ++k) {
        const uint32_t i = (uint32_t)k * 256u + threadIdx.x;
        slot[k] = i < chunk ? __ldcg(P.in_slot + in0 + i) : kBadSlot;
      }
#pragma unroll
      for (int k = 0; k < kLookupItems; ++k) {
        const uint32_t i = (uint32_t)k * 256u + threadIdx.x;
        if (slot[k] >= kAbsent) continue;
        float g; uint32_t dpos, dneg;
        load_acc<kCounts>(abase, lt0 + i, peer, &g, &dpos, &dneg);
        apply_slot(P.tab, slot[k], g, dpos, dneg, H, acc);
      }
      __syncthreads();
    }
  }
}

// Tail-filter form of the owner's update: a sender's counts must all be in the sketch before any
// of its keys is queried, so every sender is bracketed by grid-wide barriers; keys that pass the
// filter and have no entry yet get one here (the pull did not create them).
__device__ __forceinline__ void phase_apply_filtered(cg::grid_group& grid, const FtrlPeers& P, const LocalScratch& L,
                                                     const FtrlHyper& H, uint32_t seq, ApplyAcc& acc, int* sh_ok) {
  const int world = P.seps.world;
  const uint64_t region = 1ull << P.region_log2;
  const size_t abytes = L.lt_slots * sizeof(AccSlot);
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, gsz = (size_t)gridDim.x * blockDim.x;
  for (int s = 0; s < world; ++s) {
    const bool ok = s == P.rank ? true : block_wait_flag(P.grads[P.rank] + s, seq, P.timeout_ns, sh_ok);
    if (!ok && threadIdx.x == 0) set_status(L.status, kWaitTimeout, (uint32_t)s, 2);
    const size_t in0 = (size_t)s << P.region_log2, lt0 = (size_t)P.rank << P.region_log2;
    const bool peer = s != P.rank;
    const char* abase = reinterpret_cast<const char*>(P.lt_acc[s]) + (size_t)L.parity * abytes;
    for (size_t i = gtid; ok && i < region; i += gsz) {
      const uint64_t key = P.in_keys[in0 + i];
      if (key == kEmptyKey) continue;
      float g; uint32_t dpos, dneg;
      load_acc<true>(abase, lt0 + i, peer, &g, &dpos, &dneg);
      cm_insert(H.cm, H.cm_width, H.cm_k, key, dpos + dneg);
    }
    grid.sync();
    for (size_t i = gtid; ok && i < region; i += gsz) {
      const uint64_t key = P.in_keys[in0 + i];
      if (key == kEmptyKey) continue;
      if (cm_query(H.cm, H.cm_width, H.cm_k, key, 0xFFFFFFFFu) <= H.tail_freq) continue;
      uint32_t slot = __ldcg(P.in_slot + in0 + i);
      if (slot >= kAbsent) {
        float w;
        slot = shard_find_or_insert(P.tab, P.tab_mask, P.tab_shift, key, P.max_probe, &w, &acc.dins);
        if (slot == kAbsent) { set_status(L.status, kShardTableFull, 0, 0); continue; }
      }
      float g; uint32_t dpos, dneg;
      load_acc<true>(abase, lt0 + i, peer, &g, &dpos, &dneg);
      apply_slot(P.tab, slot, g, dpos, dneg, H, acc);
    }
    grid.sync();
  }
}

// ------------------------------------------------------------ fused kernels
// 8 blocks of 256 threads per SM (32 registers per thread): the phases of this kernel are bound by
// memory latency and speed up with every resident warp.
constexpr int kPullBlocksPerSM = 8;
constexpr uint32_t kPullInsert = 1u;   // flags: create missing keys in the shard

__global__ void __launch_bounds__(256, kPullBlocksPerSM)
ftrl_pull_spmv_kernel(FtrlPeers P, Minibatch M, LocalScratch L, uint32_t seq, uint32_t flags) {
  cg::grid_group grid = cg::this_grid();
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gsz = (size_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int world = P.seps.world;
  __shared__ int sh_ok;

  if (gtid == 0) L.stats[1] += (double)M.rows;
  PSB_TRACE(L, gtid, 0);
  phase_localize(P, M, L, gtid, gsz);
  if (world > 1) __threadfence_system();   // the table must be visible to its owners before the flag is
  grid.sync();
  PSB_TRACE(L, gtid, 1);
  // this worker's table is complete: tell every owner, then serve the other workers' tables
  if (blockIdx.x == 0 && threadIdx.x < world && world > 1) {
    __threadfence_system();
    st_release_sys_u64(P.ready[threadIdx.x] + P.rank, (uint64_t)seq << 32);
  }
  phase_lookup(P, L, seq, (flags & kPullInsert) != 0u, &sh_ok);
  if (world > 1) __threadfence_system();   // the weights must be visible to their workers before the flag is
  grid.sync();
  if (blockIdx.x == 0 && threadIdx.x < world && world > 1)
    st_release_sys_u64(P.replied[threadIdx.x] + P.rank, (uint64_t)seq << 32);
  // every owner must have answered before the rows are multiplied
  if (world > 1) {
    __syncthreads();
    if (threadIdx.x < world && threadIdx.x != P.rank) {
      bool ok;
      wait_epoch_ge(P.replied[P.rank] + threadIdx.x, seq, P.timeout_ns, &ok);
      if (!ok) set_status(L.status, kWaitTimeout, threadIdx.x, 3);
    }
    __syncthreads();
  }
  PSB_TRACE(L, gtid, 2);
  phase_spmv_loss(M, L, gtid >> 5, gsz >> 5, lane);
  PSB_TRACE(L, gtid, 3);
}

// 6 blocks per SM (42 registers): measured best; 3 blocks (69 registers, no cap) and 8 blocks
// (32 registers, spills) are both about 4 % slower per step.
constexpr int kPushBlocksPerSM = 6;
template <bool kCounts>
__global__ void __launch_bounds__(256, kPushBlocksPerSM)
ftrl_push_update_kernel(FtrlPeers P, Minibatch M, LocalScratch L, FtrlHyper H, uint32_t seq) {
  cg::grid_group grid = cg::this_grid();
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gsz = (size_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int world = P.seps.world;

  __shared__ HotCache hot;
  __shared__ int sh_ok;
  PSB_TRACE(L, gtid, 4);
  phase_grad<kCounts>(M, L, gtid >> 5, gsz >> 5, lane, &hot);
  if (world > 1) __threadfence_system();   // the accumulators must be visible to their owners before the flag is
  grid.sync();
  PSB_TRACE(L, gtid, 5);
  if (blockIdx.x == 0 && threadIdx.x < world && world > 1)
    st_release_sys_u64(P.grads[threadIdx.x] + P.rank, (uint64_t)seq << 32);
  phase_reset_tables<kCounts>(L, gtid, gsz);
  PSB_TRACE(L, gtid, 6);
  {
    ApplyAcc acc;
    if (kCounts && tail_filter_on(H)) {
      phase_apply_filtered(grid, P, L, H, seq, acc, &sh_ok);
    } else {
      phase_apply_chunks<kCounts>(P, L, H, seq, acc, &sh_ok);
    }
    apply_flush(acc, L.stats);
  }
  PSB_TRACE(L, gtid, 8);
}

// ------------------------------------------------- stand-alone phase kernels
// (the unfused baseline: same arithmetic, records packed by owner and exchanged with all_to_all)
__global__ void k_localize(FtrlPeers P, Minibatch M, LocalScratch L) {
  phase_localize(P, M, L, (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
}
__global__ void k_spmv_loss(Minibatch M, LocalScratch L) {
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gtid == 0) L.stats[1] += (double)M.rows;
  phase_spmv_loss(M, L, gtid >> 5, ((size_t)gridDim.x * blockDim.x) >> 5, threadIdx.x & 31);
}
__global__ void k_grad(Minibatch M, LocalScratch L) {
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  __shared__ HotCache hot;
  phase_grad<true>(M, L, gtid >> 5, ((size_t)gridDim.x * blockDim.x) >> 5, threadIdx.x & 31, &hot);
}
// count unique keys per owner (pass 1 of packing for all_to_all_v)
__global__ void k_count_owner(KeySeps seps, LocalScratch L, uint32_t* counts) {
  const size_t gsz = (size_t)gridDim.x * blockDim.x;
  uint32_t c[PSB_MAX_RANKS] = {0};
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s < L.lt_slots; s += gsz) {
    const uint64_t key = L.lt_keys[s];
    if (key != kEmptyKey) {
      const int o = route_owner(seps, key);
#pragma unroll
      for (int t = 0; t < PSB_MAX_RANKS; ++t) c[t] += (o == t);
    }
  }
#pragma unroll
  for (int t = 0; t < PSB_MAX_RANKS; ++t) {
    const uint32_t v = __reduce_add_sync(0xffffffffu, c[t]);
    if ((threadIdx.x & 31) == 0 && v) atomicAdd(counts + t, v);
  }
}
// pass 2: write (key, slot) grouped by owner; cursors[] start at the segment bases
__global__ void k_pack_keys(KeySeps seps, LocalScratch L, uint32_t* cursors, uint64_t* out_keys,
                            uint32_t* out_slot) {
  const size_t gsz = (size_t)gridDim.x * blockDim.x;
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s < L.lt_slots; s += gsz) {
    const uint64_t key = L.lt_keys[s];
    if (key != kEmptyKey) {
      const int o = route_owner(seps, key);
      const unsigned m = __match_any_sync(__activemask(), o);
      const int leader = __ffs(m) - 1, lane = threadIdx.x & 31;
      uint32_t base = 0;
      if (lane == leader) base = atomicAdd(cursors + o, (uint32_t)__popc(m));
      base = __shfl_sync(m, base, leader);
      const uint32_t at = base + __popc(m & ((1u << lane) - 1u));
      out_keys[at] = key;
      out_slot[at] = (uint32_t)s;
    }
  }
}
// owner side of an unfused pull: w for each requested key (0 when absent)
__global__ void k_lookup(const ShardSlot* tab, uint64_t mask, uint32_t shift, int max_probe,
                         const uint64_t* keys, uint32_t n, float* out_w) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float w;
    shard_find(tab, mask, shift, keys[i], max_probe, &w);
    out_w[i] = w;
  }
}
__global__ void k_scatter_w(const uint32_t* slots, const float* w, uint32_t n, LocalScratch L) {
  AccSlot* acc = reinterpret_cast<AccSlot*>(L.lt_acc) + (size_t)L.parity * L.lt_slots;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t s = slots[i];
    L.lt_w[s] = w[i];
    AccSlot z;
    z.g = 0.f; z.pos = 0.f; z.neg = 0.f; z.pad = 0.f;
    acc[s] = z;
  }
}
__global__ void k_pack_push(const uint32_t* slots, uint32_t n, LocalScratch L, float* out_g, uint64_t* out_cnt) {
  const AccSlot* acc = reinterpret_cast<const AccSlot*>(L.lt_acc) + (size_t)L.parity * L.lt_slots;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t s = slots[i];
    out_g[i] = acc[s].g;
    out_cnt[i] = ((uint64_t)(uint32_t)acc[s].pos << 32) | (uint64_t)(uint32_t)acc[s].neg;
    L.lt_keys[s] = kEmptyKey;
  }
}
__global__ void k_sketch_insert(const uint64_t* rk, const uint64_t* rc, uint32_t n, FtrlHyper h) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t key = __ldcg(rk + i);
    if (key == kEmptyKey) continue;
    const uint64_t c = __ldcg(rc + i);
    cm_insert(h.cm, h.cm_width, h.cm_k, key, (uint32_t)(c >> 32) + (uint32_t)c);
  }
}
// one flat record list of one sender: find or create every key, apply the update
__global__ void k_apply(ShardSlot* tab, uint64_t mask, uint32_t shift, int max_probe, const uint64_t* rk,
                        const float* rg, const uint64_t* rc, uint32_t n, FtrlHyper h, double* stats,
                        uint32_t* status) {
  ApplyAcc acc;
  const bool filter = tail_filter_on(h);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint64_t key = __ldcg(rk + i);
    if (key == kEmptyKey) continue;
    if (filter && cm_query(h.cm, h.cm_width, h.cm_k, key, 0xFFFFFFFFu) <= h.tail_freq) continue;
    float w;
    const uint32_t slot = shard_find_or_insert(tab, mask, shift, key, max_probe, &w, &acc.dins);
    if (slot == kAbsent) { set_status(status, kShardTableFull, 0, 0); continue; }
    const uint64_t c = __ldcg(rc + i);
    apply_slot(tab, slot, __ldcg(rg + i), (uint32_t)(c >> 32), (uint32_t)c, h, acc);
  }
  apply_flush(acc, stats);
}
__global__ void k_clear_local(LocalScratch L) {
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s < L.lt_slots; s += (size_t)gridDim.x * blockDim.x)
    L.lt_keys[s] = kEmptyKey;
}
// dump the non-zero weights of a shard: out_keys/out_w sized by capacity, *count receives the number
__global__ void k_dump_nonzero(const ShardSlot* tab, uint64_t mask, uint64_t* out_keys,
                               float* out_w, unsigned long long* count) {
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s <= mask; s += (size_t)gridDim.x * blockDim.x) {
    const uint64_t k = tab[s].key;
    if (k != kEmptyKey && tab[s].w != 0.f) {
      const unsigned long long at = atomicAdd(count, 1ull);
      out_keys[at] = k;
      out_w[at] = tab[s].w;
    }
  }
}
// Move every entry of a shard into a larger table (same hash, more top bits): the table grows
// like the reference's unordered_map (src/linear_method/ftrl_model.h:57) instead of filling up.
__global__ void k_rehash(const ShardSlot* from, uint64_t from_mask, ShardSlot* to, uint64_t to_mask, uint32_t to_shift,
                         int max_probe, uint32_t* status) {
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s <= from_mask; s += (size_t)gridDim.x * blockDim.x) {
    const ShardSlot e = from[s];
    if (e.key == kEmptyKey) continue;
    float w;
    int ins = 0;
    const uint32_t slot = shard_find_or_insert(to, to_mask, to_shift, e.key, max_probe, &w, &ins);
    if (slot == kAbsent) { set_status(status, kShardTableFull, 0, 1); continue; }
    *reinterpret_cast<float2*>(&to[slot].w) = make_float2(e.w, e.z);
    *reinterpret_cast<uint2*>(&to[slot].pos) = make_uint2(e.pos, e.neg);
  }
}

}  // namespace psb

// ------------------------------------------------------------------ C ABI
using namespace psb;

namespace {
int g_coop_blocks_pull[16] = {0}, g_coop_blocks_push[2][16] = {{0}};

template <typename K>
int coop_grid(K kernel, int* cache) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (cache[dev] == 0) {
    int per_sm = 0, sms = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (per_sm > 8) per_sm = 8;
    cache[dev] = per_sm * sms;
  }
  return cache[dev];
}
inline int flat_grid(size_t n, int cap = 148 * 8) {
  size_t b = (n + 255) / 256;
  if (b < 1) b = 1;
  if (b > (size_t)cap) b = cap;
  return (int)b;
}
}  // namespace

extern "C" {

// flags bit 0: create missing keys in the shard (a training step; off for predictions)
int psb_ftrl_pull_spmv(const FtrlPeers* P, const Minibatch* M, const LocalScratch* L, uint32_t seq, uint32_t flags,
                       cudaStream_t stream) {
  if (L->lt_w == nullptr || L->lt_acc == nullptr || P->in_slot == nullptr) return (int)cudaErrorInvalidValue;
  const int grid = coop_grid(ftrl_pull_spmv_kernel, g_coop_blocks_pull);
  if (grid <= 0) return (int)cudaErrorLaunchFailure;
  FtrlPeers p = *P; Minibatch m = *M; LocalScratch l = *L;
  void* args[] = {&p, &m, &l, &seq, &flags};
  return (int)cudaLaunchCooperativeKernel((void*)ftrl_pull_spmv_kernel, dim3(grid), dim3(256), args, 0, stream);
}

int psb_ftrl_push_update(const FtrlPeers* P, const Minibatch* M, const LocalScratch* L, const FtrlHyper* H,
                         uint32_t seq, cudaStream_t stream) {
  const bool soa = L->soa != 0;
  const bool filter = H->tail_freq != 0u && H->cm != nullptr;
  // the count-based rule and the tail filter need the pos/neg counts that the one-float accumulators do not carry
  if (soa && (H->rule == 0 || filter)) return (int)cudaErrorInvalidValue;
  if (filter && P->in_keys == nullptr) return (int)cudaErrorInvalidValue;
  void* kernel = soa ? (void*)ftrl_push_update_kernel<false> : (void*)ftrl_push_update_kernel<true>;
  const int grid = soa ? coop_grid(ftrl_push_update_kernel<false>, g_coop_blocks_push[0])
                       : coop_grid(ftrl_push_update_kernel<true>, g_coop_blocks_push[1]);
  if (grid <= 0) return (int)cudaErrorLaunchFailure;
  FtrlPeers p = *P; Minibatch m = *M; LocalScratch l = *L; FtrlHyper h = *H;
  void* args[] = {&p, &m, &l, &h, &seq};
  return (int)cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(256), args, 0, stream);
}

int psb_ftrl_localize(const FtrlPeers* P, const Minibatch* M, const LocalScratch* L, cudaStream_t s) {
  k_localize<<<flat_grid(M->nnz), 256, 0, s>>>(*P, *M, *L);
  return (int)cudaGetLastError();
}
int psb_ftrl_spmv_loss(const Minibatch* M, const LocalScratch* L, cudaStream_t s) {
  k_spmv_loss<<<flat_grid((size_t)M->rows * 32), 256, 0, s>>>(*M, *L);
  return (int)cudaGetLastError();
}
int psb_ftrl_grad(const Minibatch* M, const LocalScratch* L, cudaStream_t s) {
  k_grad<<<flat_grid((size_t)M->rows * 32), 256, 0, s>>>(*M, *L);
  return (int)cudaGetLastError();
}
int psb_ftrl_count_owner(const KeySeps* seps, const LocalScratch* L, uint32_t* counts, cudaStream_t s) {
  k_count_owner<<<flat_grid(L->lt_slots), 256, 0, s>>>(*seps, *L, counts);
  return (int)cudaGetLastError();
}
int psb_ftrl_pack_keys(const KeySeps* seps, const LocalScratch* L, uint32_t* cursors, uint64_t* out_keys,
                       uint32_t* out_slot, cudaStream_t s) {
  k_pack_keys<<<flat_grid(L->lt_slots), 256, 0, s>>>(*seps, *L, cursors, out_keys, out_slot);
  return (int)cudaGetLastError();
}
int psb_ftrl_lookup(const void* tab, uint64_t mask, uint32_t shift, int max_probe, const uint64_t* keys,
                    uint32_t n, float* out_w, cudaStream_t s) {
  k_lookup<<<flat_grid(n), 256, 0, s>>>((const ShardSlot*)tab, mask, shift, max_probe, keys, n, out_w);
  return (int)cudaGetLastError();
}
int psb_ftrl_scatter_w(const uint32_t* slots, const float* w, uint32_t n, const LocalScratch* L, cudaStream_t s) {
  k_scatter_w<<<flat_grid(n), 256, 0, s>>>(slots, w, n, *L);
  return (int)cudaGetLastError();
}
int psb_ftrl_pack_push(const uint32_t* slots, uint32_t n, const LocalScratch* L, float* out_g, uint64_t* out_cnt,
                       cudaStream_t s) {
  k_pack_push<<<flat_grid(n), 256, 0, s>>>(slots, n, *L, out_g, out_cnt);
  return (int)cudaGetLastError();
}
int psb_ftrl_apply(void* tab, uint64_t mask, uint32_t shift, int max_probe, const uint64_t* rk, const float* rg,
                   const uint64_t* rc, uint32_t n, const FtrlHyper* h, double* stats, uint32_t* status,
                   cudaStream_t s) {
  if (h->tail_freq != 0u && h->cm != nullptr) k_sketch_insert<<<flat_grid(n), 256, 0, s>>>(rk, rc, n, *h);
  k_apply<<<flat_grid(n), 256, 0, s>>>((ShardSlot*)tab, mask, shift, max_probe, rk, rg, rc, n, *h, stats, status);
  return (int)cudaGetLastError();
}
int psb_ftrl_clear_local(const LocalScratch* L, cudaStream_t s) {
  k_clear_local<<<flat_grid(L->lt_slots), 256, 0, s>>>(*L);
  return (int)cudaGetLastError();
}
int psb_ftrl_dump_nonzero(const void* tab, uint64_t mask, uint64_t* out_keys, float* out_w,
                          unsigned long long* count, cudaStream_t s) {
  k_dump_nonzero<<<flat_grid(mask + 1), 256, 0, s>>>((const ShardSlot*)tab, mask, out_keys, out_w, count);
  return (int)cudaGetLastError();
}
int psb_ftrl_rehash(const void* from, uint64_t from_mask, void* to, uint64_t to_mask, uint32_t to_shift, int max_probe,
                    uint32_t* status, cudaStream_t s) {
  k_rehash<<<flat_grid(from_mask + 1), 256, 0, s>>>((const ShardSlot*)from, from_mask, (ShardSlot*)to, to_mask, to_shift,
                                                     max_probe, status);
  return (int)cudaGetLastError();
}

}  // extern "C"
