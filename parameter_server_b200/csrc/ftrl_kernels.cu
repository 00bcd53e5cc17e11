// Online FTRL-proximal on key-range sharded device hash tables: the two fused
// communication+compute kernels of the product path, plus the same phases as
// stand-alone kernels for the unfused NCCL baseline.
//
// One rank = one GPU = worker r (streams minibatches) + server r (owns the keys
// of [sep[r], sep[r+1]) in an open-addressing table {key -> w, z, pos, neg}).
//
//   ftrl_pull_spmv  : de-duplicate the minibatch's keys into an L2-resident local
//                     table, gather each unique key's weight straight from the
//                     owner shard's table with peer loads over NVLink, then run
//                     the CSR SpMV X·w, the logistic loss and the per-row
//                     coefficient −y/(1+e^{y·Xw}) — one cooperative kernel.
//   ftrl_push_update: Xᵀ·coef and the pos/neg row counts per unique key, routed by
//                     key range into the owner's per-sender inbox with peer
//                     stores, a release flag per (sender, owner), and — on
//                     arrival of all senders — the owner-side FTRL update applied
//                     sender by sender, then an "applied" notification to every
//                     peer — one cooperative kernel.
//
// The arithmetic is the reference's server rule FTRLModel::setValue
// (src/linear_method/ftrl_model.h:81-112), the worker gradient of LogitLoss
// (src/linear_method/loss.h:73-88) and FTRL::countKeys
// (src/linear_method/ftrl.cc:154-174); the message flow replaces
// SharedParameter::push/pull (src/parameter/shared_parameter.h:14-26,90-149).
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

// One slot of an owner's table: 32 bytes = one DRAM/NVLink sector.  Key and weight sit in
// the same 16 bytes, so a pull probe is ONE 16-byte peer load; an update is a
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

struct FtrlPeers {
  KeySeps seps;
  int rank;
  int max_probe;
  uint64_t tab_mask;                       // table capacity − 1 (same on all ranks)
  ShardSlot* tab[PSB_MAX_RANKS];
  uint64_t* in_keys[PSB_MAX_RANKS];        // owner o: [sender][in_cap]
  float* in_g[PSB_MAX_RANKS];
  uint64_t* in_cnt[PSB_MAX_RANKS];         // pos<<32 | neg
  uint64_t* in_flag[PSB_MAX_RANKS];        // owner o: [sender] = epoch<<32 | count
  uint64_t* applied[PSB_MAX_RANKS];        // rank r: [owner] = epoch<<32
  uint64_t timeout_ns;
  uint32_t in_cap;
  uint32_t tab_shift;                      // 64 − log2(table capacity): slot = mix64(key) >> tab_shift
  uint32_t* in_chunk[PSB_MAX_RANKS];       // owner o: [sender][nchunks] records in every chunk segment of the inbox
  uint32_t nchunks;                        // chunks of kChunkSlots slots in a per-minibatch table (same on all ranks)
  uint32_t pad;
};

// The per-minibatch table is cut into aligned chunks of kChunkSlots slots; probing never leaves a
// chunk.  All ranks hash with the same function into tables of the same size, so chunk c holds the
// same range of hash values on every rank, and hence of every owner's shard table.  The records
// that sender s routes to owner o from its chunk c go to a FIXED segment of o's inbox:
//   [s · in_cap + c · kChunkSlots, … + in_chunk[o][s · nchunks + c])
// (in_cap = table capacity, so the segments tile the inbox exactly).  No cursor atomics on the
// sending side, and on the owner one thread block can apply chunk c of sender 0, 1, … in order
// with block-level barriers only: no other block ever touches the keys of that hash range.
constexpr int kChunkSlots = 1024;

struct Minibatch {
  const int64_t* offsets;  // rows+1
  const uint64_t* keys;    // nnz global keys
  const float* vals;       // nnz values or nullptr (binary features)
  const float* y;          // rows, ±1
  int64_t nnz;
  int rows;
  int pad;
};

struct __align__(16) LocalSlot {  // 16 B payload of one local dedup-table slot
  float w;    // pulled weight
  float g;    // gradient accumulator
  float pos;  // #positive rows containing the key (exact in fp32: a minibatch has < 2^24 rows)
  float neg;  // #negative rows containing the key
};

// One 16-byte vector reduction per non-zero instead of separate atomics on g and counts.
__device__ __forceinline__ void red_add_slot(LocalSlot* p, float g, float pos, float neg) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(0.f), "f"(g), "f"(pos), "f"(neg) : "memory");
}

struct LocalScratch {
  uint64_t* lt_keys;   // per-minibatch dedup table (all kEmptyKey between steps)
  LocalSlot* lt_val;   // payload per slot (one 16-byte sector: w, g, counts)
  uint64_t lt_mask;
  uint64_t lt_shift;   // 64 − log2(local capacity): slot = mix64(key) >> lt_shift
  uint32_t* slot_of;   // nnz: local slot of each non-zero
  float* coef;         // rows: −y/(1+e^{y·Xw})
  float* xw;           // rows: X·w (predictions)
  uint32_t* send_cnt;  // [PSB_MAX_RANKS] scratch of the unfused baseline (the fused push uses fixed chunk segments)
  uint32_t* recv_cnt;  // [PSB_MAX_RANKS] 1 = sender s's records of this step arrived, 0 = its flag wait ran out
  double* stats;       // [0] Σloss [1] rows [2] ‖w‖₁ [3] ‖w‖₂² [4] nnz(w) [5] unique keys [6] table entries
  uint32_t* status;    // StatusCode etc.
  uint64_t* trace;     // optional [16]: globaltimer at phase boundaries of the last step (see kTrace*)
  // Split layout for update rules that need no pos/neg counts (soa != 0): the pulled weight and
  // the gradient accumulator live in two 4-byte arrays, a quarter of the footprint of lt_val, so
  // the random accesses of the SpMV and of the gradient scatter stay inside L2.  The gather
  // phase writes lt_w and resets lt_g for every key of the minibatch.
  float* lt_w;
  float* lt_g;
  uint32_t soa;
  uint32_t pad;
};

// Streams (keys, slot map, inbox records) are read or written once per phase; with
// PSB_L2_HINTS they carry an evict-first L2 policy so that the hash tables stay resident.
#ifndef PSB_L2_HINTS
#define PSB_L2_HINTS 1
#endif
#if PSB_L2_HINTS
#define PSB_STREAM_POLICY(pol) const uint64_t pol = l2_evict_first_policy()
#define PSB_LD_U64(p, pol) ld_stream_u64((p), (pol))
#define PSB_LD_U32(p, pol) ld_stream_u32((p), (pol))
#define PSB_LD_F32(p, pol) ld_stream_f32((p), (pol))
#define PSB_ST_U32(p, v, pol) st_stream_u32((p), (v), (pol))
#else
#define PSB_STREAM_POLICY(pol) const uint64_t pol = 0; (void)pol
#define PSB_LD_U64(p, pol) (*(p))
#define PSB_LD_U32(p, pol) (*(p))
#define PSB_LD_F32(p, pol) (*(p))
#define PSB_ST_U32(p, v, pol) (*(p) = (v))
#endif

// trace slots: pull kernel 0 start, 1 localized, 2 gathered, 3 block-0 end;
//              push kernel 4 start, 5 gradients done, 6 records sent, 7 all senders arrived, 8 applied
#define PSB_TRACE(L, gtid, i) do { if ((L).trace != nullptr && (gtid) == 0) (L).trace[i] = globaltimer_ns(); } while (0)

constexpr uint32_t kBadSlot = 0xFFFFFFFFu;

// Both tables index with the TOP bits of the same 64-bit hash.  A scan of the local table in
// slot order therefore visits keys in (nearly) increasing shard-slot order, so the gather and
// the owner-side update walk the big shard table monotonically instead of at random.
__device__ __forceinline__ uint64_t shard_hash(uint64_t key, uint32_t shift) { return mix64(key) >> shift; }

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

__device__ __forceinline__ void phase_localize(const Minibatch& M, const LocalScratch& L, int max_probe,
                                               size_t gtid, size_t gsz) {
  PSB_STREAM_POLICY(pol);
  const int64_t step = (int64_t)gsz;
  const uint64_t cmask = L.lt_mask < (uint64_t)(kChunkSlots - 1) ? L.lt_mask : (uint64_t)(kChunkSlots - 1);
  int64_t i = (int64_t)gtid;
  if (i >= M.nnz) return;
  uint64_t key0 = PSB_LD_U64(M.keys + i, pol);
  uint64_t key1 = i + step < M.nnz ? PSB_LD_U64(M.keys + i + step, pol) : kEmptyKey;
  uint64_t h0 = (mix64(key0) >> L.lt_shift) & L.lt_mask;
  uint64_t cur0 = ld_table_u64(L.lt_keys + h0);
  for (; i < M.nnz; i += step) {
    uint64_t key2 = kEmptyKey, h1 = 0, cur1 = 0;
    if (i + 2 * step < M.nnz) key2 = PSB_LD_U64(M.keys + i + 2 * step, pol);
    if (i + step < M.nnz) {
      h1 = (mix64(key1) >> L.lt_shift) & L.lt_mask;
      cur1 = ld_table_u64(L.lt_keys + h1);
    }
    uint32_t slot = (uint32_t)h0;
    if (cur0 != key0) {
      const uint64_t s = table_find_or_insert(L.lt_keys, L.lt_mask, cmask, h0, key0, max_probe);
      if (s == ~0ull) {
        set_status(L.status, kLocalTableFull, 0, 0);
        slot = kBadSlot;
      } else {
        slot = (uint32_t)s;
      }
    }
    PSB_ST_U32(L.slot_of + i, slot, pol);
    key0 = key1; h0 = h1; cur0 = cur1; key1 = key2;
  }
}

// weight of `key` in owner's table (peer memory), 0 when absent; one 16-byte load per probe
// (`peer` = the table is another GPU's: system scope; this GPU's own shard is read at GPU scope)
__device__ __forceinline__ float probe_weight(const ShardSlot* tab, uint64_t mask, uint32_t shift, uint64_t key,
                                              int max_probe, bool peer = true) {
  uint64_t slot = shard_hash(key, shift) & mask;
  for (int i = 0; i < max_probe; ++i) {
    uint64_t k, wz;
    if (peer)
      asm volatile("ld.relaxed.sys.global.v2.u64 {%0, %1}, [%2];" : "=l"(k), "=l"(wz) : "l"(tab + slot) : "memory");
    else
      asm volatile("ld.relaxed.gpu.global.v2.u64 {%0, %1}, [%2];" : "=l"(k), "=l"(wz) : "l"(tab + slot) : "memory");
    if (k == key) return __uint_as_float((uint32_t)wz);
    if (k == kEmptyKey) return 0.f;
    slot = (slot + 1) & mask;
  }
  return 0.f;
}

template <bool kCounts>
__device__ __forceinline__ void phase_gather(const FtrlPeers& P, const LocalScratch& L, size_t gtid,
                                             size_t gsz) {
  uint32_t uniq = 0;
  for (uint64_t s = gtid; s <= L.lt_mask; s += gsz) {
    const uint64_t key = __ldcg(L.lt_keys + s);
    if (key != kEmptyKey) {
      const int o = route_owner(P.seps, key);
      const float w = probe_weight(P.tab[o], P.tab_mask, P.tab_shift, key, P.max_probe, o != P.rank);
      if (kCounts) {
        LocalSlot v;
        v.w = w;
        v.g = 0.f;
        v.pos = 0.f;
        v.neg = 0.f;
        *reinterpret_cast<float4*>(L.lt_val + s) = *reinterpret_cast<float4*>(&v);
      } else {
        L.lt_w[s] = w;
        L.lt_g[s] = 0.f;  // here, not after the read in the routing phase: a store there costs 70 us
      }
      ++uniq;
    }
  }
  uniq = __reduce_add_sync(0xffffffffu, uniq);
  if ((threadIdx.x & 31) == 0 && uniq) atomicAdd(&L.stats[5], (double)uniq);
}

// Rows are walked a warp at a time; a lane first issues the loads of up to kRowBatch of its
// non-zeros, then consumes them, so that several slot-map loads are in flight per lane.
#ifndef PSB_ROW_BATCH
#define PSB_ROW_BATCH 4
#endif
constexpr int kRowBatch = PSB_ROW_BATCH;

template <bool kCounts>
__device__ __forceinline__ void phase_spmv_loss(const Minibatch& M, const LocalScratch& L, size_t gwarp,
                                                size_t nwarps, int lane) {
  double loss = 0.0;
  PSB_STREAM_POLICY(pol);
  for (int64_t row = (int64_t)gwarp; row < M.rows; row += (int64_t)nwarps) {
    const int64_t b = M.offsets[row], e = M.offsets[row + 1];
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
        if (sl[k] != kBadSlot) s += x[k] * (kCounts ? L.lt_val[sl[k]].w : L.lt_w[sl[k]]);
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
#ifndef PSB_HOT_LOG2
#define PSB_HOT_LOG2 10
#endif
constexpr int kHotEntries = 1 << PSB_HOT_LOG2;
struct HotCache {
  uint32_t slot[kHotEntries];
  float g[kHotEntries];
  unsigned long long cnt[kHotEntries];
};

template <bool kCounts>
__device__ __forceinline__ void phase_grad(const Minibatch& M, const LocalScratch& L, size_t gwarp,
                                           size_t nwarps, int lane, HotCache* hc) {
  for (int i = threadIdx.x; i < kHotEntries; i += blockDim.x) {
    hc->slot[i] = kBadSlot;
    hc->g[i] = 0.f;
    if (kCounts) hc->cnt[i] = 0ull;
  }
  __syncthreads();
  PSB_STREAM_POLICY(pol);
  for (int64_t row = (int64_t)gwarp; row < M.rows; row += (int64_t)nwarps) {
    const int64_t b = M.offsets[row], e = M.offsets[row + 1];
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
        const int h = (int)((sl * 2654435761u) >> (32 - PSB_HOT_LOG2));  // top bits
        uint32_t cur = hc->slot[h];
        if (cur == kBadSlot) {
          const uint32_t prev = atomicCAS(&hc->slot[h], kBadSlot, sl);
          cur = prev == kBadSlot ? sl : prev;
        }
        if (cur == sl) {
          atomicAdd(&hc->g[h], gv);
          if (kCounts) atomicAdd(&hc->cnt[h], inc);
        } else if (kCounts) {
          red_add_slot(L.lt_val + sl, gv, is_pos ? 1.f : 0.f, is_pos ? 0.f : 1.f);
        } else {
          atomicAdd(L.lt_g + sl, gv);
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
        red_add_slot(L.lt_val + sl, hc->g[i], (float)(uint32_t)(c >> 32), (float)(uint32_t)c);
      } else {
        atomicAdd(L.lt_g + sl, hc->g[i]);
      }
    }
  }
}

// Scan the local table, write every unique key's record into its owner's inbox and empty the
// table for the next minibatch.  A block handles one chunk of kSendChunk slots per iteration.
// The records of a chunk are first grouped by owner in shared memory, then written out so that
// consecutive threads write consecutive inbox entries of one owner: the stores that cross NVLink
// are full, coalesced lines instead of scattered 8-byte pieces.  Chunk c always writes to the
// c-th segment of the sender's part of the inbox and leaves the number of records beside it.
constexpr int kSendItems = 4;
constexpr int kSendChunk = 256 * kSendItems;
static_assert(kSendChunk == kChunkSlots, "a block of 256 threads routes exactly one chunk per iteration");
struct SendStage {
  uint64_t key[kSendChunk];
  uint64_t cnt[kSendChunk];
  float g[kSendChunk];
  uint32_t count[PSB_MAX_RANKS];      // records per owner in this chunk
  uint32_t off[PSB_MAX_RANKS + 1];    // start of every owner's run in the staging arrays
  uint32_t base[PSB_MAX_RANKS];       // first inbox index granted to this chunk, per owner
};

template <bool kCounts>
__device__ __forceinline__ void phase_route_send(const FtrlPeers& P, const LocalScratch& L, SendStage* st) {
  const uint64_t n = L.lt_mask + 1;
  const uint64_t chunk = (uint64_t)blockDim.x * kSendItems;
  const int lane = threadIdx.x & 31;
  const int world = P.seps.world;
  for (uint64_t c0 = (uint64_t)blockIdx.x * chunk; c0 < n; c0 += (uint64_t)gridDim.x * chunk) {
    if (threadIdx.x < PSB_MAX_RANKS) st->count[threadIdx.x] = 0;
    __syncthreads();
    uint64_t key[kSendItems];
    uint32_t pos[kSendItems];
    int own[kSendItems];
#pragma unroll
    for (int k = 0; k < kSendItems; ++k) {
      const uint64_t s = c0 + (uint64_t)k * blockDim.x + threadIdx.x;
      key[k] = s < n ? __ldcg(L.lt_keys + s) : kEmptyKey;
      own[k] = key[k] != kEmptyKey ? route_owner(P.seps, key[k]) : -1;
      pos[k] = 0;
    }
#pragma unroll
    for (int k = 0; k < kSendItems; ++k) {
      for (int t = 0; t < world; ++t) {
        const unsigned m = __ballot_sync(0xffffffffu, own[k] == t);
        if (m == 0u) continue;
        const int leader = __ffs(m) - 1;
        uint32_t base = 0;
        if (lane == leader) base = atomicAdd(&st->count[t], (uint32_t)__popc(m));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (own[k] == t) pos[k] = base + __popc(m & ((1u << lane) - 1u));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t run = 0;
      for (int t = 0; t < world; ++t) { st->off[t] = run; run += st->count[t]; }
      st->off[world] = run;
    }
    // fixed segment of this chunk in every owner's inbox; its fill level goes next to it
    if (threadIdx.x < world) {
      st->base[threadIdx.x] = (uint32_t)c0;
      P.in_chunk[threadIdx.x][(size_t)P.rank * P.nchunks + (size_t)(c0 / chunk)] = st->count[threadIdx.x];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kSendItems; ++k) {
      if (own[k] < 0) continue;
      const uint64_t s = c0 + (uint64_t)k * blockDim.x + threadIdx.x;
      const uint32_t at = st->off[own[k]] + pos[k];
      st->key[at] = key[k];
      L.lt_keys[s] = kEmptyKey;
      if (kCounts) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(L.lt_val + s));
        st->g[at] = v.y;
        st->cnt[at] = ((uint64_t)(uint32_t)v.z << 32) | (uint64_t)(uint32_t)v.w;
      } else {
        st->g[at] = __ldcg(L.lt_g + s);
      }
    }
    __syncthreads();
    const uint32_t total = st->off[world];
    for (uint32_t i = threadIdx.x; i < total; i += blockDim.x) {
      int t = 0;
      while (t + 1 < world && i >= st->off[t + 1]) ++t;
      const uint32_t idx = st->base[t] + (i - st->off[t]);
      if (idx < P.in_cap) {
        const size_t at = (size_t)P.rank * P.in_cap + idx;
        P.in_keys[t][at] = st->key[i];
        P.in_g[t][at] = st->g[i];
        if (kCounts) P.in_cnt[t][at] = st->cnt[i];
      } else {
        set_status(L.status, kInboxOverflow, (uint32_t)t, idx);
      }
    }
    __syncthreads();
  }
  // the records must be visible to their owners before the flag is: system scope only when other GPUs
  // exist (a fence by one thread per block after the barrier measured the same: 48.4 vs 49.2 us at N=2)
  if (world > 1) __threadfence_system(); else __threadfence();
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

// first half of the tail-feature filter: add one sender's row counts to the owner's sketch
__device__ __forceinline__ void phase_sketch_insert(const uint64_t* rk, const uint64_t* rc, uint32_t n,
                                                    const FtrlHyper& h, size_t gtid, size_t gsz) {
  for (size_t i = gtid; i < n; i += gsz) {
    const uint64_t key = __ldcg(rk + i);
    if (key == kEmptyKey) continue;
    const uint64_t c = __ldcg(rc + i);
    cm_insert(h.cm, h.cm_width, h.cm_k, key, (uint32_t)(c >> 32) + (uint32_t)c);
  }
}

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

// apply records [0, n) of one sender; thread `tid` of `nthr` takes records tid, tid + nthr, …
template <bool kCounts>
__device__ __forceinline__ void apply_records(ShardSlot* tab, uint64_t mask, uint32_t shift, int max_probe,
                                              const uint64_t* rk, const float* rg, const uint64_t* rc,
                                              uint32_t n, const FtrlHyper& h, ApplyAcc& acc, uint32_t* status,
                                              size_t gtid, size_t gsz) {
  float dn1 = 0.f, dn2 = 0.f;
  int dnnz = 0, dins = 0;
  const bool filter = kCounts && tail_filter_on(h);
  for (size_t i = gtid; i < n; i += gsz) {
    const uint64_t key = __ldcg(rk + i);
    if (key == kEmptyKey) continue;
    if (filter && cm_query(h.cm, h.cm_width, h.cm_k, key, 0xFFFFFFFFu) <= h.tail_freq) continue;
    const float g = __ldcg(rg + i);
    const uint64_t c = kCounts ? __ldcg(rc + i) : 0ull;
    uint64_t slot = shard_hash(key, shift) & mask;
    bool found = false;
    for (int p = 0; p < max_probe; ++p) {
      const uint64_t cur = tab[slot].key;
      if (cur == key) { found = true; break; }
      if (cur == kEmptyKey) {
        const unsigned long long prev = atomicCAS(reinterpret_cast<unsigned long long*>(&tab[slot].key),
                                                  (unsigned long long)kEmptyKey, (unsigned long long)key);
        if (prev == kEmptyKey) { found = true; ++dins; break; }
        if (prev == key) { found = true; break; }
      }
      slot = (slot + 1) & mask;
    }
    if (!found) {
      set_status(status, kShardTableFull, 0, 0);
      continue;
    }
    const float2 wz = *reinterpret_cast<const float2*>(&tab[slot].w);
    const uint2 pn = *reinterpret_cast<const uint2*>(&tab[slot].pos);
    ShardState e;
    e.w = wz.x; e.z = wz.y; e.pos = pn.x; e.neg = pn.y;
    ftrl_update(e, g, (uint32_t)(c >> 32), (uint32_t)c, h, dn1, dn2, dnnz);
    *reinterpret_cast<float2*>(&tab[slot].w) = make_float2(e.w, e.z);
    *reinterpret_cast<uint2*>(&tab[slot].pos) = make_uint2(e.pos, e.neg);
  }
  acc.dn1 += dn1; acc.dn2 += dn2; acc.dnnz += dnnz; acc.dins += dins;
}

// stand-alone form: one flat record list (unfused baseline)
template <bool kCounts>
__device__ __forceinline__ void phase_apply(ShardSlot* tab, uint64_t mask, uint32_t shift, int max_probe,
                                            const uint64_t* rk, const float* rg, const uint64_t* rc,
                                            uint32_t n, const FtrlHyper& h, double* stats, uint32_t* status,
                                            size_t gtid, size_t gsz) {
  ApplyAcc acc;
  apply_records<kCounts>(tab, mask, shift, max_probe, rk, rg, rc, n, h, acc, status, gtid, gsz);
  apply_flush(acc, stats);
}

// ------------------------------------------------------------ fused kernels
// 8 blocks of 256 threads per SM (32 registers per thread): the phases of this kernel are bound by
// memory latency and speed up with every resident warp.
#ifndef PSB_PULL_MIN_BLOCKS
#define PSB_PULL_MIN_BLOCKS 8
#endif
template <bool kCounts>
__global__ void __launch_bounds__(256, PSB_PULL_MIN_BLOCKS)
ftrl_pull_spmv_kernel(FtrlPeers P, Minibatch M, LocalScratch L, uint32_t epoch) {
  cg::grid_group grid = cg::this_grid();
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gsz = (size_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;

  // every owner must have applied step epoch-1 before its table is read
  if (blockIdx.x == 0 && threadIdx.x < P.seps.world) {
    bool ok;
    wait_epoch_ge(P.applied[P.rank] + threadIdx.x, epoch - 1, P.timeout_ns, &ok);
    if (!ok) set_status(L.status, kWaitTimeout, threadIdx.x, 1);
  }
  if (gtid == 0) L.stats[1] += (double)M.rows;
  PSB_TRACE(L, gtid, 0);
  phase_localize(M, L, P.max_probe, gtid, gsz);
  grid.sync();
  PSB_TRACE(L, gtid, 1);
  phase_gather<kCounts>(P, L, gtid, gsz);
  grid.sync();
  PSB_TRACE(L, gtid, 2);
  phase_spmv_loss<kCounts>(M, L, gtid >> 5, gsz >> 5, lane);
  PSB_TRACE(L, gtid, 3);
}

// 6 blocks per SM (42 registers): measured best; 3 blocks (69 registers, no cap) and 8 blocks
// (32 registers, spills) are both about 4 % slower per step.
#ifndef PSB_PUSH_MIN_BLOCKS
#define PSB_PUSH_MIN_BLOCKS 6
#endif
template <bool kCounts>
__global__ void __launch_bounds__(256, PSB_PUSH_MIN_BLOCKS)
ftrl_push_update_kernel(FtrlPeers P, Minibatch M, LocalScratch L, FtrlHyper H, uint32_t epoch) {
  cg::grid_group grid = cg::this_grid();
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gsz = (size_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const int world = P.seps.world;

  // the hot-slot cache (gradient phase) and the send staging area (routing phase) are never live together
  __shared__ union PushSmem { HotCache hot; SendStage stage; } sm;
  PSB_TRACE(L, gtid, 4);
  phase_grad<kCounts>(M, L, gtid >> 5, gsz >> 5, lane, &sm.hot);
  grid.sync();
  PSB_TRACE(L, gtid, 5);
  phase_route_send<kCounts>(P, L, &sm.stage);
  grid.sync();
  PSB_TRACE(L, gtid, 6);
  // tell every owner that this sender's records and fill levels are in place, then wait for all senders
  if (blockIdx.x == 0 && threadIdx.x < world) {
    const int t = threadIdx.x;
    __threadfence_system();
    st_release_sys_u64(P.in_flag[t] + P.rank, (uint64_t)epoch << 32);
    bool ok;
    wait_epoch_ge(P.in_flag[P.rank] + t, epoch, P.timeout_ns, &ok);
    L.recv_cnt[t] = ok ? 1u : 0u;  // a sender that never arrived is skipped
    if (!ok) set_status(L.status, kWaitTimeout, t, 2);
  }
  grid.sync();
  PSB_TRACE(L, gtid, 7);
  // Apply sender by sender (the reference applies each worker's push separately).  The order only
  // matters per key, and a key lives in one chunk: a block takes chunk c and walks the senders'
  // segments of that chunk in rank order with block-level barriers.  With the tail filter on, a
  // sender's counts must all be in the sketch before any of its keys is queried, so that case keeps
  // grid-wide barriers around every sender.
  {
    ApplyAcc acc;
    ShardSlot* tab = P.tab[P.rank];
    const uint64_t* rk = P.in_keys[P.rank];
    const float* rg = P.in_g[P.rank];
    const uint64_t* rc = P.in_cnt[P.rank];
    const uint32_t* fill = P.in_chunk[P.rank];
    if (!(kCounts && tail_filter_on(H))) {
      for (uint32_t c = blockIdx.x; c < P.nchunks; c += gridDim.x) {
        for (int s = 0; s < world; ++s) {
          if (__ldcg(L.recv_cnt + s) == 0u) continue;
          const uint32_t n = min(__ldcg(fill + (size_t)s * P.nchunks + c), (uint32_t)kChunkSlots);
          const size_t off = (size_t)s * P.in_cap + (size_t)c * kChunkSlots;
          apply_records<kCounts>(tab, P.tab_mask, P.tab_shift, P.max_probe, rk + off, rg + off, rc + off, n, H, acc,
                                 L.status, threadIdx.x, blockDim.x);
          __syncthreads();
        }
      }
    } else {
      for (int s = 0; s < world; ++s) {
        const bool have = __ldcg(L.recv_cnt + s) != 0u;
        for (uint32_t c = blockIdx.x; have && c < P.nchunks; c += gridDim.x) {
          const uint32_t n = min(__ldcg(fill + (size_t)s * P.nchunks + c), (uint32_t)kChunkSlots);
          const size_t off = (size_t)s * P.in_cap + (size_t)c * kChunkSlots;
          phase_sketch_insert(rk + off, rc + off, n, H, threadIdx.x, blockDim.x);
        }
        grid.sync();
        for (uint32_t c = blockIdx.x; have && c < P.nchunks; c += gridDim.x) {
          const uint32_t n = min(__ldcg(fill + (size_t)s * P.nchunks + c), (uint32_t)kChunkSlots);
          const size_t off = (size_t)s * P.in_cap + (size_t)c * kChunkSlots;
          apply_records<kCounts>(tab, P.tab_mask, P.tab_shift, P.max_probe, rk + off, rg + off, rc + off, n, H, acc,
                                 L.status, threadIdx.x, blockDim.x);
        }
        grid.sync();
      }
    }
    apply_flush(acc, L.stats);
  }
  grid.sync();
  PSB_TRACE(L, gtid, 8);
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys_u64(P.applied[threadIdx.x] + P.rank, (uint64_t)epoch << 32);
  }
}

// ------------------------------------------------- stand-alone phase kernels
__global__ void k_localize(Minibatch M, LocalScratch L, int max_probe) {
  phase_localize(M, L, max_probe, (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
}
__global__ void k_spmv_loss(Minibatch M, LocalScratch L) {
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gtid == 0) L.stats[1] += (double)M.rows;
  phase_spmv_loss<true>(M, L, gtid >> 5, ((size_t)gridDim.x * blockDim.x) >> 5, threadIdx.x & 31);
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
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s <= L.lt_mask; s += gsz) {
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
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s <= L.lt_mask; s += gsz) {
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
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out_w[i] = probe_weight(tab, mask, shift, keys[i], max_probe, false);
}
__global__ void k_scatter_w(const uint32_t* slots, const float* w, uint32_t n, LocalScratch L) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t s = slots[i];
    LocalSlot v;
    v.w = w[i];
    v.g = 0.f;
    v.pos = 0.f;
    v.neg = 0.f;
    L.lt_val[s] = v;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) L.stats[5] += (double)n;
}
__global__ void k_pack_push(const uint32_t* slots, uint32_t n, LocalScratch L, float* out_g, uint64_t* out_cnt) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const uint32_t s = slots[i];
    out_g[i] = L.lt_val[s].g;
    out_cnt[i] = ((uint64_t)(uint32_t)L.lt_val[s].pos << 32) | (uint64_t)(uint32_t)L.lt_val[s].neg;
    L.lt_keys[s] = kEmptyKey;
  }
}
__global__ void k_apply(ShardSlot* tab, uint64_t mask, uint32_t shift, int max_probe, const uint64_t* rk,
                        const float* rg, const uint64_t* rc, uint32_t n, FtrlHyper h, double* stats,
                        uint32_t* status) {
  phase_apply<true>(tab, mask, shift, max_probe, rk, rg, rc, n, h, stats, status,
                    (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
}
__global__ void k_sketch_insert(const uint64_t* rk, const uint64_t* rc, uint32_t n, FtrlHyper h) {
  phase_sketch_insert(rk, rc, n, h, (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
}
__global__ void k_clear_local(LocalScratch L) {
  for (uint64_t s = (size_t)blockIdx.x * blockDim.x + threadIdx.x; s <= L.lt_mask; s += (size_t)gridDim.x * blockDim.x)
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

}  // namespace psb

// ------------------------------------------------------------------ C ABI
using namespace psb;

namespace {
int g_coop_blocks_pull[2][16] = {{0}}, g_coop_blocks_push[2][16] = {{0}};

template <typename K>
int coop_grid(K kernel, int* cache) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (cache[dev] == 0) {
    int per_sm = 0, sms = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, 256, 0);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int cap = 8;
    if (const char* e = getenv("PSB_FTRL_CTAS_PER_SM")) cap = atoi(e) > 0 ? atoi(e) : cap;
    if (per_sm > cap) per_sm = cap;
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

int psb_ftrl_pull_spmv(const FtrlPeers* P, const Minibatch* M, const LocalScratch* L, uint32_t epoch,
                       cudaStream_t stream) {
  const bool soa = L->soa != 0;
  if (soa && (L->lt_w == nullptr || L->lt_g == nullptr)) return (int)cudaErrorInvalidValue;
  void* kernel = soa ? (void*)ftrl_pull_spmv_kernel<false> : (void*)ftrl_pull_spmv_kernel<true>;
  const int grid = soa ? coop_grid(ftrl_pull_spmv_kernel<false>, g_coop_blocks_pull[0])
                       : coop_grid(ftrl_pull_spmv_kernel<true>, g_coop_blocks_pull[1]);
  if (grid <= 0) return (int)cudaErrorLaunchFailure;
  FtrlPeers p = *P; Minibatch m = *M; LocalScratch l = *L;
  void* args[] = {&p, &m, &l, &epoch};
  return (int)cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(256), args, 0, stream);
}

int psb_ftrl_push_update(const FtrlPeers* P, const Minibatch* M, const LocalScratch* L, const FtrlHyper* H,
                         uint32_t epoch, cudaStream_t stream) {
  const bool soa = L->soa != 0;
  // the count-based rule needs the pos/neg counts that the split layout does not carry
  if (soa && (H->rule == 0 || (H->tail_freq != 0u && H->cm != nullptr) || L->lt_w == nullptr || L->lt_g == nullptr))
    return (int)cudaErrorInvalidValue;
  void* kernel = soa ? (void*)ftrl_push_update_kernel<false> : (void*)ftrl_push_update_kernel<true>;
  const int grid = soa ? coop_grid(ftrl_push_update_kernel<false>, g_coop_blocks_push[0])
                       : coop_grid(ftrl_push_update_kernel<true>, g_coop_blocks_push[1]);
  if (grid <= 0) return (int)cudaErrorLaunchFailure;
  FtrlPeers p = *P; Minibatch m = *M; LocalScratch l = *L; FtrlHyper h = *H;
  void* args[] = {&p, &m, &l, &h, &epoch};
  return (int)cudaLaunchCooperativeKernel(kernel, dim3(grid), dim3(256), args, 0, stream);
}

int psb_ftrl_localize(const Minibatch* M, const LocalScratch* L, int max_probe, cudaStream_t s) {
  k_localize<<<flat_grid(M->nnz), 256, 0, s>>>(*M, *L, max_probe);
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
  k_count_owner<<<flat_grid(L->lt_mask + 1), 256, 0, s>>>(*seps, *L, counts);
  return (int)cudaGetLastError();
}
int psb_ftrl_pack_keys(const KeySeps* seps, const LocalScratch* L, uint32_t* cursors, uint64_t* out_keys,
                       uint32_t* out_slot, cudaStream_t s) {
  k_pack_keys<<<flat_grid(L->lt_mask + 1), 256, 0, s>>>(*seps, *L, cursors, out_keys, out_slot);
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
  k_clear_local<<<flat_grid(L->lt_mask + 1), 256, 0, s>>>(*L);
  return (int)cudaGetLastError();
}
int psb_ftrl_dump_nonzero(const void* tab, uint64_t mask, uint64_t* out_keys, float* out_w,
                          unsigned long long* count, cudaStream_t s) {
  k_dump_nonzero<<<flat_grid(mask + 1), 256, 0, s>>>((const ShardSlot*)tab, mask, out_keys, out_w, count);
  return (int)cudaGetLastError();
}

}  // extern "C"
