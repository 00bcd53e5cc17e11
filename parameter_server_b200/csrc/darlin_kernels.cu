// DARLIN: delayed block proximal-Newton coordinate descent for L1 logistic regression,
// as one persistent cooperative kernel per pass over the feature blocks.
//
// One rank = worker r (rows shard in CSC over its local unique keys) + server r (the
// weights of its key range).  For every feature block, in schedule order:
//
//   A  worker  G_j = −Σ y_i τ_i x_ij ,  U_j = Σ min(τ_i(1−τ_i)·e^{|x_ij|δ_j}, ¼)·x_ij²   (τ_i = 1/(1+e^{m_i}))
//              computed nnz-parallel with warp-segmented sums and pushed straight into the
//              owner shard's (G,U) accumulators with red.add.v2.f32 over NVLink
//      ── the rank's last CTA to finish adds 1 to each owner's arrival counter (release, system scope) ──
//   B  server  on arrival of all workers' CTAs: KKT filter, proximal-Newton step inside the
//              trust region δ, δ update — on the authoritative copy of w in the owner's shard
//   C  worker  in the SAME phase, on every rank: m_i += y_i·x_ij·Δw_j over the block's non-zeros, where
//              Δw_j is recomputed from the summed (G_j,U_j) (one 8-byte peer load from the owner) and the
//              worker's own copy of (w_j, δ_j, active_j).  The step is a pure function of those inputs and
//              is written with explicitly rounded operations, so every worker gets bit for bit the owner's
//              Δw: no second cross-GPU round ("weights updated") is needed.
//      ── one in-GPU barrier ──
//              The worker's copy of w, δ and the active set of these columns is brought up to date one
//              phase later, next to the gradients of the following block (other columns); the accumulators
//              rotate over three buffers and a block's slots are zeroed by the owner one block later, when
//              every rank has read them for the last time.
//   A block therefore costs ONE cross-GPU synchronisation and one in-GPU barrier.
//
// Arithmetic follows Darling::computeGradients / updateWeight / updateDual
// (src/linear_method/darling.cc:306-356, 437-477, 358-435).  Instead of
// dual_i = exp(y_i·Xw_i) the worker keeps the margin m_i = y_i·Xw_i (dual = e^m), so the
// multiplicative dual update becomes an additive, atomics-friendly one and fp32 does not
// drift.  Inactive (KKT-filtered) keys are NaN in the server's weight array, exactly the
// reference's sentinel convention.
//
// All waits (cross-GPU counters and the in-GPU barrier) are bounded; on expiry the kernel
// records the place in the status word, raises the abort flag and every CTA leaves the
// block loop.
#include <cstdlib>

#include "psb_common.cuh"

namespace psb {

struct DarlinWorker {
  const int64_t* col_ptr;   // cols+1 offsets into row_idx/vals (CSC over local columns)
  const uint32_t* row_idx;  // nnz
  const float* vals;        // nnz, or nullptr for binary features
  float2* ym;               // rows: {y_i (±1), margin m_i = y_i·(Xw)_i} — one 8-byte gather per non-zero
  const uint32_t* col_of;   // nnz: local column of every non-zero, or nullptr (then found by binary search)
  float* w;                 // cols: worker's copy of the weights
  float* delta;             // cols: trust region
  uint8_t* active;          // cols: 1 = in the active set
  const uint32_t* gslot;    // cols: slot in the owner's shard
  const uint8_t* gowner;    // cols: owner rank
  float* dw;                // cols: scratch Δw of the current block
  int64_t cols;
  int rows;
  int pad;
  const int64_t* gcol;      // cols: position of the column's key in the global sorted key list (all owners)
};

struct DarlinPeers {
  float* w[PSB_MAX_RANKS];        // owner shard weights (NaN = filtered)
  float2* gu[PSB_MAX_RANKS];      // owner shard (G,U) accumulators
  uint64_t* arrive[PSB_MAX_RANKS];   // on owner o: +1 per worker whose CTAs all finished phase A of a group
  int rank, world;
  uint64_t timeout_ns;
  int64_t gu_stride;                 // float2 elements between the three accumulator buffers of a shard
  // small groups of blocks (see kGatherCols): rank t's inbox of partial sums, [3 buffers][world senders][kGatherCols],
  // and this rank's own partial sums of the group in flight
  float2* part[PSB_MAX_RANKS];
  float2* mine;
  // very wide groups on several GPUs (see kListCols): per LOCAL column of rank r, its partial (G,U), its slot
  // in the owner's shard and the owner's answer Δw; and the second arrival counter of those groups
  float2* colgu[PSB_MAX_RANKS];
  const uint32_t* colslot[PSB_MAX_RANKS];
  float* coldw[PSB_MAX_RANKS];
  uint64_t* arrive2[PSB_MAX_RANKS];
};

struct DarlinServer {     // local arrays of this rank's shard
  float* delta;           // slots
  uint8_t* active;        // slots
  uint32_t* violation;    // float bits of max violation (non-negative)
  int64_t slots;
  float* d_slot;          // slots: Δw of the group in flight (NaN: key dropped), very wide groups only
};

struct DarlinSched {
  const int32_t* order;     // nblk block ids in pass order
  const int64_t* blk_lc;    // [nblocks_total][2] local column range of each block
  const int64_t* blk_sl;    // [nblocks_total][2] slot range of each block on this owner
  int nblk;
  int group;                // blocks per synchronisation group (max_block_delay + 1)
  uint64_t seq0;            // groups processed before this launch (same on all ranks)
  uint64_t* local_bar;      // [0] in-GPU barrier counter (monotone), [1] CTAs that finished a gradient phase,
                            // [3] barrier rounds completed so far (kept on the device: a launch runs one round
                            // per group plus one per wide group, which only the kernel counts)
  uint64_t bar0;            // unused (the round count lives in local_bar[3])
  uint32_t* abort_flag;
  uint32_t* status;
  // out-of-core mode: stage_base[q] = device address where the packed [row ids | values] of block
  // order[q] were copied; nullptr = the matrix is resident (Wk.row_idx / Wk.vals hold it all)
  const uint64_t* stage_base;
  // blocks of the group that ran last before this launch (its accumulators are still to be zeroed), or nullptr
  const int32_t* prev;
  int nprev;
  int wide_cols;            // groups with more local columns than this take phase C in two steps (0: kWideBlockCols)
  const int64_t* blk_gc;    // [nblocks_total][2] range of each block in the global sorted key list
  const int64_t* blk_gs0;   // [nblocks_total] position in that list of this owner's first slot of every block
  int gather;               // small groups exchange per-rank partial sums (needs part / mine / gcol / blk_gc)
  int pad2;
  // optional [12]: nanoseconds that thread block 0 spent, summed over the launch's groups, in
  // [0] commit + gradients, [1] arrival + cross-GPU wait, [2] sums + update + margins, [3] the in-GPU barrier;
  // of [2] for very wide groups on several GPUs: [4] owner sums the senders' columns, [5] owner update,
  // [6] answers written back, [7] second arrival + wait, [8] worker applies the answers, [9] margins
  uint64_t* trace;
  // very wide groups: on every rank and for every block, the first local column of every owner's share of the
  // block, so that an owner can address the senders' columns of its share
  const int64_t* all_cb;       // [world][nblocks_total][world + 1]
  int64_t nblocks_total;
  int64_t list_cols;           // groups with more columns over all owners than this take the list path (0: kListCols)
};

struct DarlinHyper {
  float lambda, eta, delta_max, kkt_threshold;
};

__device__ __forceinline__ uint64_t ld_acquire_gpu_u64(const uint64_t* p) {
  uint64_t v; asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void red_release_sys_add_u64(uint64_t* p, uint64_t v) {
  asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// single-rank forms of the push and of the weight load: same operations at GPU scope
__device__ __forceinline__ void red_add_v2_f32_gpu(float2* p, float a, float b) {
  asm volatile("red.relaxed.gpu.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ float ld_relaxed_gpu_f32(const float* p) {
  float v; asm volatile("ld.relaxed.gpu.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void red_add_v2_f32(float2* p, float a, float b) {
  asm volatile("red.relaxed.sys.global.add.v2.f32 [%0], {%1, %2};" ::"l"(p), "f"(a), "f"(b) : "memory");
}

// Cross-GPU arrival, two levels.  Every CTA first counts itself on a counter of its own GPU; the
// CTA that completes the count (G·seq) notifies every rank's counter once.  A rank's counter thus
// receives `world` remote increments per synchronisation point instead of world × G increments
// on one address, which the owner's L2 would serialise (G = 148 CTAs: > 1000 remote atomics).
// Ordering: the CTA's pushes → __syncthreads → fence.sys → acq_rel add (gpu scope) by thread 0;
// the last adder therefore observes all CTAs' pushes before its release.sys notifications.
// The notifications go out from `world` threads at once: a release at system scope waits for the
// thread's earlier remote writes, so one thread sending them one after the other would pay a
// round trip per rank.
__device__ __forceinline__ void cta_arrive_all(const DarlinPeers& P, uint64_t* const* ctrs, uint64_t* local_ctr,
                                               uint64_t local_target, bool* s_last) {
  // With a single rank nothing leaves the GPU and every fence, release and poll stays at GPU scope:
  // system-scope operations issued at every synchronisation point kept host-to-device copies that
  // ran beside the kernel from overlapping with it (out-of-core pass = copy time + kernel time).
  const bool multi = P.world > 1;
  __syncthreads();
  if (threadIdx.x == 0) {
    if (multi) __threadfence_system(); else __threadfence();
    unsigned long long prev;
    asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], %2;" : "=l"(prev) : "l"(local_ctr), "l"(1ull) : "memory");
    *s_last = prev + 1ull == local_target;
  }
  __syncthreads();
  if (*s_last && threadIdx.x < P.world) {
    uint64_t* ctr = ctrs[threadIdx.x];
    if (multi) {
      __threadfence_system();
      red_release_sys_add_u64(ctr, 1ull);
    } else {
      __threadfence();
      asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(ctr), "l"(1ull) : "memory");
    }
  }
}

// thread 0 of the CTA waits until *ctr >= target (bounded); result broadcast to the CTA
__device__ __forceinline__ bool cta_wait_counter(const uint64_t* ctr, uint64_t target, uint64_t timeout_ns,
                                                 bool sys_scope, bool* s_ok) {
  if (threadIdx.x == 0) {
    const uint64_t t0 = globaltimer_ns();
    const uint64_t max_iters = timeout_ns / 32 + 1024;
    bool ok = false;
    for (uint64_t it = 0; it < max_iters; ++it) {
      const uint64_t v = sys_scope ? ld_acquire_sys_u64(ctr) : ld_acquire_gpu_u64(ctr);
      if (v >= target) { ok = true; break; }
      if ((it & 63) == 63 && globaltimer_ns() - t0 > timeout_ns) break;
      __nanosleep(20);
    }
    *s_ok = ok;
  }
  __syncthreads();
  return *s_ok;
}

__device__ __forceinline__ int64_t find_col(const int64_t* col_ptr, int64_t lo, int64_t hi, int64_t e) {
  // largest j in [lo, hi) with col_ptr[j] <= e
  while (hi - lo > 1) {
    const int64_t mid = (lo + hi) >> 1;
    if (col_ptr[mid] <= e) lo = mid; else hi = mid;
  }
  return lo;
}

// Column of CSC position e when the lanes of a warp hold consecutive positions (e = base + lane) and no
// per-nnz column array is kept (out-of-core mode): one binary search per warp (lane 0, always valid), then
// every lane walks forward over the few column boundaries inside the warp's 32 positions.  A binary search
// per non-zero costs ~log2(columns of the block) dependent loads; with 485 k columns per block it made the
// streamed pass twice as slow as the resident one.  Must be called by all 32 lanes.
__device__ __forceinline__ int64_t find_col_warp(const int64_t* col_ptr, int64_t lo, int64_t hi, int64_t e, bool valid) {
  const int64_t e0 = __shfl_sync(0xffffffffu, e, 0);
  int64_t j = (threadIdx.x & 31) == 0 ? find_col(col_ptr, lo, hi, e0) : 0;
  j = __shfl_sync(0xffffffffu, j, 0);
  if (valid) {
    for (int steps = 0; j + 1 < hi && col_ptr[j + 1] <= e; ++j) {
      if (++steps > 48) { j = find_col(col_ptr, j, hi, e); break; }   // many empty columns: finish by bisection
    }
  }
  return j;
}

// Without the per-non-zero column array a warp takes one contiguous share of the block's positions instead of
// every nwarps-th group of 32, so that only its first group needs a bisection; every later group starts its
// walk at the column where the previous one ended (streamed pass of 10^6 rows x 120 non-zeros, 485 k columns
// per block: 14.2 ms against 19.2 ms with a bisection per group).
constexpr bool kRangeWalk = true;

// Share of warp `gwarp` of the positions [p0, p1): a multiple of 32 long, so only the last share is ragged.
__device__ __forceinline__ void warp_share(int64_t p0, int64_t p1, size_t gwarp, size_t nwarps, int64_t* b, int64_t* e) {
  const int64_t per = (((p1 - p0) + (int64_t)nwarps - 1) / (int64_t)nwarps + 31) & ~(int64_t)31;
  const int64_t lo = p0 + (int64_t)gwarp * per;
  *b = lo < p1 ? lo : p1;
  *e = *b + per < p1 ? *b + per : p1;
}

// find_col_warp with a starting point: `hint` is the column found for this warp's previous 32 positions
// (-1: none yet, bisect).  Must be called by all 32 lanes.
__device__ __forceinline__ int64_t find_col_from(const int64_t* col_ptr, int64_t lo, int64_t hi, int64_t hint, int64_t e,
                                                 bool valid) {
  const int64_t e0 = __shfl_sync(0xffffffffu, e, 0);
  int64_t j = 0;
  if ((threadIdx.x & 31) == 0) {
    if (hint < 0) {
      j = find_col(col_ptr, lo, hi, e0);
    } else {
      j = hint;
      for (int steps = 0; j + 1 < hi && col_ptr[j + 1] <= e0; ++j) {
        if (++steps > 48) { j = find_col(col_ptr, j, hi, e0); break; }
      }
    }
  }
  j = __shfl_sync(0xffffffffu, j, 0);
  if (valid) {
    for (int steps = 0; j + 1 < hi && col_ptr[j + 1] <= e; ++j) {
      if (++steps > 48) { j = find_col(col_ptr, j, hi, e); break; }
    }
  }
  return j;
}

// ---- phase A: block gradient (G,U) pushed into the owners' accumulators
__device__ __forceinline__ void darlin_grad_push(const DarlinWorker& Wk, const DarlinPeers& P, int64_t lc0,
                                                 int64_t lc1, int64_t p0, int64_t p1, int buf, float2* mine, int64_t bias,
                                                 size_t gwarp, size_t nwarps, int lane, bool by_local_column = false) {
  const int64_t boff = (int64_t)buf * P.gu_stride;
  const bool binary = Wk.vals == nullptr;
  const bool shares = kRangeWalk && Wk.col_of == nullptr;
  int64_t base = p0 + (int64_t)gwarp * 32, end = p1, step = (int64_t)nwarps * 32, hint = -1;
  if (shares) { warp_share(p0, p1, gwarp, nwarps, &base, &end); step = 32; }
  for (; base < end; base += step) {
    const int64_t e = base + lane;
    const bool valid = e < end;
    // the warp-level search is collective: every lane takes part, valid or not
    const int64_t jc = Wk.col_of ? (valid ? (int64_t)Wk.col_of[e] : -1)
                       : shares  ? find_col_from(Wk.col_ptr, lc0, lc1, hint, e, valid)
                                 : find_col_warp(Wk.col_ptr, lc0, lc1, e, valid);
    if (shares) hint = __shfl_sync(0xffffffffu, jc, 31);
    int64_t j = -1;
    float g = 0.f, u = 0.f;
    if (valid) {
      j = jc;
      if (Wk.active[j]) {
        const float2 ym = Wk.ym[Wk.row_idx[e]];
        const float yi = ym.x;
        const float tau = 1.f / (1.f + __expf(ym.y));
        const float t2 = tau * (1.f - tau);
        const float dj = Wk.delta[j];
        if (binary) {
          g = -yi * tau;
          u = fminf(t2 * __expf(dj), 0.25f);
        } else {
          const float v = Wk.vals[e];
          g = -yi * tau * v;
          u = fminf(t2 * __expf(fabsf(v) * dj), 0.25f) * v * v;
        }
      } else {
        j = -2 - j;  // inactive: keeps the segment boundary, contributes nothing
      }
    }
    // segmented sum over runs of equal j (non-zeros of a column are contiguous)
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int64_t oj = __shfl_down_sync(0xffffffffu, j, off);
      const float og = __shfl_down_sync(0xffffffffu, g, off);
      const float ou = __shfl_down_sync(0xffffffffu, u, off);
      if (lane + off < 32 && oj == j) { g += og; u += ou; }
    }
    const int64_t pj = __shfl_up_sync(0xffffffffu, j, 1);
    const bool head = valid && j >= 0 && (lane == 0 || pj != j);
    if (head) {
      if (mine != nullptr) {   // gather / list group: this rank's own partial sums
        red_add_v2_f32_gpu(mine + (by_local_column ? j : bias + Wk.gcol[j]), g, u);
      } else {
        float2* acc = P.gu[Wk.gowner[j]] + boff + Wk.gslot[j];
        if (P.world > 1) red_add_v2_f32(acc, g, u); else red_add_v2_f32_gpu(acc, g, u);
      }
    }
  }
}

// The proximal-Newton step of one coordinate inside its trust region (Darling::updateWeight,
// src/linear_method/darling.cc:437-477): a pure function of the summed (G,U), the weight, the trust
// region and the pass constants.  The owner applies it to its shard and every worker re-evaluates it
// for its own copy of the column, so each operation is an explicitly rounded intrinsic: the compiler
// may not contract or reorder them differently at the different call sites, and all ranks get the
// same bits.
struct DarlinStep {
  float d;       // Δw (0 when the key is dropped)
  float delta;   // new trust region
  float vio;     // KKT violation of a zero weight
  bool drop;     // the KKT filter takes the key out of the active set
};
__device__ __forceinline__ DarlinStep darlin_step(float g, float u_sum, float wk, float dl, const DarlinHyper& H) {
  DarlinStep r;
  const float u = __fadd_rn(__fdiv_rn(u_sum, H.eta), 1e-10f);
  const float gp = __fadd_rn(g, H.lambda), gn = __fsub_rn(g, H.lambda);
  r.d = -wk; r.vio = 0.f; r.drop = false; r.delta = dl;
  if (wk == 0.f) {
    if (gp < 0.f) r.vio = -gp;
    else if (gn > 0.f) r.vio = gn;
    else if (gp > H.kkt_threshold && gn < -H.kkt_threshold) { r.drop = true; r.d = 0.f; return r; }
  }
  const float uw = __fmul_rn(u, wk);
  if (gp <= uw) r.d = __fdiv_rn(-gp, u);
  else if (gn >= uw) r.d = __fdiv_rn(-gn, u);
  r.d = fminf(dl, fmaxf(-dl, r.d));
  r.delta = fminf(H.delta_max, __fmaf_rn(2.f, fabsf(r.d), 0.1f));
  return r;
}

// Where a column's summed (G,U) comes from: the owner's accumulator (smem == nullptr) or, for a gather group,
// the group's vector in shared memory, element smem[bias + global position of the column]
struct SumSrc {
  const float2* smem;
  int64_t bias;
};

__device__ __forceinline__ float2 ld_gu(const float2* p, bool multi) {
  float2 v;
  if (multi) asm volatile("ld.relaxed.sys.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
  else asm volatile("ld.relaxed.gpu.global.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p) : "memory");
  return v;
}

// ---- phase B: server-side proximal-Newton update of the block's slots.  `clear`: zero the accumulators
// right away (the unfused baseline); the fused pass leaves them for the workers and zeroes them a block later.
__device__ __forceinline__ void darlin_update_weight(const DarlinPeers& P, const DarlinServer& S,
                                                     const DarlinHyper& H, int64_t s0, int64_t s1, int buf, bool clear,
                                                     size_t gtid, size_t gsz, SumSrc src = SumSrc{nullptr, 0},
                                                     float* d_out = nullptr) {
  float* w = P.w[P.rank];
  float2* gu = P.gu[P.rank] + (int64_t)buf * P.gu_stride;
  float vmax = 0.f;
  for (int64_t k = s0 + (int64_t)gtid; k < s1; k += (int64_t)gsz) {
    const float2 a = src.smem != nullptr ? src.smem[src.bias + k] : __ldcg(gu + k);   // (bias maps the slot to its place in the group's vector)
    if (clear) gu[k] = make_float2(0.f, 0.f);
    if (!S.active[k]) { if (d_out != nullptr) d_out[k] = 0.f; continue; }
    const DarlinStep st = darlin_step(a.x, a.y, w[k], S.delta[k], H);
    if (st.drop) {
      S.active[k] = 0;
      w[k] = __int_as_float(0x7fffffff);  // NaN sentinel: key filtered
      if (d_out != nullptr) d_out[k] = __int_as_float(0x7fffffff);
      continue;
    }
    vmax = fmaxf(vmax, st.vio);
    S.delta[k] = st.delta;
    w[k] = __fadd_rn(w[k], st.d);
    if (d_out != nullptr) d_out[k] = st.d;
  }
  vmax = warp_max(vmax);
  if ((threadIdx.x & 31) == 0 && vmax > 0.f) atomicMax(S.violation, __float_as_uint(vmax));
}

// zero the accumulators of a block that every rank has finished reading
__device__ __forceinline__ void darlin_clear_gu(const DarlinPeers& P, int64_t s0, int64_t s1, int buf, size_t gtid,
                                                size_t gsz) {
  float2* gu = P.gu[P.rank] + (int64_t)buf * P.gu_stride;
  for (int64_t k = s0 + (int64_t)gtid; k < s1; k += (int64_t)gsz) gu[k] = make_float2(0.f, 0.f);
}

// ---- worker's copy of a block's columns brought up to date (w, δ, active set): the same step as the owner's,
// from the same sums.  Runs one phase after the block's margin update, when no CTA reads these columns any more.
__device__ __forceinline__ void darlin_commit(const DarlinWorker& Wk, const DarlinPeers& P, const DarlinHyper& H,
                                              int64_t lc0, int64_t lc1, int buf, size_t gtid, size_t gsz,
                                              SumSrc src = SumSrc{nullptr, 0}) {
  const int64_t boff = (int64_t)buf * P.gu_stride;
  const bool multi = P.world > 1;
  for (int64_t j = lc0 + (int64_t)gtid; j < lc1; j += (int64_t)gsz) {
    if (!Wk.active[j]) continue;
    const float2 a = src.smem != nullptr ? src.smem[src.bias + Wk.gcol[j]]
                                         : ld_gu(P.gu[Wk.gowner[j]] + boff + Wk.gslot[j], multi);
    const DarlinStep st = darlin_step(a.x, a.y, Wk.w[j], Wk.delta[j], H);
    if (st.drop) {
      Wk.active[j] = 0;      // its weight is 0 here (NaN only in the owner's shard)
    } else {
      Wk.delta[j] = st.delta;
      Wk.w[j] = __fadd_rn(Wk.w[j], st.d);
    }
  }
}

// ---- margin update of the unfused baseline: m_i += y_i x_ij Δw_j over the block's non-zeros (Δw in Wk.dw)
__device__ __forceinline__ void darlin_update_margin(const DarlinWorker& Wk, int64_t lc0, int64_t lc1, size_t gtid,
                                                     size_t gsz) {
  const int64_t p0 = Wk.col_ptr[lc0], p1 = Wk.col_ptr[lc1];
  for (int64_t e = p0 + (int64_t)gtid; e < p1; e += (int64_t)gsz) {
    const int64_t j = Wk.col_of ? (int64_t)Wk.col_of[e] : find_col(Wk.col_ptr, lc0, lc1, e);
    const float d = __ldcg(Wk.dw + j);
    if (d != 0.f) {
      const uint32_t i = Wk.row_idx[e];
      const float v = Wk.vals ? Wk.vals[e] : 1.f;
      atomicAdd(&Wk.ym[i].y, Wk.ym[i].x * v * d);
    }
  }
}

// Blocks with many columns take phase C in two steps: first every column fetches its (G,U) once, steps and
// brings the worker's copy of the column up to date (Δw kept in Wk.dw), then, after one more in-GPU barrier,
// the non-zeros read Δw locally.  With n non-zeros per column that is n times fewer loads from the owners'
// memory — on 8 GPUs the out-of-core configuration (485 k columns and 1.9 M non-zeros per block and GPU) spent
// most of a pass on one 8-byte NVLink load per non-zero — and one barrier more per group, which only
// matters for small blocks.  The choice depends on this rank's columns only (the extra barrier is local).
constexpr int64_t kWideBlockCols = 16384;

// first step of a wide block: step every column, commit it, keep Δw for the margin update
__device__ __forceinline__ void darlin_step_columns(const DarlinWorker& Wk, const DarlinPeers& P, const DarlinHyper& H,
                                                    int64_t lc0, int64_t lc1, int buf, size_t gtid, size_t gsz) {
  const int64_t boff = (int64_t)buf * P.gu_stride;
  const bool multi = P.world > 1;
  for (int64_t j = lc0 + (int64_t)gtid; j < lc1; j += (int64_t)gsz) {
    float d = 0.f;
    if (Wk.active[j]) {
      const float2 a = ld_gu(P.gu[Wk.gowner[j]] + boff + Wk.gslot[j], multi);
      const DarlinStep st = darlin_step(a.x, a.y, Wk.w[j], Wk.delta[j], H);
      if (st.drop) {
        Wk.active[j] = 0;
      } else {
        d = st.d;
        Wk.delta[j] = st.delta;
        Wk.w[j] = __fadd_rn(Wk.w[j], st.d);
      }
    }
    Wk.dw[j] = d;
  }
}

// second step of a wide block: m_i += y_i x_ij Δw_j with Δw from Wk.dw
__device__ __forceinline__ void darlin_margin_from_dw(const DarlinWorker& Wk, int64_t lc0, int64_t lc1, int64_t p0, int64_t p1,
                                                      size_t gtid, size_t gsz) {
  const int lane = threadIdx.x & 31;
  const bool shares = kRangeWalk && Wk.col_of == nullptr;
  int64_t base = p0 + (int64_t)gtid - lane, end = p1, step = (int64_t)gsz, hint = -1;
  if (shares) { warp_share(p0, p1, gtid >> 5, gsz >> 5, &base, &end); step = 32; }
  for (; base < end; base += step) {
    const int64_t e = base + lane;
    const bool valid = e < end;
    const int64_t j = Wk.col_of ? (valid ? (int64_t)Wk.col_of[e] : -1)
                      : shares  ? find_col_from(Wk.col_ptr, lc0, lc1, hint, e, valid)
                                : find_col_warp(Wk.col_ptr, lc0, lc1, e, valid);
    if (shares) hint = __shfl_sync(0xffffffffu, j, 31);
    if (!valid) continue;
    const float d = __ldcg(Wk.dw + j);
    if (d != 0.f) {
      const uint32_t i = Wk.row_idx[e];
      const float v = Wk.vals ? Wk.vals[e] : 1.f;
      atomicAdd(&Wk.ym[i].y, Wk.ym[i].x * v * d);
    }
  }
}

// ---- fused phase C of the persistent kernel: every non-zero fetches its column's summed (G,U) from the
// owner and the column's state from the worker, re-evaluates the step and moves the margin by y·x·Δw.  The
// worker-side column state (w, δ, active) is NOT written here — other CTAs are still reading it — but one
// phase later by darlin_commit.
__device__ __forceinline__ void darlin_step_margin(const DarlinWorker& Wk, const DarlinPeers& P, const DarlinHyper& H,
                                                   int64_t lc0, int64_t lc1, int64_t p0, int64_t p1, int buf, size_t gtid,
                                                   size_t gsz, SumSrc src = SumSrc{nullptr, 0}) {
  const int lane = threadIdx.x & 31;
  const int64_t boff = (int64_t)buf * P.gu_stride;
  const bool multi = P.world > 1;
  // warp-uniform trip count (gsz is a multiple of 32): the column search without col_of is a warp collective
  const bool shares = kRangeWalk && Wk.col_of == nullptr;
  int64_t base = p0 + (int64_t)gtid - lane, end = p1, step = (int64_t)gsz, hint = -1;
  if (shares) { warp_share(p0, p1, gtid >> 5, gsz >> 5, &base, &end); step = 32; }
  for (; base < end; base += step) {
    const int64_t e = base + lane;
    const bool valid = e < end;
    const int64_t j = Wk.col_of ? (valid ? (int64_t)Wk.col_of[e] : -1)
                      : shares  ? find_col_from(Wk.col_ptr, lc0, lc1, hint, e, valid)
                                : find_col_warp(Wk.col_ptr, lc0, lc1, e, valid);
    if (shares) hint = __shfl_sync(0xffffffffu, j, 31);
    if (!valid || !Wk.active[j]) continue;
    const float2 a = src.smem != nullptr ? src.smem[src.bias + Wk.gcol[j]]
                                         : ld_gu(P.gu[Wk.gowner[j]] + boff + Wk.gslot[j], multi);
    const DarlinStep st = darlin_step(a.x, a.y, Wk.w[j], Wk.delta[j], H);
    if (st.d != 0.f) {
      const uint32_t i = Wk.row_idx[e];
      const float v = Wk.vals ? Wk.vals[e] : 1.f;
      atomicAdd(&Wk.ym[i].y, Wk.ym[i].x * v * st.d);
    }
  }
}

// ---- small groups on several GPUs: partial sums gathered on every rank
// A group with at most kGatherCols columns over all owners does not push into the owners' accumulators.  Every
// rank sums its gradients into a buffer of its own (GPU-scope reductions, nothing leaves the GPU, no system-scope
// fence per thread block); the thread block that completes the rank's count copies that buffer into every
// rank's inbox (coalesced peer stores), fences once and raises the arrival counters.  After the one cross-GPU
// wait each thread block adds the `world` partial vectors in rank order into shared memory — every rank gets
// bit for bit the same sums, whatever the timing — and the owner's update, the margin update and the commit of
// the worker's columns all read them from there: no load crosses NVLink in phase C.  With 300 blocks of ~160
// columns and 8 GPUs this path decides the time of a pass (a block is a few microseconds of work between two
// synchronisations).
constexpr int kGatherCols = 2048;

// Everything the pass needs to know about the block at one position of the order, fetched ahead of time
// into shared memory: a group costs a handful of microseconds, and chasing order -> block table -> column
// offsets through global memory at the start of every phase was a third of that.
struct BlkMeta {
  int64_t p0, p1;      // CSC positions of the block's non-zeros on this worker
  int64_t gc0;         // first column of the block in the global sorted key list
  int32_t lc0, lc1;    // local columns
  int32_t sl0, sl1;    // slots on this owner
  int32_t gw;          // columns of the block over all owners
  int32_t blk;         // block id
};
constexpr int kMetaSlots = 512;

__device__ __forceinline__ void load_meta(const DarlinWorker& Wk, const DarlinSched& Q, int first, int count, BlkMeta* m) {
  for (int i = threadIdx.x; i < count; i += blockDim.x) {
    const int blk = Q.order[first + i];
    BlkMeta x;
    x.blk = blk;
    x.lc0 = (int32_t)Q.blk_lc[2 * blk]; x.lc1 = (int32_t)Q.blk_lc[2 * blk + 1];
    x.sl0 = (int32_t)Q.blk_sl[2 * blk]; x.sl1 = (int32_t)Q.blk_sl[2 * blk + 1];
    x.p0 = Wk.col_ptr[x.lc0]; x.p1 = Wk.col_ptr[x.lc1];
    x.gc0 = Q.blk_gc != nullptr ? Q.blk_gc[2 * blk] : 0;
    x.gw = Q.blk_gc != nullptr ? (int32_t)(Q.blk_gc[2 * blk + 1] - Q.blk_gc[2 * blk]) : 0x7fffffff / 4096;
    m[i] = x;
  }
}
// of the blocks m[0 .. n): local columns, columns over all owners
__device__ __forceinline__ int64_t meta_lcols(const BlkMeta* m, int n) {
  int64_t c = 0;
  for (int i = 0; i < n; ++i) c += m[i].lc1 - m[i].lc0;
  return c;
}
__device__ __forceinline__ int64_t meta_gcols(const BlkMeta* m, int n) {
  int64_t c = 0;
  for (int i = 0; i < n; ++i) c += m[i].gw;
  return c;
}
// index of block m[i]'s first column inside its group's vector, minus the block's first global column:
// adding a column's global position gives its place in the vector
__device__ __forceinline__ int64_t meta_bias(const BlkMeta* m, int i) {
  int64_t off = 0;
  for (int k = 0; k < i; ++k) off += m[k].gw;
  return off - m[i].gc0;
}

// arrival of a gather group (see cta_arrive_all for the two-level count)
__device__ __forceinline__ void cta_arrive_gather(const DarlinPeers& P, uint64_t* local_ctr, uint64_t local_target, int n,
                                                  int buf, bool* s_last) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned long long prev;
    asm volatile("atom.acq_rel.gpu.global.add.u64 %0, [%1], %2;" : "=l"(prev) : "l"(local_ctr), "l"(1ull) : "memory");
    *s_last = prev + 1ull == local_target;
  }
  __syncthreads();
  if (!*s_last) return;
  const size_t slot = ((size_t)buf * P.world + P.rank) * kGatherCols;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float2 v = __ldcg(P.mine + i);
    P.mine[i] = make_float2(0.f, 0.f);        // ready for the next group
    for (int t = 0; t < P.world; ++t) {
      float2* dst = P.part[t] + slot + i;
      if (t == P.rank) *dst = v;
      else asm volatile("st.relaxed.sys.global.v2.f32 [%0], {%1, %2};" ::"l"(dst), "f"(v.x), "f"(v.y) : "memory");
    }
  }
  __syncthreads();
  if (threadIdx.x < P.world) {
    __threadfence_system();
    red_release_sys_add_u64(P.arrive[threadIdx.x], 1ull);
  }
}

// sums of a gather group in shared memory: the partial vectors of all ranks added in rank order
__device__ __forceinline__ void gather_reduce(const DarlinPeers& P, int n, int buf, float2* s_sum) {
  const float2* in = P.part[P.rank] + (size_t)buf * P.world * kGatherCols;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float2 a = make_float2(0.f, 0.f);
    for (int r = 0; r < P.world; ++r) {
      const float2 v = __ldcg(in + (size_t)r * kGatherCols + c);   // written by other GPUs: from L2
      a.x = __fadd_rn(a.x, v.x);
      a.y = __fadd_rn(a.y, v.y);
    }
    s_sum[c] = a;
  }
  __syncthreads();
}

// ---- very wide groups on several GPUs: push and pull as bulk transfers over resolved column lists
// With hundreds of thousands of columns per block and GPU, one small NVLink operation per column (a reduction
// into the owner's accumulator, a load of its sums) is what a pass costs on 8 GPUs: 7/8 of them leave the GPU.
// Every owner holds one run of consecutive keys of every block, so a worker's columns of one owner and block are
// contiguous in its local (key) order, and their slots in the owner's shard were resolved once — the steady state of the reference's key cache
// (src/system/remote_node.cc:96-184).  So for these groups
//   * a worker sums (G,U) per LOCAL column in its own memory;
//   * after the arrival the owner reads, for every sender, the contiguous run of that sender's columns in its
//     share of the block — the partial sums and their slots — with coalesced peer loads, and adds them into its
//     accumulators with GPU-scope reductions;
//   * the owner steps its slots, keeps Δw per slot, and writes Δw back per sender column, again contiguous;
//   * after a second arrival the worker brings its copy of the columns up to date from Δw (δ follows from Δw by
//     the owner's formula, NaN = dropped) and moves the margins.
// Two cross-GPU rounds and four in-GPU barriers per group, all NVLink traffic in full lines.
constexpr int64_t kListCols = 262144;

// sender r's local columns of block `blk` that this rank owns: [a, e)
__device__ __forceinline__ void list_range(const DarlinPeers& P, const DarlinSched& Q, int r, int blk, int64_t* a, int64_t* e) {
  const int64_t* cb = Q.all_cb + ((int64_t)r * Q.nblocks_total + blk) * (P.world + 1);
  *a = cb[P.rank];
  *e = cb[P.rank + 1];
}

// The senders' runs of one block, laid end to end: position g of [0, total) belongs to sender r with
// s_pre[r] <= g < s_pre[r + 1], column s_a[r] + g − s_pre[r].  One flat loop over all senders keeps every peer
// load in flight at once; a loop per sender paid one NVLink round trip after the other (355 us per block on 8 GPUs).
struct ListRuns {
  int64_t a[PSB_MAX_RANKS];
  int64_t pre[PSB_MAX_RANKS + 1];
  int rk[PSB_MAX_RANKS];      // sender of every run: the owners start at different senders (rank, rank + 1, ...), so
                              // that they do not all read the same GPU's memory at the same time
};
__device__ __forceinline__ void list_runs(const DarlinPeers& P, const DarlinSched& Q, int blk, ListRuns* s_runs) {
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t run = 0;
    for (int i = 0; i < P.world; ++i) {
      const int r = (P.rank + i) % P.world;
      int64_t a, e;
      list_range(P, Q, r, blk, &a, &e);
      s_runs->rk[i] = r;
      s_runs->a[i] = a;
      s_runs->pre[i] = run;
      run += e > a ? e - a : 0;
    }
    for (int i = P.world; i <= PSB_MAX_RANKS; ++i) s_runs->pre[i] = run;
  }
  __syncthreads();
}
__device__ __forceinline__ int list_sender(const ListRuns* s_runs, int world, int64_t g) {
  int r = 0;
#pragma unroll
  for (int i = 1; i < PSB_MAX_RANKS; ++i) r += (i < world && g >= s_runs->pre[i]) ? 1 : 0;
  return r;
}

__device__ __forceinline__ void darlin_list_sum(const DarlinPeers& P, const DarlinSched& Q, int blk, int buf, size_t gtid, size_t gsz,
                                                ListRuns* s_runs) {
  float2* acc = P.gu[P.rank] + (int64_t)buf * P.gu_stride;
  list_runs(P, Q, blk, s_runs);
  const int64_t total = s_runs->pre[PSB_MAX_RANKS];
  for (int64_t g = (int64_t)gtid; g < total; g += (int64_t)gsz) {
    const int i = list_sender(s_runs, P.world, g);
    const int r = s_runs->rk[i];
    const int64_t j = s_runs->a[i] + (g - s_runs->pre[i]);
    const bool peer = r != P.rank;
    const float2 v = peer ? ld_gu(P.colgu[r] + j, true) : __ldcg(P.colgu[r] + j);
    const uint32_t slot = peer ? ld_relaxed_sys_u32(P.colslot[r] + j) : P.colslot[r][j];
    if (v.x == 0.f && v.y == 0.f) continue;     // inactive or absent on that worker
    red_add_v2_f32_gpu(acc + slot, v.x, v.y);
  }
}

__device__ __forceinline__ void darlin_list_reply(const DarlinPeers& P, const DarlinServer& S, const DarlinSched& Q, int blk,
                                                  size_t gtid, size_t gsz, ListRuns* s_runs) {
  list_runs(P, Q, blk, s_runs);
  const int64_t total = s_runs->pre[PSB_MAX_RANKS];
  for (int64_t g = (int64_t)gtid; g < total; g += (int64_t)gsz) {
    const int i = list_sender(s_runs, P.world, g);
    const int r = s_runs->rk[i];
    const int64_t j = s_runs->a[i] + (g - s_runs->pre[i]);
    const bool peer = r != P.rank;
    const uint32_t slot = peer ? ld_relaxed_sys_u32(P.colslot[r] + j) : P.colslot[r][j];
    const float d = __ldcg(S.d_slot + slot);
    if (peer) st_relaxed_sys_f32(P.coldw[r] + j, d); else P.coldw[r][j] = d;
  }
}

// worker: its copy of the group's columns from the owners' answers; its partial sums zeroed for the next use
__device__ __forceinline__ void darlin_list_apply(const DarlinWorker& Wk, const DarlinPeers& P, const DarlinHyper& H, int64_t lc0,
                                                  int64_t lc1, size_t gtid, size_t gsz) {
  const float* in = P.coldw[P.rank];
  float2* mine = P.colgu[P.rank];
  for (int64_t j = lc0 + (int64_t)gtid; j < lc1; j += (int64_t)gsz) {
    mine[j] = make_float2(0.f, 0.f);
    float d = 0.f;
    if (Wk.active[j]) {
      d = __ldcg(in + j);
      if (d != d) {
        Wk.active[j] = 0;
        d = 0.f;
      } else {
        Wk.delta[j] = fminf(H.delta_max, __fmaf_rn(2.f, fabsf(d), 0.1f));   // the owner's rule (darlin_step)
        Wk.w[j] = __fadd_rn(Wk.w[j], d);
      }
    }
    Wk.dw[j] = d;
  }
}

// worker view for the block at position q of the order: in out-of-core mode its row ids and values sit
// in a staging buffer; the phases index them with absolute CSC positions, so the pointers are biased by p0
__device__ __forceinline__ DarlinWorker worker_for(const DarlinWorker& Wk, const DarlinSched& Q, int q, int64_t p0,
                                                   int64_t p1) {
  DarlinWorker W = Wk;
  if (Q.stage_base != nullptr) {
    const uint32_t* base = reinterpret_cast<const uint32_t*>(Q.stage_base[q]);
    W.row_idx = base - p0;
    W.vals = Wk.vals != nullptr ? reinterpret_cast<const float*>(base + (p1 - p0)) - p0 : nullptr;
  }
  return W;
}

__global__ void __launch_bounds__(512)
darlin_pass_kernel(DarlinWorker Wk, DarlinPeers P, DarlinServer S, DarlinSched Q, DarlinHyper H) {
  __shared__ bool s_ok, s_last;
  __shared__ uint32_t s_abort;
  __shared__ float2 s_sum[kGatherCols];     // sums of the gather group in flight (kept until the next one is reduced)
  __shared__ BlkMeta s_meta[kMetaSlots];    // metadata of a window of the order, one group of history in front
  __shared__ ListRuns s_runs;
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gsz = (size_t)gridDim.x * blockDim.x;
  const int lane = threadIdx.x & 31;
  const uint64_t G = gridDim.x;
  uint64_t bar = *(volatile uint64_t*)(Q.local_bar + 3);   // every CTA reads it before any CTA can finish the launch

  // Blocks are processed in groups of Q.group consecutive entries of the order (group = max_block_delay + 1):
  // the gradients of all blocks of a group are computed before any of them is updated, i.e. a block may see
  // weights that are up to `group - 1` block updates old — the bounded-delay schedule of the reference
  // (wait_time = time - tau, src/linear_method/darling.cc:45-69) with one set of synchronisation points per group.
  // Group number `seq` (counted over all launches, the same on every rank) accumulates into buffer seq % 3.
  const int group = min(Q.group > 0 ? Q.group : 1, kMetaSlots / 4);
  const bool multi = P.world > 1;
  const int64_t wide_cols = Q.wide_cols > 0 ? (int64_t)Q.wide_cols : kWideBlockCols;
  const int64_t list_cols = Q.list_cols > 0 ? Q.list_cols : kListCols;
  // by default only from four GPUs on: on two, one 8-byte peer load per column (the wide path) is cheaper than the
  // three extra sweeps over the column lists (6.7 against 10.5 ms per pass on 2 x 10^6 rows x 120 non-zeros); on
  // eight, 7/8 of those loads cross NVLink as small packets and the pass took 30.5 ms
  const bool can_list = multi && Q.all_cb != nullptr && Q.blk_gc != nullptr && (Q.list_cols > 0 || P.world >= 4);
  uint64_t seq = Q.seq0;
  uint64_t seq2 = *(volatile uint64_t*)(Q.local_bar + 4);   // list groups completed so far (second arrival counter)
// in-GPU barrier (bounded); leaves the group loop when it runs out
#define PSB_LOCAL_BARRIER(code)                                                                            \
  __syncthreads();                                                                                         \
  if (threadIdx.x == 0) { __threadfence(); atomicAdd((unsigned long long*)Q.local_bar, 1ull); }            \
  if (!cta_wait_counter(Q.local_bar, (++bar) * G, P.timeout_ns, false, &s_ok)) {                           \
    if (threadIdx.x == 0) { set_status(Q.status, kWaitTimeout, (uint32_t)mg[0].blk, code); *Q.abort_flag = 1u; } \
    break;                                                                                                 \
  }
  int wbase = 0, wend = 0;     // s_meta[q - wbase] describes position q of the order, for wbase <= q < wend
  for (int b = 0; b < Q.nblk; b += group) {
    if (threadIdx.x == 0) s_abort = *(volatile uint32_t*)Q.abort_flag;
    __syncthreads();
    if (s_abort) break;  // uniform over the CTA
    const int ge = min(b + group, Q.nblk);
    const int pb = max(b - group, 0);
    if (ge > wend) {     // next window: from the previous group (its commit is still to come) onwards
      wbase = pb;
      wend = min(Q.nblk, wbase + kMetaSlots);
      load_meta(Wk, Q, wbase, wend - wbase, s_meta);
      __syncthreads();
    }
    const BlkMeta* mp = s_meta + (pb - wbase);   // previous group (b - pb blocks)
    const BlkMeta* mg = s_meta + (b - wbase);    // this group (ge - b blocks)
    const int ng = ge - b, np = b - pb;
    ++seq;
    const int buf = (int)(seq % 3), pbuf = (int)((seq + 2) % 3);
    const bool timed = Q.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
    uint64_t t0 = timed ? globaltimer_ns() : 0, t1;

    // A: gradient + push, then announce arrival at every owner.  In the same phase: the worker's copy of the
    // previous group's columns is brought up to date (a different set of columns; all CTAs are past its
    // phase C; the previous launch did this itself for its last group; a wide group committed its columns itself).
    const bool prev_gather = np > 0 && multi && Q.gather != 0 && Q.blk_gc != nullptr && meta_gcols(mp, np) <= kGatherCols;
    const bool prev_list = np > 0 && can_list && meta_gcols(mp, np) > list_cols;
    const bool prev_commit = np > 0 && !prev_list && (prev_gather || meta_lcols(mp, np) <= wide_cols);
    const bool gat = multi && Q.gather != 0 && Q.blk_gc != nullptr && meta_gcols(mg, ng) <= kGatherCols;
    const int gcols = gat ? (int)meta_gcols(mg, ng) : 0;
    const bool lst = !gat && can_list && meta_gcols(mg, ng) > list_cols;     // the same choice on every rank
    const bool wide = !gat && !lst && meta_lcols(mg, ng) > wide_cols;
    if (prev_commit && !prev_gather) {   // sums in the owners' accumulators: read them before this rank arrives
      for (int i = 0; i < np; ++i) darlin_commit(Wk, P, H, mp[i].lc0, mp[i].lc1, pbuf, gtid, gsz);
    }
    for (int i = 0; i < ng; ++i) {
      darlin_grad_push(worker_for(Wk, Q, b + i, mg[i].p0, mg[i].p1), P, mg[i].lc0, mg[i].lc1, mg[i].p0, mg[i].p1, buf,
                       gat ? P.mine : (lst ? P.colgu[P.rank] : nullptr), gat ? meta_bias(mg, i) : 0, gtid >> 5, gsz >> 5,
                       lane, lst);
    }
    if (timed) { t1 = globaltimer_ns(); Q.trace[0] += t1 - t0; t0 = t1; }
    if (gat) cta_arrive_gather(P, Q.local_bar + 1, seq * G, gcols, buf, &s_last);
    else cta_arrive_all(P, P.arrive, Q.local_bar + 1, seq * G, &s_last);
    if (prev_commit && prev_gather) {    // sums still in shared memory: commit while the other ranks arrive
      for (int i = 0; i < np; ++i)
        darlin_commit(Wk, P, H, mp[i].lc0, mp[i].lc1, pbuf, gtid, gsz, SumSrc{s_sum, meta_bias(mp, i)});
    }
    if (!cta_wait_counter(P.arrive[P.rank], seq * (uint64_t)P.world, P.timeout_ns, multi, &s_ok)) {
      if (threadIdx.x == 0) { set_status(Q.status, kWaitTimeout, (uint32_t)mg[0].blk, 11); *Q.abort_flag = 1u; }
      break;
    }
    if (timed) { t1 = globaltimer_ns(); Q.trace[1] += t1 - t0; t0 = t1; }
    if (lst) {
      // owner: sum the senders' runs of columns into the accumulators, step, answer per sender column
      uint64_t u0 = timed ? globaltimer_ns() : 0, u1;
      for (int i = 0; i < ng; ++i) darlin_list_sum(P, Q, mg[i].blk, buf, gtid, gsz, &s_runs);
      PSB_LOCAL_BARRIER(15)
      if (timed) { u1 = globaltimer_ns(); Q.trace[4] += u1 - u0; u0 = u1; }
      for (int i = 0; i < ng; ++i)
        darlin_update_weight(P, S, H, mg[i].sl0, mg[i].sl1, buf, true, gtid, gsz, SumSrc{nullptr, 0}, S.d_slot);
      PSB_LOCAL_BARRIER(16)
      if (timed) { u1 = globaltimer_ns(); Q.trace[5] += u1 - u0; u0 = u1; }
      for (int i = 0; i < ng; ++i) darlin_list_reply(P, S, Q, mg[i].blk, gtid, gsz, &s_runs);
      if (timed) { u1 = globaltimer_ns(); Q.trace[6] += u1 - u0; u0 = u1; }
      ++seq2;
      cta_arrive_all(P, P.arrive2, Q.local_bar + 2, seq2 * G, &s_last);
      if (!cta_wait_counter(P.arrive2[P.rank], seq2 * (uint64_t)P.world, P.timeout_ns, true, &s_ok)) {
        if (threadIdx.x == 0) { set_status(Q.status, kWaitTimeout, (uint32_t)mg[0].blk, 12); *Q.abort_flag = 1u; }
        break;
      }
      // worker: columns from the answers, then the margins
      if (timed) { u1 = globaltimer_ns(); Q.trace[7] += u1 - u0; u0 = u1; }
      for (int i = 0; i < ng; ++i) darlin_list_apply(Wk, P, H, mg[i].lc0, mg[i].lc1, gtid, gsz);
      PSB_LOCAL_BARRIER(17)
      if (timed) { u1 = globaltimer_ns(); Q.trace[8] += u1 - u0; u0 = u1; }
      for (int i = 0; i < ng; ++i)
        darlin_margin_from_dw(worker_for(Wk, Q, b + i, mg[i].p0, mg[i].p1), mg[i].lc0, mg[i].lc1, mg[i].p0, mg[i].p1, gtid, gsz);
      __syncthreads();
      if (timed) { t1 = globaltimer_ns(); Q.trace[9] += t1 - u0; Q.trace[2] += t1 - t0; t0 = t1; }
      PSB_LOCAL_BARRIER(14)
      if (timed) { t1 = globaltimer_ns(); Q.trace[3] += t1 - t0; t0 = t1; }
      continue;
    }
    if (gat) gather_reduce(P, gcols, buf, s_sum);
    // B and C in one phase.  Owner: update this shard's slots of the group's blocks; zero the accumulators of
    // the previous group, which every rank has read for the last time (its arrival above came after that).
    for (int i = 0; i < ng; ++i) {
      const SumSrc src = gat ? SumSrc{s_sum, meta_bias(mg, i) + Q.blk_gs0[mg[i].blk] - mg[i].sl0} : SumSrc{nullptr, 0};
      darlin_update_weight(P, S, H, mg[i].sl0, mg[i].sl1, buf, false, gtid, gsz, src);
    }
    if (np > 0) {
      for (int i = 0; i < np && !prev_gather && !prev_list; ++i) darlin_clear_gu(P, mp[i].sl0, mp[i].sl1, pbuf, gtid, gsz);
    } else if (Q.prev != nullptr) {
      for (int q = 0; q < Q.nprev; ++q) {
        const int blk = Q.prev[q];
        darlin_clear_gu(P, Q.blk_sl[2 * blk], Q.blk_sl[2 * blk + 1], pbuf, gtid, gsz);
      }
    }
    // Worker: margins of the rows that the group's columns touch.
    if (wide) {
      for (int i = 0; i < ng; ++i) darlin_step_columns(Wk, P, H, mg[i].lc0, mg[i].lc1, buf, gtid, gsz);
      __syncthreads();
      if (threadIdx.x == 0) { __threadfence(); atomicAdd((unsigned long long*)Q.local_bar, 1ull); }
      if (!cta_wait_counter(Q.local_bar, (++bar) * G, P.timeout_ns, false, &s_ok)) {
        if (threadIdx.x == 0) { set_status(Q.status, kWaitTimeout, (uint32_t)mg[0].blk, 13); *Q.abort_flag = 1u; }
        break;
      }
    }
    for (int i = 0; i < ng; ++i) {
      const DarlinWorker W = worker_for(Wk, Q, b + i, mg[i].p0, mg[i].p1);
      if (wide) darlin_margin_from_dw(W, mg[i].lc0, mg[i].lc1, mg[i].p0, mg[i].p1, gtid, gsz);
      else darlin_step_margin(W, P, H, mg[i].lc0, mg[i].lc1, mg[i].p0, mg[i].p1, buf, gtid, gsz,
                              gat ? SumSrc{s_sum, meta_bias(mg, i)} : SumSrc{nullptr, 0});
    }
    __syncthreads();
    if (timed) { t1 = globaltimer_ns(); Q.trace[2] += t1 - t0; t0 = t1; }
    if (threadIdx.x == 0) { __threadfence(); atomicAdd((unsigned long long*)Q.local_bar, 1ull); }
    if (!cta_wait_counter(Q.local_bar, (++bar) * G, P.timeout_ns, false, &s_ok)) {
      if (threadIdx.x == 0) { set_status(Q.status, kWaitTimeout, (uint32_t)mg[0].blk, 14); *Q.abort_flag = 1u; }
      break;
    }
    if (timed) { t1 = globaltimer_ns(); Q.trace[3] += t1 - t0; t0 = t1; }
    if (ge == Q.nblk && !wide) {  // last group of the launch: bring the worker's copy of its columns up to date now
      for (int i = 0; i < ng; ++i)
        darlin_commit(Wk, P, H, mg[i].lc0, mg[i].lc1, buf, gtid, gsz, gat ? SumSrc{s_sum, meta_bias(mg, i)} : SumSrc{nullptr, 0});
    }
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) { Q.local_bar[3] = bar; Q.local_bar[4] = seq2; }
#undef PSB_LOCAL_BARRIER
}

// ---- stand-alone phase kernels (unfused NCCL baseline; gradients go to local buffers)
__global__ void k_darlin_grad_local(DarlinWorker Wk, int64_t lc0, int64_t lc1, float2* gu_local) {
  // same reduction as phase A, accumulated into a local per-column buffer (index j − lc0)
  DarlinPeers P{};
  const size_t gtid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t gwarp = gtid >> 5, nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int64_t p0 = Wk.col_ptr[lc0], p1 = Wk.col_ptr[lc1];
  const bool binary = Wk.vals == nullptr;
  (void)P;
  for (int64_t base = p0 + (int64_t)gwarp * 32; base < p1; base += (int64_t)nwarps * 32) {
    const int64_t e = base + lane;
    const bool valid = e < p1;
    int64_t j = -1;
    float g = 0.f, u = 0.f;
    if (valid) {
      j = Wk.col_of ? (int64_t)Wk.col_of[e] : find_col(Wk.col_ptr, lc0, lc1, e);
      if (Wk.active[j]) {
        const float2 ym = Wk.ym[Wk.row_idx[e]];
        const float yi = ym.x;
        const float tau = 1.f / (1.f + __expf(ym.y));
        const float t2 = tau * (1.f - tau);
        const float dj = Wk.delta[j];
        if (binary) { g = -yi * tau; u = fminf(t2 * __expf(dj), 0.25f); }
        else { const float v = Wk.vals[e]; g = -yi * tau * v; u = fminf(t2 * __expf(fabsf(v) * dj), 0.25f) * v * v; }
      } else {
        j = -2 - j;
      }
    }
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int64_t oj = __shfl_down_sync(0xffffffffu, j, off);
      const float og = __shfl_down_sync(0xffffffffu, g, off);
      const float ou = __shfl_down_sync(0xffffffffu, u, off);
      if (lane + off < 32 && oj == j) { g += og; u += ou; }
    }
    const int64_t pj = __shfl_up_sync(0xffffffffu, j, 1);
    if (valid && j >= 0 && (lane == 0 || pj != j)) {
      atomicAdd(&gu_local[j - lc0].x, g);
      atomicAdd(&gu_local[j - lc0].y, u);
    }
  }
}
__global__ void k_darlin_update_weight(DarlinPeers P, DarlinServer S, DarlinHyper H, int64_t s0, int64_t s1) {
  darlin_update_weight(P, S, H, s0, s1, 0, true, (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
}
// Δw etc. from an explicit array of new weights (w_new[j − lc0]) instead of peer loads
__global__ void k_darlin_apply_pull(DarlinWorker Wk, DarlinHyper H, int64_t lc0, int64_t lc1, const float* w_new) {
  for (int64_t j = lc0 + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < lc1; j += (int64_t)gridDim.x * blockDim.x) {
    float d = 0.f;
    if (Wk.active[j]) {
      const float wn = w_new[j - lc0];
      if (wn != wn) { Wk.active[j] = 0; Wk.w[j] = 0.f; }
      else { d = wn - Wk.w[j]; Wk.delta[j] = fminf(H.delta_max, 2.f * fabsf(d) + 0.1f); Wk.w[j] = wn; }
    }
    Wk.dw[j] = d;
  }
}
__global__ void k_darlin_update_margin(DarlinWorker Wk, int64_t lc0, int64_t lc1) {
  darlin_update_margin(Wk, lc0, lc1, (size_t)blockIdx.x * blockDim.x + threadIdx.x, (size_t)gridDim.x * blockDim.x);
}
// margin_i = y_i · Σ_j x_ij w_j from scratch (initialisation with non-zero weights, drift checks)
__global__ void k_darlin_margin_init(DarlinWorker Wk) {
  const int64_t p1 = Wk.col_ptr[Wk.cols];
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < p1; e += (int64_t)gridDim.x * blockDim.x) {
    const int64_t j = Wk.col_of ? (int64_t)Wk.col_of[e] : find_col(Wk.col_ptr, 0, Wk.cols, e);
    const float wj = Wk.w[j];
    if (wj != 0.f && wj == wj) {
      const uint32_t i = Wk.row_idx[e];
      atomicAdd(&Wk.ym[i].y, Wk.ym[i].x * (Wk.vals ? Wk.vals[e] : 1.f) * wj);
    }
  }
}

}  // namespace psb

using namespace psb;

namespace {
int g_darlin_grid[16] = {0};
}

extern "C" {

// Number of CTAs of the pass kernel on the current device (every rank must use the same value).
int psb_darlin_grid() {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) dev = 0;
  if (g_darlin_grid[dev] == 0) {
    int per_sm = 0, sms = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, darlin_pass_kernel, 512, 0);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int want = 2;  // CTAs per SM (upper bound of the grid; the solver launches 1 per SM when every block synchronises): more CTAs hide gather latency, fewer make the per-block barriers cheaper
    g_darlin_grid[dev] = sms * (per_sm > want ? want : per_sm);  // upper bound; callers may launch fewer
  }
  return g_darlin_grid[dev];
}

int psb_darlin_pass(const DarlinWorker* Wk, const DarlinPeers* P, const DarlinServer* S, const DarlinSched* Q,
                    const DarlinHyper* H, int grid, cudaStream_t stream) {
  if (grid <= 0 || grid > psb_darlin_grid()) return (int)cudaErrorInvalidValue;
  DarlinWorker w = *Wk; DarlinPeers p = *P; DarlinServer s = *S; DarlinSched q = *Q; DarlinHyper h = *H;
  void* args[] = {&w, &p, &s, &q, &h};
  return (int)cudaLaunchCooperativeKernel((void*)darlin_pass_kernel, dim3(grid), dim3(512), args, 0, stream);
}

// ---- out-of-core pass: the role of FeatureStation's prefetch threads
// (src/linear_method/feature_station.cc:212-279) as one native call per pass.
// The column blocks live in pinned host memory, packed per block as [row ids | values].  The block
// order is cut into batches of `batch` blocks; a ring of `depth` device buffers, one batch each, is
// filled on two alternating copy streams ahead of the order (one copy per block), and every batch
// runs as ONE launch of the pass kernel on the compute stream: a cooperative launch costs about
// 28 us, as much as a whole block, so one launch per block doubles the time of a pass
// (measured, resident data: 8.5 ms per pass with one launch, 9.3 ms with 10 blocks per launch,
// 16.2 ms with one block per launch).  The streamer owns the copy streams and the ring's events.
struct DarlinStreamer {
  int depth = 0;
  cudaStream_t copy[2] = {nullptr, nullptr};  // alternated: the fixed cost of consecutive small copies overlaps
  cudaEvent_t ready[16] = {nullptr};
  cudaEvent_t vacant[16] = {nullptr};
};

void psb_darlin_streamer_destroy(void* handle);

void* psb_darlin_streamer_create(int depth) {
  if (depth < 2 || depth > 16) return nullptr;
  DarlinStreamer* h = new DarlinStreamer();
  h->depth = depth;
  for (int i = 0; i < 2; ++i)
    if (cudaStreamCreateWithFlags(&h->copy[i], cudaStreamNonBlocking) != cudaSuccess) {
      psb_darlin_streamer_destroy(h);
      return nullptr;
    }
  for (int i = 0; i < depth; ++i) {
    cudaEventCreateWithFlags(&h->ready[i], cudaEventDisableTiming);
    cudaEventCreateWithFlags(&h->vacant[i], cudaEventDisableTiming);
  }
  return h;
}

void psb_darlin_streamer_destroy(void* handle) {
  DarlinStreamer* h = static_cast<DarlinStreamer*>(handle);
  if (h == nullptr) return;
  for (int i = 0; i < h->depth; ++i) {
    if (h->ready[i]) cudaEventDestroy(h->ready[i]);
    if (h->vacant[i]) cudaEventDestroy(h->vacant[i]);
  }
  for (int i = 0; i < 2; ++i)
    if (h->copy[i]) cudaStreamDestroy(h->copy[i]);
  delete h;
}

// order_host[n]: block ids of this pass; blk_nnz_host[2·b], [2·b+1]: CSC range [p0, p1) of block b;
// host_pack: pinned, block b at word offset words·p0 (words = 2 with values, 1 without): p1−p0 row
// ids, then p1−p0 values; stage[depth]: device buffers of at least batch·words·max(p1−p0) 4-byte
// words; stage_base_dev[n]: device scratch for the address of every block's data; batch: blocks
// per launch (rounded up to a multiple of the pass's synchronisation group).  Q0 describes the
// pass like for psb_darlin_pass (order on the device, group, seq0, bar0).  *h2d_bytes is advanced
// by the bytes copied, *launches by the kernel launches.
int psb_darlin_pass_streamed(void* handle, const DarlinWorker* Wk, const DarlinPeers* P, const DarlinServer* S,
                             const DarlinSched* Q0, const DarlinHyper* H, int grid, const int32_t* order_host, int n,
                             const int64_t* blk_nnz_host, const uint32_t* host_pack, int has_vals,
                             void* const* stage, uint64_t* stage_base_dev, int batch, cudaStream_t compute,
                             unsigned long long* h2d_bytes, int* launches) {
  DarlinStreamer* h = static_cast<DarlinStreamer*>(handle);
  if (h == nullptr || grid <= 0 || grid > psb_darlin_grid() || stage_base_dev == nullptr) return (int)cudaErrorInvalidValue;
  const int d = h->depth;
  const size_t words = has_vals ? 2 : 1;
  const int grp = Q0->group > 0 ? Q0->group : 1;
  if (batch < 1) batch = 1;
  batch = (batch + grp - 1) / grp * grp;
  const int nbatch = (n + batch - 1) / batch;
  // where every block of the pass will sit: batch k uses ring slot k % d, blocks packed back to back
  uint64_t* bases = static_cast<uint64_t*>(malloc(sizeof(uint64_t) * (size_t)(n > 0 ? n : 1)));
  if (bases == nullptr) return (int)cudaErrorMemoryAllocation;
  for (int k = 0; k < nbatch; ++k) {
    size_t off = 0;
    for (int i = k * batch; i < n && i < (k + 1) * batch; ++i) {
      const int64_t p0 = blk_nnz_host[2 * order_host[i]], p1 = blk_nnz_host[2 * order_host[i] + 1];
      bases[i] = (uint64_t)(uintptr_t)(static_cast<uint32_t*>(stage[k % d]) + off);
      off += (size_t)(p1 - p0) * words;
    }
  }
  cudaError_t e = cudaMemcpyAsync(stage_base_dev, bases, sizeof(uint64_t) * (size_t)n, cudaMemcpyHostToDevice, compute);
  if (e == cudaSuccess) e = cudaStreamSynchronize(compute);  // pageable source: make sure it is consumed before free()
  if (e != cudaSuccess) { free(bases); return (int)e; }
  // One cudaMemcpyAsync per block (46 GB/s for 1.3 MB copies, measured).  A staging kernel that reads
  // the pinned memory through its device mapping, one launch per batch, was tried and is slower
  // (16.7 ms per pass against 11.3 ms).
  auto issue = [&](int k) -> cudaError_t {
    const int s = k % d;
    cudaStream_t cs = h->copy[k & 1];
    cudaError_t e2 = cudaStreamWaitEvent(cs, h->vacant[s], 0);  // no-op until the slot was used once
    if (e2 != cudaSuccess) return e2;
    const int first = k * batch;
    const int count = n - first < batch ? n - first : batch;
    for (int i = first; i < first + count; ++i) {
      const int64_t p0 = blk_nnz_host[2 * order_host[i]], p1 = blk_nnz_host[2 * order_host[i] + 1];
      if (p1 <= p0) continue;
      const size_t bytes = (size_t)(p1 - p0) * words * 4;
      e2 = cudaMemcpyAsync(reinterpret_cast<void*>((uintptr_t)bases[i]), host_pack + (size_t)p0 * words, bytes,
                           cudaMemcpyHostToDevice, cs);
      if (e2 != cudaSuccess) return e2;
      if (h2d_bytes) *h2d_bytes += bytes;
    }
    return cudaEventRecord(h->ready[s], cs);
  };
  for (int k = 0; k < d - 1 && k < nbatch && e == cudaSuccess; ++k) e = issue(k);
  for (int k = 0; k < nbatch && e == cudaSuccess; ++k) {
    if (k + d - 1 < nbatch && (e = issue(k + d - 1)) != cudaSuccess) break;
    const int s = k % d;
    if ((e = cudaStreamWaitEvent(compute, h->ready[s], 0)) != cudaSuccess) break;
    DarlinWorker w = *Wk; DarlinPeers p = *P; DarlinServer sv = *S; DarlinSched q = *Q0; DarlinHyper hy = *H;
    const int first = k * batch;
    const int count = n - first < batch ? n - first : batch;
    // batch is a multiple of the synchronisation group, so `first / grp` groups ran before this launch
    q.order = Q0->order + first;
    q.nblk = count;
    q.group = grp;
    q.seq0 = Q0->seq0 + (uint64_t)(first / grp);
    q.bar0 = Q0->bar0 + (uint64_t)(first / grp);
    q.stage_base = stage_base_dev + first;
    if (first > 0) {   // the group that ran last before this launch: the last `grp` blocks of the previous batch
      q.prev = Q0->order + first - grp;
      q.nprev = grp;
    }
    w.vals = has_vals ? reinterpret_cast<const float*>(stage[s]) : nullptr;  // only null / non-null matters
    void* args[] = {&w, &p, &sv, &q, &hy};
    e = cudaLaunchCooperativeKernel((void*)darlin_pass_kernel, dim3(grid), dim3(512), args, 0, compute);
    if (e != cudaSuccess) break;
    if (launches) ++*launches;
    e = cudaEventRecord(h->vacant[s], compute);
  }
  free(bases);
  return (int)e;
}

static inline int dgrid(int64_t n) {
  int64_t b = (n + 255) / 256;
  if (b < 1) b = 1;
  if (b > 148 * 8) b = 148 * 8;
  return (int)b;
}
int psb_darlin_grad_local(const DarlinWorker* Wk, int64_t lc0, int64_t lc1, void* gu_local, int64_t nnz_hint,
                          cudaStream_t s) {
  k_darlin_grad_local<<<dgrid(nnz_hint), 256, 0, s>>>(*Wk, lc0, lc1, (float2*)gu_local);
  return (int)cudaGetLastError();
}
int psb_darlin_update_weight(const DarlinPeers* P, const DarlinServer* S, const DarlinHyper* H, int64_t s0, int64_t s1,
                             cudaStream_t s) {
  k_darlin_update_weight<<<dgrid(s1 - s0), 256, 0, s>>>(*P, *S, *H, s0, s1);
  return (int)cudaGetLastError();
}
int psb_darlin_apply_pull(const DarlinWorker* Wk, const DarlinHyper* H, int64_t lc0, int64_t lc1, const float* w_new,
                          cudaStream_t s) {
  k_darlin_apply_pull<<<dgrid(lc1 - lc0), 256, 0, s>>>(*Wk, *H, lc0, lc1, w_new);
  return (int)cudaGetLastError();
}
int psb_darlin_update_margin(const DarlinWorker* Wk, int64_t lc0, int64_t lc1, int64_t nnz_hint, cudaStream_t s) {
  k_darlin_update_margin<<<dgrid(nnz_hint), 256, 0, s>>>(*Wk, lc0, lc1);
  return (int)cudaGetLastError();
}
int psb_darlin_margin_init(const DarlinWorker* Wk, int64_t nnz, cudaStream_t s) {
  k_darlin_margin_init<<<dgrid(nnz), 256, 0, s>>>(*Wk);
  return (int)cudaGetLastError();
}

}  // extern "C"
