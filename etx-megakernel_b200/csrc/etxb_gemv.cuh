// bf16 streaming GEMV family of the B200 megakernel: plain / norm-folded projections (QKV, O, router, lm_head),
// MoE gate+up with the SiLU*mul epilogue, MoE down with the routing-weight epilogue, and the softmax top-k.
//
// Function of the reference these tiles take over (same argument block, same task -> row mapping):
//   dsl_gemv / dsl_gemv_fold      etx/ops/gemv.py:816-840   (+ norm fold dsl_stage_norm_at, gemv.py:552-700)
//   dsl_moe_up[_fold]             etx/ops/gemv.py:841-911
//   dsl_moe_down[_fold]           etx/ops/gemv.py:912-953
//   dsl_topk / dsl_topk_lds       etx/ops/topk.py:35-156, etx/ops/gemv.py:712-749
// Rounding points are those of the reference's CPU numerical path (examples/llm/ref_numpy.py:105-158): every
// materialised vector is rounded to bf16, RMSNorm rounds twice, SiLU is rounded before the product, the routing
// weight is a bf16 value, expert outputs are accumulated in bf16 in ascending expert id.
//
// Weight streaming.  The weight rows of a task are one or two contiguous byte ranges.  The CTA's producer warp walks
// the task queue AHEAD of the consumer warps and copies those ranges, whole rows at a time, into a ring of
// ETXB_NSTAGE x 24 KB shared-memory stages with bulk asynchronous copies (cp.async.bulk, the TMA engine; completion
// on an mbarrier per stage).  Weights depend on no event (expert weights: only on the routing), so the stream keeps
// running while the consumers wait for their activations: HBM stays busy across phase boundaries.  The consumer
// warps take the stages in order; warp w owns the rows q with q % 16 == w, reads 16-byte weight and activation
// vectors from shared memory, accumulates in fp32 in a fixed order (lane-strided, then xor butterfly), and hands the
// row result to the tile's epilogue.
#pragma once
#include "etxb_prims.cuh"

namespace etxb {

struct Smem {
  float* xs;                 // general region (ETXB_GEN_BYTES): fp32 scratch, bf16 activations, row results
  float* scr;                // ETXB_SCR_FLOATS of reduction / routing scratch
  unsigned char* ring;       // ETXB_NSTAGE stages
  uint64_t* full;            // [ETXB_NSTAGE] stage filled (transaction bytes landed)
  uint64_t* empty;           // [ETXB_NSTAGE] stage drained by all consumer warps
  int32_t* prod;             // producer-warp scratch: 16 ids + 16 weights
  const unsigned long long* deadline;
  int32_t* ctrl;
  int* stop;                 // CTA-local: a wait inside a body gave up (the body's results are not to be announced)
  uint64_t* tr;              // 8 stamps of the running task when tracing, else null (slots 4..7 are in-body marks)
  struct TcShared* tc;       // state of the tensor-core tiles of a batched step (null where the kernel has none)
  uint32_t epoch;            // the step (sharded sessions: the flag of this step's exchanged words derives from it)
  int cur;                   // the running task's index in the queue order (reported when a wait gives up)
};
// in-body time stamp k (0..3) of the running task; thread 0 only, no-op unless tracing
__device__ __forceinline__ void mark(const Smem& sm, int k) { if (sm.tr != nullptr && tidx() == 0) sm.tr[4 + k] = globaltimer(); }
__device__ __forceinline__ __nv_bfloat16* smem_xb(const Smem& sm) { return (__nv_bfloat16*)((unsigned char*)sm.xs + ETXB_XB_OFF); }
__device__ __forceinline__ float* smem_g(const Smem& sm) { return (float*)((unsigned char*)sm.xs + ETXB_G_OFF); }

// Bounded mbarrier wait: true when the phase completed; false when the step is being abandoned (another thread gave
// up, the host aborted, or the deadline passed -- then this thread records it).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const Smem& sm, int where) {
  uint32_t n = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++n & 255u) == 0) {
      if (ld_relaxed(sm.ctrl) != 0) { *(volatile int*)sm.stop = 1; return false; }
      if ((n & 4095u) == 0 && globaltimer() > *sm.deadline) {
        if (atomicOr(sm.ctrl, ETXB_CTRL_TIMEOUT) == 0) { sm.ctrl[1] = where; sm.ctrl[2] = -1; sm.ctrl[3] = (int32_t)parity; sm.ctrl[4] = -1; }
        *(volatile int*)sm.stop = 1;
        return false;
      }
    }
  }
  return true;
}

// ---------------------------------------------------------------------------------------------- what a task streams
// The weight rows of a task: `nranges` contiguous ranges of `n` rows each (row_bytes per row), taken range by range.
//   plain GEMV   one range: rows [r0, r0 + n) of W
//   MoE gate+up  per expert slot of the task: the gate rows, then the up rows (2 * spt ranges)
//   MoE down     per expert slot of the task: rows [r0, r0 + n) of that expert's W2 (spt ranges)
struct GemvTask {
  int nranges, n, row_bytes, r0, group, spt;
};
// ---------------------------------------------------------------------------------------------- top-k
// softmax over E bf16 logits (fp32), K rounds of argmax with the lower index winning ties, optional renormalisation
// over the selected weights (numpy's summation order for <= 16 values), optional bf16 rounding of the weights.
// One warp (all 32 lanes call); E <= 256, K <= 16.  ids / wts / tei may point to shared or global memory.
template <int NK>
__device__ __forceinline__ void warp_topk_n(const void* logits, int E, int K, bool renorm, bool bf16w,
                                            int32_t* ids, float* wts, int32_t* tei) {
  const int lane = tidx() & 31;
  float p[NK];
  float m = -INFINITY;
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int e = lane + 32 * k;
    p[k] = e < E ? ld_bf(logits, e) : -INFINITY;
    m = fmaxf(m, p[k]);
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < NK; ++k) { p[k] = (lane + 32 * k < E) ? expf(__fsub_rn(p[k], m)) : 0.f; s = __fadd_rn(s, p[k]); }
  s = warp_sum(s);
  // Selection keys: a probability is a non-negative float, so its bit pattern orders like the value; + 1 keeps a valid
  // zero probability above "no candidate" (0).  A candidate is the 64-bit pair (key, ~expert): the larger pair is the
  // larger probability or, on a tie, the lower expert.  Each lane sorts its NK candidates once (descending), so a
  // round only looks at the lane's head: two warp reductions (redux.sync) find the winner, whose lane pops its head.
  // A NaN anywhere in the row makes the sum, and so every probability, NaN: no candidate is valid then and every round
  // writes id 0x7fffffff with weight -1 (the behaviour the reference's model pins for its wave path,
  // etx/ops/topk_key32.py:122-147; the expert tiles map such an id to expert 0 before they form an address).
  unsigned long long c[NK];
#pragma unroll
  for (int k = 0; k < NK; ++k) {
    const int e = lane + 32 * k;
    const float pq = __fdiv_rn(p[k], s);
    const uint32_t key = (e < E && pq == pq) ? __float_as_uint(pq) + 1u : 0u;
    c[k] = ((unsigned long long)key << 32) | (uint32_t)(0xffffffffu - (uint32_t)e);
  }
#pragma unroll
  for (int i = 1; i < NK; ++i)                                      // insertion network: c[0] >= c[1] >= ...
#pragma unroll
    for (int j = i; j > 0; --j) {
      const unsigned long long hi = c[j - 1] > c[j] ? c[j - 1] : c[j], lo = c[j - 1] > c[j] ? c[j] : c[j - 1];
      c[j - 1] = hi; c[j] = lo;
    }
  float myw = 0.f; int myid = 0x7fffffff;
#pragma unroll 1
  for (int t = 0; t < K; ++t) {
    const uint32_t hk = (uint32_t)(c[0] >> 32), hi_ = (uint32_t)c[0];
    const uint32_t top = __reduce_max_sync(0xffffffffu, hk);
    const uint32_t wl = __reduce_max_sync(0xffffffffu, hk == top ? hi_ : 0u);
    const bool any = top != 0u;
    if (any && hk == top && hi_ == wl) {                            // the winner's lane pops its head
#pragma unroll
      for (int k = 0; k + 1 < NK; ++k) c[k] = c[k + 1];
      c[NK - 1] = 0ull;
    }
    if (lane == t) { myw = any ? __uint_as_float(top - 1u) : -1.f; myid = any ? (int)(0xffffffffu - wl) : 0x7fffffff; }
  }
  if (renorm) {
    // numpy's order for the sum of the K selected weights: K < 8 left to right, else 8 accumulators + tree + tail
    float tot;
    if (K < 8) {
      tot = 0.f;
#pragma unroll 1
      for (int t = 0; t < K; ++t) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, myw, t));
    } else {
      float r = lane < 8 ? myw : 0.f;                              // accumulator j = lane j
      const float second = __shfl_sync(0xffffffffu, myw, (lane & 7) + 8);
      if (K >= 16 && lane < 8) r = __fadd_rn(r, second);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, o));
      tot = __shfl_sync(0xffffffffu, r, 0);
#pragma unroll 1
      for (int t = (K >= 16 ? 16 : 8); t < K; ++t) tot = __fadd_rn(tot, __shfl_sync(0xffffffffu, myw, t));
    }
    myw = __fdiv_rn(myw, tot);
  }
  if (bf16w) myw = bfr(myw);
  if (lane < K) { ids[lane] = myid; wts[lane] = myw; if (tei) tei[lane] = lane; }
  __syncwarp();
}

// LEAN: the form the host picks when every top-k of the plan has E <= 128 (no code for more experts in that kernel).
template <bool LEAN>
__device__ __noinline__ void warp_topk(const void* logits, int E, int K, bool renorm, bool bf16w,
                                       int32_t* ids, float* wts, int32_t* tei) {
  if (LEAN || E <= 128) warp_topk_n<4>(logits, E, K, renorm, bf16w, ids, wts, tei);
  else warp_topk_n<8>(logits, E, K, renorm, bf16w, ids, wts, tei);
}

__device__ __forceinline__ void tile_topk(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_topk_args& d = *(const etxb_topk_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int nb = (d.nbsv & 0xff) ? (d.nbsv & 0xff) : 1, sv = d.nbsv >> 8;
  const int w = tidx() >> 5;
  if (w >= nb) return;
  warp_topk<false>((const __nv_bfloat16*)d.logits + (size_t)w * d.E, d.E, d.K, (d.mode & 0xff) == 1, (d.mode & ETXB_MODE_BF16_WTS) != 0,
            d.ids + (size_t)w * sv, d.wts + (size_t)w * sv, d.tei ? d.tei + (size_t)w * sv : nullptr);
}

// Decode task `blk` of a GEMV-family tile (pure arithmetic on the argument block).  Slots per task: mode bits 16..23
// (0 = 1): task blk covers slots [group * spt, (group + 1) * spt), group = blk / tpe, row chunk j = blk % tpe.
__device__ __forceinline__ GemvTask gemv_task(int body, const etxb_gemv_args& d, int blk) {
  GemvTask t;
  t.nranges = 0; t.n = 0; t.row_bytes = d.K * 2; t.r0 = 0; t.group = 0; t.spt = 1;
  if (blk >= (int)d.nblocks) return t;
  if (body == 3) {
    const int r0 = blk * d.rpt, r1 = min(d.M, r0 + d.rpt);
    if (r0 < r1) { t.nranges = 1; t.n = r1 - r0; t.r0 = r0; }
    return t;
  }
  const int spt = ((d.mode >> 16) & 0xff) ? ((d.mode >> 16) & 0xff) : 1;
  const int group = blk / d.tpe, j = blk - group * d.tpe;
  const int r0 = j * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 < r1) { t.nranges = (body == 4 ? 2 : 1) * spt; t.n = r1 - r0; t.r0 = r0; t.group = group; t.spt = spt; }
  return t;
}

// Expert ids (and routing weights) of the task's slots into `lids` / `lwts` (indexed by global slot).  One warp, all
// lanes call.  Top-k fold: recomputed from the logits; else read from the ids / wts buffers; no ids: expert 0.
// SH: the kernel variant supports always-on (shared) experts -- mode bits 24..27: ns experts that every token uses, stored
// after the E routed ones; they take the last ns slots with weight 1, the top-k picks the others.  (A template parameter
// and not a run-time branch: the lean kernels of the models without shared experts measured 1.4 % slower with it.)
template <bool LEAN, bool SH = !LEAN>
__device__ __forceinline__ void gemv_routing(const etxb_gemv_args& d, int32_t* lids, float* lwts) {
  const int fold = d.mode & 0xff, lane = tidx() & 31;
  if (fold >= 2) {
    if constexpr (SH) {
      const int ns = (d.mode >> 24) & 0xf;
      warp_topk<LEAN>(d.logits, d.E, d.R - ns, fold == 3, (d.mode & ETXB_MODE_BF16_WTS) != 0, lids, lwts, nullptr);
      if (ns > 0) {
        if (lane < ns) { lids[d.R - ns + lane] = d.E + lane; lwts[d.R - ns + lane] = 1.f; }
        __syncwarp();
      }
    } else {
      warp_topk<LEAN>(d.logits, d.E, d.R, fold == 3, (d.mode & ETXB_MODE_BF16_WTS) != 0, lids, lwts, nullptr);
    }
  } else {
    if (lane < 16) {
      lids[lane] = (d.ids && lane < d.R) ? __ldcg(d.ids + lane) : 0;
      lwts[lane] = (d.wts && lane < d.R) ? __ldcg(d.wts + lane) : 1.f;
    }
    __syncwarp();
  }
}

template <bool SH = true>
__device__ __forceinline__ const unsigned char* gemv_range_base(int body, const etxb_gemv_args& d, const GemvTask& t, int i, const int32_t* lids) {
  if (body == 3) return (const unsigned char*)d.W + (size_t)t.r0 * t.row_bytes;
  const int slot = t.group * t.spt + (body == 4 ? i >> 1 : i);
  int e = lids[slot];
  if (d.E > 0 && (unsigned)e >= (unsigned)(d.E + (SH ? ((d.mode >> 24) & 0xf) : 0))) e = 0;   // "no candidate" (a NaN row): never an address
  const unsigned char* We = (const unsigned char*)d.W + (size_t)e * d.estride * 2;
  const int row = t.r0 + ((body == 4 && (i & 1)) ? d.M : 0);        // up rows follow the M gate rows
  return We + (size_t)row * t.row_bytes;
}

// ---------------------------------------------------------------------------------------------- producer side
// Issue the bulk copies of one task.  One warp; lane 0 issues.  n = running stage counter of this CTA.
// ptr: the task's trace row when tracing (slot 7 <- time the first stage was issued, slot 6 <- the last), else null.
template <bool SH = true>
__device__ __forceinline__ bool produce_task(int body, const etxb_gemv_args& d, const GemvTask& t, const int32_t* lids, uint32_t& n,
                                             const Smem& sm, int where, uint64_t* ptr = nullptr) {
  const int total = t.nranges * t.n;
  if (total <= 0) return true;
  const int rps = ETXB_STAGE_BYTES / t.row_bytes;
  bool ok = true;
  if (rps < 1 || t.row_bytes <= 0) {                               // a row longer than a stage: refused by the host; never loop on it
    if ((tidx() & 31) == 0) { atomicOr(sm.ctrl, ETXB_CTRL_BADTASK); *(volatile int*)sm.stop = 1; }
    return false;
  }
  if ((tidx() & 31) == 0) {
    const uint64_t pol = l2_policy_evict_first();
    for (int q0 = 0; q0 < total && ok; q0 += rps) {
      const uint32_t st = n % ETXB_NSTAGE, par = (n / ETXB_NSTAGE) & 1;
      ok = mbar_wait(sm.empty + st, par ^ 1, sm, where);           // a fresh barrier passes the first round
      if (!ok) break;
      const int nr = min(rps, total - q0);
      unsigned char* dst = sm.ring + (size_t)st * ETXB_STAGE_BYTES;
      mbar_expect_tx(sm.full + st, (uint32_t)(nr * t.row_bytes));
      int q = q0;
      while (q < q0 + nr) {                                        // one copy per piece of a range that falls into this stage
        const int rg = q / t.n, r = q - rg * t.n;
        const int cnt = min(t.n - r, q0 + nr - q);
        bulk_g2s_hint(dst + (size_t)(q - q0) * t.row_bytes, gemv_range_base<SH>(body, d, t, rg, lids) + (size_t)r * t.row_bytes,
                      (uint32_t)(cnt * t.row_bytes), sm.full + st, pol);
        q += cnt;
      }
      if (ptr != nullptr) { if (q0 == 0) ptr[7] = globaltimer(); ptr[6] = globaltimer(); }
      ++n;
    }
  }
  ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
  n = __shfl_sync(0xffffffffu, n, 0);
  return ok;
}

// ---------------------------------------------------------------------------------------------- consumer side
__device__ __forceinline__ float dot8(const uint4 w, const uint4 x, float a) {
  a = __fmaf_rn(bf_lo(w.x), bf_lo(x.x), a); a = __fmaf_rn(bf_hi(w.x), bf_hi(x.x), a);
  a = __fmaf_rn(bf_lo(w.y), bf_lo(x.y), a); a = __fmaf_rn(bf_hi(w.y), bf_hi(x.y), a);
  a = __fmaf_rn(bf_lo(w.z), bf_lo(x.z), a); a = __fmaf_rn(bf_hi(w.z), bf_hi(x.z), a);
  a = __fmaf_rn(bf_lo(w.w), bf_lo(x.w), a); a = __fmaf_rn(bf_hi(w.w), bf_hi(x.w), a);
  return a;
}

// Consume the stages of one task: row q (0 .. total-1, range q / rows_per_range) . its activation vector -> epi(q, value),
// called by lane 0 of the owning warp.  Range i uses the vector at xb + i * xstride (xstride = 0: one vector for all).
// Every consumer warp walks every stage (so the stage counter stays in step) and arrives on its `empty` barrier.
// (Measured and not kept: the packed fma.rn.f32x2 form of the inner loop, +1.3 % step time; a lane's share of the
// activations held in registers as fp32 pairs, which spills at the 96 registers this kernel gets, +45 %; a ring of
// 7 stages instead of 6, +0.6 %; the short tasks (a projection's 14 .. 42 rows per SM, resident in the ring before they
// are needed) multiplied with mma.sync m16n8k16 from the ring, the activation vector as column 0 of B, +25 % -- the
// legacy tensor path is slow on this part, and with one bulk copy per row padded for conflict-free fragment reads +60 %,
// because a bulk copy costs the copy engine about 0.3 us whatever its size.  This loop runs at about 21 bytes of
// weights per clock and SM, HBM delivers 22.5.)
template <typename Epi>
__device__ __forceinline__ void consume_task(int total, int rows_per_range, int row_bytes, uint32_t& n, const Smem& sm, const __nv_bfloat16* xb,
                                             int xstride, int where, Epi epi) {
  if (total <= 0) return;
  const int lane = tidx() & 31, cw = tidx() >> 5;
  const int rps = row_bytes > 0 ? ETXB_STAGE_BYTES / row_bytes : 0, nvec = row_bytes >> 4;
  if (rps < 1) return;                                             // (the producer raised the bad-task bit)
  bool alive = true;
  for (int q0 = 0; q0 < total; q0 += rps) {
    const uint32_t st = n % ETXB_NSTAGE, par = (n / ETXB_NSTAGE) & 1;
    ++n;
    if (alive) alive = mbar_wait(sm.full + st, par, sm, where);
    if (!alive) continue;                                          // step abandoned: keep counting, touch nothing
    if (q0 == 0) mark(sm, 1);
    const int nr = min(rps, total - q0);
    const unsigned char* stage = sm.ring + (size_t)st * ETXB_STAGE_BYTES;
    for (int j = (cw - q0) & (ETXB_CONSUMER_WARPS - 1); j < nr; j += ETXB_CONSUMER_WARPS) {
      const uint4* wv = (const uint4*)(stage + (size_t)j * row_bytes);
      const uint4* xv = (const uint4*)(xb + (size_t)((q0 + j) / rows_per_range) * xstride);
      float acc = 0.f;
#pragma unroll 8
      for (int v = lane; v < nvec; v += 32) acc = dot8(wv[v], xv[v], acc);
      acc = warp_sum(acc);
      if (lane == 0) epi(q0 + j, acc);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(sm.empty + st);
  }
}

// ---------------------------------------------------------------------------------------------- activation staging
// K bf16 values (written by other CTAs) -> shared memory, K % 8 == 0.
__device__ __forceinline__ void stage_xb(const void* x, int K, __nv_bfloat16* xb) {
  const int nv = K >> 3;
  for (int i = tidx(); i < nv; i += ETXB_CONSUMERS) ((uint4*)xb)[i] = ld_act16((const __nv_bfloat16*)x + 8 * i);
  csync();
}

// Norm fold: z = bf16(resid_in + acc), acc = the R rows added one by one in bf16 in ascending id order (R == 1: the row
// itself; rows == null: z = resid_in), then x = bf16(ln * bf16(z * r)), r = 1 / sqrt(mean(z^2) + eps) with the mean summed
// in numpy's order.  x goes to shared memory (xb); `store`: this task also writes resid_out (z) and xout (x).  K <= 8192.
// LEAN: the form the host picks when every norm fold of the plan adds at most one row (R <= 1): no ordering, no row loop.
// fl != 0 (sharded model): `rows` holds R rows of K flagged words published by the ranks (row r by rank r); every word is
// re-read until its flag is `fl` (bounded like every wait: on a give-up the step is abandoned through sm.stop), then the
// rows are added in rank order -- every rank adds the same values in the same order and gets the same bits.
// XCH: the kernel variant of a sharded session; without it the flagged form is compiled out (the single-GPU kernels
// carry none of the exchange code: it cost them about 5 % when it was a run-time branch).
template <bool LEAN, bool XCH = false>
__device__ __noinline__ void stage_norm_col(const void* rows, const void* rin, void* rout, void* xout, const void* ln,
                                            const int32_t* ids, int R, int K, float eps, float* xf, __nv_bfloat16* xb, float* scr, bool store,
                                            uint32_t fl = 0u, const Smem* smp = nullptr) {
  int* order = (int*)(scr + 64);
  if (!LEAN && R > 1 && (!XCH || fl == 0u)) {
    if (R <= 32) {
      // one load per lane, the other ids by shuffle (no loop of R loads from L2 in front of the rows)
      if (tidx() < 32) {
        const int lane = tidx();
        const int mine = (ids && lane < R) ? __ldcg(ids + lane) : 0;
        int rank = ids ? 0 : lane;
        if (ids)
          for (int j = 0; j < R; ++j) {
            const int o = __shfl_sync(0xffffffffu, mine, j);
            rank += (o < mine) || (o == mine && j < lane);
          }
        if (lane < R) order[rank] = lane;
      }
    } else if (tidx() < R) {
      int rank = tidx();
      if (ids) {
        const int mine = __ldcg(ids + tidx());
        rank = 0;
        for (int j = 0; j < R; ++j) {
          const int o = __ldcg(ids + j);
          rank += (o < mine) || (o == mine && j < tidx());
        }
      }
      order[rank] = tidx();
    }
    csync();
  }
  const int nv = K >> 3;
  uint4 lw[2];                                                     // norm weights of this thread's (at most two) vectors, fetched with the rows
#pragma unroll 1
  for (int i = tidx(), it = 0; i < nv; i += ETXB_CONSUMERS, ++it) {
    float z[8];
    if (it < 2) lw[it] = __ldg((const uint4*)((const __nv_bfloat16*)ln + 8 * i));
    const uint4 ri = ld_act16((const __nv_bfloat16*)rin + 8 * i);
    const float rf[8] = {bf_lo(ri.x), bf_hi(ri.x), bf_lo(ri.y), bf_hi(ri.y), bf_lo(ri.z), bf_hi(ri.z), bf_lo(ri.w), bf_hi(ri.w)};
    if (rows == nullptr || R == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) z[j] = rf[j];
    } else if (XCH && fl != 0u) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
#pragma unroll 1
      for (int s0 = 0; s0 < R; ++s0) {
        const uint32_t* src = (const uint32_t*)rows + (size_t)s0 * K + 8 * i;
        uint4 a, b;
        uint32_t spins = 0;
        for (;;) {
          a = ld_volatile16(src); b = ld_volatile16(src + 4);
          if ((((a.x ^ fl) | (a.y ^ fl) | (a.z ^ fl) | (a.w ^ fl) | (b.x ^ fl) | (b.y ^ fl) | (b.z ^ fl) | (b.w ^ fl)) >> 16) == 0u) break;
          if ((++spins & 63u) == 0) {
            if (ld_relaxed(smp->ctrl) != 0) { *(volatile int*)smp->stop = 1; break; }
            if ((spins & 1023u) == 0 && globaltimer() > *smp->deadline) {
              if (atomicOr(smp->ctrl, ETXB_CTRL_TIMEOUT) == 0) { smp->ctrl[1] = smp->cur; smp->ctrl[2] = -2 - s0; smp->ctrl[3] = (int32_t)(a.x >> 16); smp->ctrl[4] = (int32_t)(fl >> 16); }
              *(volatile int*)smp->stop = 1;
              break;
            }
            __nanosleep(32);
          }
        }
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = bfr(__fadd_rn(acc[j], __uint_as_float(w[j] << 16)));
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) z[j] = bfr(__fadd_rn(rf[j], acc[j]));
    } else if (LEAN) {
      const uint4 rv = ld_act16((const __nv_bfloat16*)rows + 8 * i);
      const float v[8] = {bf_lo(rv.x), bf_hi(rv.x), bf_lo(rv.y), bf_hi(rv.y), bf_lo(rv.z), bf_hi(rv.z), bf_lo(rv.w), bf_hi(rv.w)};
#pragma unroll
      for (int j = 0; j < 8; ++j) z[j] = bfr(__fadd_rn(rf[j], v[j]));      // bf16(0 + row) = row: the one-row case of the loop below
    } else {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int s0 = 0; s0 < R; s0 += 8) {                       // up to 8 rows in flight, added in order
        uint4 rv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (s0 + u < R) {
            const int row = R > 1 ? order[s0 + u] : 0;
            rv[u] = ld_act16((const __nv_bfloat16*)rows + (size_t)row * K + 8 * i);
          }
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (s0 + u < R) {
            const float v[8] = {bf_lo(rv[u].x), bf_hi(rv[u].x), bf_lo(rv[u].y), bf_hi(rv[u].y),
                                bf_lo(rv[u].z), bf_hi(rv[u].z), bf_lo(rv[u].w), bf_hi(rv[u].w)};
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = bfr(__fadd_rn(acc[j], v[j]));
          }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) z[j] = bfr(__fadd_rn(rf[j], acc[j]));
    }
    *(float4*)(xf + 8 * i) = make_float4(z[0], z[1], z[2], z[3]);
    *(float4*)(xf + 8 * i + 4) = make_float4(z[4], z[5], z[6], z[7]);
    if (store && rout != nullptr)
      *(uint4*)((__nv_bfloat16*)rout + 8 * i) = make_uint4(pack_bf(z[0], z[1]), pack_bf(z[2], z[3]), pack_bf(z[4], z[5]), pack_bf(z[6], z[7]));
  }
  csync();
  const float ss = sumsq_numpy_order(xf, K, scr);
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps)));
#pragma unroll 1
  for (int i = tidx(), it = 0; i < nv; i += ETXB_CONSUMERS, ++it) {
    const uint4 w = it == 0 ? lw[0] : lw[1];
    const float wf[8] = {bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y), bf_lo(w.z), bf_hi(w.z), bf_lo(w.w), bf_hi(w.w)};
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = bfr(__fmul_rn(wf[j], bfr(__fmul_rn(xf[8 * i + j], r))));
    const uint4 o = make_uint4(pack_bf(v[0], v[1]), pack_bf(v[2], v[3]), pack_bf(v[4], v[5]), pack_bf(v[6], v[7]));
    ((uint4*)xb)[i] = o;
    if (store && xout != nullptr) *(uint4*)((__nv_bfloat16*)xout + 8 * i) = o;
  }
  csync();
}

// ---------------------------------------------------------------------------------------------- plain / folded GEMV
template <bool LEAN, bool XCH = false>
__device__ __forceinline__ void tile_gemv(const unsigned char* a, int blk, const Smem& sm, uint32_t& n, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  const GemvTask t = gemv_task(3, d, blk);
  if (t.n <= 0) return;
  const int r0 = t.r0;
  __nv_bfloat16* xb = smem_xb(sm);
  if ((d.mode & 0xff) == ETXB_MODE_NORM)
    stage_norm_col<LEAN, XCH>(d.rows, d.resid_in, d.resid_out, (void*)d.x, d.ln, d.ids, d.R, d.K, d.eps, sm.xs, xb, sm.scr, blk == 0,
                              (XCH && (d.mode & ETXB_MODE_FLAGGED)) ? row_flag(sm.epoch) : 0u, &sm);
  else
    stage_xb(d.x, d.K, xb);
  const __nv_bfloat16* bias = (d.mode & ETXB_MODE_BIAS) ? (const __nv_bfloat16*)d.wts : nullptr;
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  mark(sm, 0);
  consume_task(t.n, t.n, t.row_bytes, n, sm, xb, 0, where, [&](int q, float v) {
    out[r0 + q] = __float2bfloat16_rn(bias ? __fadd_rn(v, __bfloat162float(bias[r0 + q])) : v);
  });
}

// ---------------------------------------------------------------------------------------------- MoE gate+up
// task blk: expert slots [group * spt, ...), row chunk j = blk % tpe; expert e = ids[slot] (no ids and no fold: expert
// 0, the dense SwiGLU MLP); act[slot][r] = bf16(bf16(silu(bf16 g)) * bf16 u), g = W_e[r,:].x, u = W_e[M + r,:].x.
template <bool LEAN, bool XCH = false, bool SH = !LEAN>
__device__ __forceinline__ void tile_moe_up(const unsigned char* a, int blk, const Smem& sm, uint32_t& n, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  const GemvTask t = gemv_task(4, d, blk);
  if (t.n <= 0) return;
  int32_t* lids = (int32_t*)(sm.scr + 96); float* lwts = sm.scr + 112;
  const int fold = d.mode & 0xff;
  if (tidx() < 32) {
    if (fold >= 2) {
      gemv_routing<LEAN, SH>(d, lids, lwts);
      if (blk - t.group * d.tpe == 0 && tidx() < t.spt) {           // the group's first chunk publishes its slots' routing
        const int sl = t.group * t.spt + tidx();
        if (d.ids) ((int32_t*)d.ids)[sl] = lids[sl];
        if (d.wts) ((float*)d.wts)[sl] = lwts[sl];
      }
    }
  }
  __nv_bfloat16* xb = smem_xb(sm);
  if (fold == ETXB_MODE_NORM)                                      // dense MLP: the post-attention norm folded in
    stage_norm_col<LEAN, XCH>(d.rows, d.resid_in, d.resid_out, (void*)d.x, d.ln, nullptr, d.R, d.K, d.eps, sm.xs, xb, sm.scr, blk == 0,
                              (XCH && (d.mode & ETXB_MODE_FLAGGED)) ? row_flag(sm.epoch) : 0u, &sm);
  else
    stage_xb(d.x, d.K, xb);
  float* g = smem_g(sm);                                           // per slot: n gate results, then n up results
  const int rows = t.n;
  mark(sm, 0);
  consume_task(t.nranges * rows, rows, t.row_bytes, n, sm, xb, 0, where, [&](int q, float v) { g[q] = bfr(v); });
  csync();
  mark(sm, 2);
  for (int i = tidx(); i < t.spt * rows; i += ETXB_CONSUMERS) {
    const int s = i / rows, r = i - s * rows;
    __nv_bfloat16* act = (__nv_bfloat16*)d.out + (size_t)(t.group * t.spt + s) * d.M;
    act[t.r0 + r] = __float2bfloat16_rn(__fmul_rn(bfr(silu_f(g[2 * s * rows + r])), g[(2 * s + 1) * rows + r]));
  }
}

// ---------------------------------------------------------------------------------------------- MoE down
// y[slot][r] = bf16(bf16(W_e[r,:] . act_slot) * wts[slot]) (no weights, the dense MLP: bf16(W_e[r,:] . act)).
// Plain form: out[slot][r] = y.  Summed form (mode bit ETXB_MODE_SUM_SLOTS, the task covers every slot): out[r] = the
// y of all slots added one by one in bf16 in ascending expert id -- the expert combine of the CPU path
// (examples/llm/ref_numpy.py:142-148), which the reference leaves to the next layer's norm fold.
template <bool LEAN, bool SH = !LEAN>
__device__ __forceinline__ void tile_moe_down(const unsigned char* a, int blk, const Smem& sm, uint32_t& n, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  const GemvTask t = gemv_task(5, d, blk);
  if (t.n <= 0) return;
  int32_t* lids = (int32_t*)(sm.scr + 96); float* lwts = sm.scr + 112;
  const int fold = d.mode & 0xff;
  const bool scaled = fold >= 2 || d.wts != nullptr;
  if (tidx() < 32) {
    if (fold >= 2 && (d.mode & ETXB_MODE_ROUTE_READY) && d.ids != nullptr && d.wts != nullptr) {
      if (tidx() < 16) {
        lids[tidx()] = tidx() < d.R ? __ldcg(d.ids + tidx()) : 0;
        lwts[tidx()] = tidx() < d.R ? __ldcg(d.wts + tidx()) : 1.f;
      }
      __syncwarp();
    } else {
      gemv_routing<LEAN, SH>(d, lids, lwts);
    }
    // the slots in ascending expert id, for the summed form: known as soon as the routing is, so it is worked out here,
    // under the weight stream, and not after it (the barrier that follows the stream publishes it to the other warps)
    if ((d.mode & ETXB_MODE_SUM_SLOTS) && tidx() < t.spt) {
      const int mine = lids[t.group * t.spt + tidx()];
      int rank = 0;
      for (int j = 0; j < t.spt; ++j) {
        const int o = lids[t.group * t.spt + j];
        rank += (o < mine) || (o == mine && j < tidx());
      }
      ((int*)(sm.scr + 64))[rank] = tidx();
    }
  }
  __nv_bfloat16* xb = smem_xb(sm);
  const int K = d.K, rows = t.n;
  const int* order = (const int*)(sm.scr + 64);
  for (int i = tidx(); i < t.spt * (K >> 3); i += ETXB_CONSUMERS) {          // the task's slots' activation vectors
    const int s = i / (K >> 3), v = i - s * (K >> 3);
    ((uint4*)xb)[i] = ld_act16((const __nv_bfloat16*)d.x + (size_t)(t.group * t.spt + s) * K + 8 * v);
  }
  csync();
  float* g = smem_g(sm);
  const bool sum = (d.mode & ETXB_MODE_SUM_SLOTS) != 0;
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  mark(sm, 0);
  consume_task(t.nranges * rows, rows, t.row_bytes, n, sm, xb, K, where, [&](int q, float v) {
    const int s = q / rows, r = q - s * rows, sl = t.group * t.spt + s;
    const float y = bfr(v);
    const float ys = scaled ? bfr(__fmul_rn(y, lwts[sl])) : y;
    if (sum) g[q] = ys;
    else out[(size_t)sl * d.M + t.r0 + r] = __float2bfloat16_rn(ys);
  });
  if (!sum) return;
  csync();
  mark(sm, 2);
  for (int r = tidx(); r < rows; r += ETXB_CONSUMERS) {
    float acc = 0.f;
    for (int k = 0; k < t.spt; ++k) acc = bfr(__fadd_rn(acc, g[order[k] * rows + r]));
    out[t.r0 + r] = __float2bfloat16_rn(acc);
  }
}

}  // namespace etxb
