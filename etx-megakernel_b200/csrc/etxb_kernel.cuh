// The persistent kernel: one CTA per SM walks its static task queue; per task it waits for the task's events
// (acquire, bounded), runs the tile body, drains its stores and arrives on the out events (release).
//
// Takes over the generated kernel of the reference: worker loop etx/codegen/kernel.py:517-572, the three-phase
// etx_run_task kernel.py:341-468, and the native prologue / argmax tiles examples/vllm_llm/vl_tiles.hip:31-89.
#pragma once
#include "etxb_attn.cuh"
#include "etxb_attn_gq.cuh"
#include "etxb_batch.cuh"
#include "etxb_tc.cuh"
#include "etxb_mla.cuh"
#include "etxb_gemv.cuh"
#include "etxb_prims.cuh"

namespace etxb {

// resid <- embedding row of token_in[t] (nrep copies), positions / seq_lens / slot_mapping <- pos (identity block table)
__device__ __forceinline__ void tile_prologue(const etxb_stepv& S) {
  const int t = S.tok;
  if (tidx() == 0) {
    if (S.token_time) S.token_time[2 * t] = globaltimer();
    S.positions[0] = S.pos; S.seq_lens[0] = S.pos + 1; S.slot_mapping[0] = S.pos;
  }
  const int id = __ldcg(S.token_in + t);
  const uint4* src = (const uint4*)((const __nv_bfloat16*)S.embed + (size_t)id * S.H);
  uint4* dst = (uint4*)S.resid;
  const int n8 = S.H / 8;
  for (int i = tidx(); i < n8 * S.nrep; i += ETXB_CONSUMERS) dst[i] = __ldg(src + i % n8);
}

// greedy sampling: first maximum of the bf16 logits (ties -> lower index, like argmax over float32)
// Sharded lm_head (p.xargmax != 0): the logits are this rank's V of ranks x V, so the rank's (maximum, global index) goes
// into its slot of every rank's argmax block as two 8-byte (payload, step flag) stores -- each atomic, so no fence --
// and the token is the best of all ranks' pairs, ties to the lower index: the same on every rank.
__device__ __forceinline__ void st_volatile8(void* p, uint32_t a, uint32_t b) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_volatile8(const void* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
__device__ __noinline__ void argmax_exchange(const etxb_params& p, const Smem& sm, float& bv, int& bi) {
  const uint32_t fl = row_flag(p.epoch);
  bi += p.rank * p.step.V;
  const int q_self = p.rank;
  for (int q = 0; q <= p.n_peers; ++q) {                            // peers in xpeer order (ranks without this one), then this rank
    unsigned char* base = q < p.n_peers ? p.xpeer[q] : p.xbase;
    unsigned char* slot = base + p.xargmax + 16 * (size_t)q_self;
    st_volatile8(slot, __float_as_uint(bv), fl);
    st_volatile8(slot + 8, (uint32_t)bi, fl);
  }
  for (int r = 0; r <= p.n_peers; ++r) {
    if (r == p.rank) continue;
    const unsigned char* slot = p.xbase + p.xargmax + 16 * (size_t)r;
    uint2 a, b;
    uint32_t spins = 0;
    for (;;) {
      a = ld_volatile8(slot); b = ld_volatile8(slot + 8);
      if (a.y == fl && b.y == fl) break;
      if ((++spins & 63u) == 0) {
        if (ld_relaxed(sm.ctrl) != 0) { *(volatile int*)sm.stop = 1; return; }
        if ((spins & 1023u) == 0 && globaltimer() > *sm.deadline) {
          if (atomicOr(sm.ctrl, ETXB_CTRL_TIMEOUT) == 0) { sm.ctrl[1] = sm.cur; sm.ctrl[2] = -100 - r; sm.ctrl[3] = (int32_t)(a.y >> 16); sm.ctrl[4] = (int32_t)(fl >> 16); }
          *(volatile int*)sm.stop = 1;
          return;
        }
        __nanosleep(32);
      }
    }
    const float ov = __uint_as_float(a.x);
    const int oi = (int)b.x;
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
}

// col / ncols: column `col` of a batched step (logits [ncols][V], token_in / token_out [step][ncols]); (0, 1) otherwise.
template <bool XCH>
__device__ __forceinline__ void tile_argmax(const etxb_params& p, const Smem& sm, int col = 0, int ncols = 1) {
  const etxb_stepv& S = p.step;
  float bv = -INFINITY; int bi = 0x7fffffff;
  const uint4* lg4 = (const uint4*)((const __nv_bfloat16*)S.logits + (size_t)col * S.V);
  const int n4 = S.V / 8;
  auto scan = [&](const uint4 w, int base) {
    const uint32_t u[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float lo = bf_lo(u[k]), hi = bf_hi(u[k]);
      if (lo > bv) { bv = lo; bi = base + 2 * k; }
      if (hi > bv) { bv = hi; bi = base + 2 * k + 1; }
    }
  };
  int j = tidx();
  const int B = ETXB_CONSUMERS;
  for (; j + 3 * B < n4; j += 4 * B) {
    const uint4 a0 = ld_act16(lg4 + j), a1 = ld_act16(lg4 + j + B), a2 = ld_act16(lg4 + j + 2 * B), a3 = ld_act16(lg4 + j + 3 * B);
    scan(a0, 8 * j); scan(a1, 8 * (j + B)); scan(a2, 8 * (j + 2 * B)); scan(a3, 8 * (j + 3 * B));
  }
  for (; j < n4; j += B) scan(ld_act16(lg4 + j), 8 * j);
  for (int i = 8 * n4 + tidx(); i < S.V; i += B) {
    const float v = ld_bf(lg4, i);
    if (v > bv) { bv = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
  }
  float* sv = sm.scr; int* si = (int*)(sm.scr + 32);
  if ((tidx() & 31) == 0) { sv[tidx() >> 5] = bv; si[tidx() >> 5] = bi; }
  csync();
  if (tidx() == 0) {
    for (int w = 1; w < ETXB_NWARPS; ++w)
      if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) { bv = sv[w]; bi = si[w]; }
    if constexpr (XCH) { if (p.n_peers > 0 && p.xargmax != 0u) argmax_exchange(p, sm, bv, bi); }
    const int t = S.tok;
    S.token_out[(size_t)t * ncols + col] = bi;
    if (S.write_next) S.token_in[(size_t)(t + 1) * ncols + col] = bi;
    if (S.token_time && col == ncols - 1) S.token_time[2 * t + 1] = globaltimer();
  }
}

// protocol demo (etx/operators/splitk_sum.py:10-33): parts[i][j] = sum of chunk j of row i; out[i] = sum_j parts[i][j]
__device__ __forceinline__ void tile_splitk_part(const unsigned char* a, int i, int j, const Smem& sm) {
  const etxb_splitk_args& d = *(const etxb_splitk_args*)a;
  const int w = d.cols / d.chunks;
  float s = 0.f;
  for (int c = tidx(); c < w; c += ETXB_CONSUMERS) s += __ldcg(d.in + (size_t)i * d.cols + j * w + c);
  s = block_sum(s, sm.scr);
  if (tidx() == 0) d.parts[i * d.chunks + j] = s;
}
__device__ __forceinline__ void tile_splitk_sum(const unsigned char* a, int i) {
  const etxb_splitk_args& d = *(const etxb_splitk_args*)a;
  if (tidx() == 0) {
    float s = 0.f;
    for (int j = 0; j < d.chunks; ++j) s += __ldcg(d.parts + i * d.chunks + j);
    d.out[i] = s;
  }
}

// A task's context in shared memory: its record and a copy of its argument block.  The last consumer warp fetches them
// with asynchronous copies (cp.async) while earlier bodies run -- the record two tasks ahead, the argument block one
// task ahead (its address is in the record) -- and only waits for them at the end of a body, so the chain task ->
// arguments -> data costs the tiles no dependent global round trip and the fetch itself is off the critical path.
struct TaskCtx {
  etxb_rec r;
  unsigned char args[ETXB_CTX_BYTES - 96];
};
static_assert(sizeof(etxb_rec) == 96 && sizeof(TaskCtx) == ETXB_CTX_BYTES, "context slot layout");

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// one warp: lanes 0..5 fetch the record of task `rec_task`, lanes 8..19 the argument block of task `arg_task` (whose
// record must already be in its slot); -1 skips either.  Asynchronous: cp_async_wait_all() completes them.
__device__ __forceinline__ void fetch_ctx(const etxb_params& p, TaskCtx* ctx, int q0, int rec_task, int arg_task) {
  const int lane = tidx() & 31;
  if (rec_task >= 0 && lane < 6) cp_async16((unsigned char*)&ctx[(rec_task - q0) & (ETXB_CTX_SLOTS - 1)].r + 16 * lane,
                                            (const unsigned char*)(p.recs + rec_task) + 16 * lane);
  if (arg_task >= 0 && lane >= 8 && lane < 20) {
    TaskCtx* c = ctx + ((arg_task - q0) & (ETXB_CTX_SLOTS - 1));
    cp_async16(c->args + 16 * (lane - 8), (const unsigned char*)c->r.args + 16 * (lane - 8));
  }
}

// Run the body of the task whose context is `c` on the consumer warps.
// GQV: the kernel variant.  0 = every tile.  1, 2, 4, 8 = the lean decode kernel: only the tiles of a fused decode step
// (prologue, argmax, the GEMV family with norm folds of at most one row and top-k folds over at most 128 experts, the
// grouped attention tile with GQV q heads per task); ETXB_VARIANT_MLA = the lean kernel of a latent-attention model (the
// same GEMV family with the latent-attention tile in place of the grouped one).  The host picks it from the plan (select_variant): the full
// kernel is 550 KB of code, of which a decode step uses a fraction scattered through it, and the step runs about 10 %
// faster from the 150 KB kernel (instruction fetch).
// XCH: the variants a sharded session launches -- the same bodies plus the exchange code (flagged-row folds of R = ranks
// rows, row publishing after the body, the argmax exchange); compiled out of the others.
#define ETXB_VARIANT_MLA 16
template <int GQV, bool XCH>
__device__ __forceinline__ void run_body(const etxb_params& p, const TaskCtx* c, int cur, const Smem& sm, uint32_t& n) {
  const unsigned char* args = c->args;
  const int c0 = c->r.c0, c1 = c->r.c1;
  constexpr bool LEAN = GQV != 0;
  constexpr bool SH = GQV == 0 || GQV == ETXB_VARIANT_MLA;         // always-on (shared) experts: the full kernel and the latent-attention variant
  constexpr bool BATCH = GQV == 0;                                 // the tiles of a batched step: full kernel only (a lean kernel of just these
                                                                   // tiles was measured: 1852 against 1873 tok/s at 32 sequences -- a batched task
                                                                   // runs long enough in one code region for instruction fetch not to matter)
  // (a body this variant does not hold: the host picks the variant from the plan's bodies, so this is a corrupted record)
#define ETXB_TILE(cond, call) if constexpr (cond) { call; } else { if (tidx() == 0) atomicOr(p.ctrl, ETXB_CTRL_BADTASK); } break
  switch (c->r.body) {
    case 0: break;
    case 1: tile_prologue(p.step); break;
    case 2: tile_argmax<XCH>(p, sm); break;
    case 3: tile_gemv<LEAN, XCH>(args, c0, sm, n, cur); break;
    case 4: tile_moe_up<LEAN, XCH, SH>(args, c0, sm, n, cur); break;
    case 5: tile_moe_down<LEAN, SH>(args, c0, sm, n, cur); break;
    case 12:
      if constexpr (GQV == ETXB_VARIANT_MLA) { if (tidx() == 0) atomicOr(p.ctrl, ETXB_CTRL_BADTASK); }      // (the latent-attention variant has no GQA tile)
      else if constexpr (LEAN) { if (c0 < (int)((const etxb_attnf_args*)args)->nblocks) attn_gq_impl<GQV ? GQV : 1>(*(const etxb_attnf_args*)args, c0, sm, p.step); }
      else tile_attn_any(args, c0, sm, p.step);
      break;
    case 6: ETXB_TILE(!LEAN, tile_topk(args, c0, sm));
    case 7: ETXB_TILE(!LEAN, tile_attnprep(args, c0, sm, p.step));
    case 8: ETXB_TILE(!LEAN, tile_attn(args, c0, sm, p.step));
    case 9: ETXB_TILE(!LEAN, tile_attn_reduce(args, c0, sm, p.step));
    case 10: ETXB_TILE(!LEAN, tile_splitk_part(args, c0, c1, sm));
    case 11: ETXB_TILE(!LEAN, tile_splitk_sum(args, c0));
    // batched decode (several columns per step): full kernel only
    case 13: ETXB_TILE(BATCH, tile_norm_col(args, c0, sm));
    case 14: ETXB_TILE(!LEAN, tile_gemv_nb(args, c0, sm));
    case 15: ETXB_TILE(BATCH, tile_route(args, c0, sm));
    case 16: ETXB_TILE(!LEAN, tile_moe_up_g(args, c0, sm));
    case 17: ETXB_TILE(!LEAN, tile_moe_down_g(args, c0, sm));
    case 18: ETXB_TILE(BATCH, tile_prologue_nb(args, c0, p.step));
    case 19: ETXB_TILE(BATCH, (c0 < ((const etxb_batch_args*)args)->nb ? tile_argmax<false>(p, sm, c0, ((const etxb_batch_args*)args)->nb) : (void)0));
    case 20: ETXB_TILE(BATCH && !XCH, tile_gemv_tc(args, c0, sm, *sm.tc, cur));
    case 21: ETXB_TILE(BATCH && !XCH, tile_moe_up_tc(args, c0, sm, *sm.tc, cur));
    case 22: ETXB_TILE(BATCH && !XCH, tile_moe_down_tc(args, c0, sm, *sm.tc, cur));
    case 23: ETXB_TILE(!LEAN || GQV == ETXB_VARIANT_MLA, tile_mla_attn(args, c0, sm, p.step));
    default:
      if (tidx() == 0) atomicOr(p.ctrl, ETXB_CTRL_BADTASK);
      break;
  }
#undef ETXB_TILE
}

// The producer warp: walks the same queue ahead of the consumers and streams the weight rows of every GEMV-family
// task into the ring.  It waits only for what the weight ADDRESSES depend on (nothing for static weights, the router's
// event for expert weights), never for the task's activations.
template <bool LEAN, bool SH = !LEAN>
__device__ __forceinline__ void producer_loop(const etxb_params& p, const Smem& sm, int q0, int q1) {
  uint32_t n = 0;
  const int lane = tidx() & 31;
  bool ok = true;
  for (int cur = q0; cur < q1 && ok; ++cur) {
    const etxb_rec* t = p.recs + cur;
    const int body = t->body;
    if (body < 3 || body > 5) continue;
    // the argument block through shared memory, fetched BEFORE the wait below (it depends on no event)
    etxb_gemv_args* pa = (etxb_gemv_args*)(sm.prod + 32);
    if (lane < 20) ((uint64_t*)pa)[lane] = __ldg((const uint64_t*)t->args + lane);
    __syncwarp();
    const int sw = t->stream_word;
    if (sw != -1) {
      int good = 1;
      if (lane == 0) {
        if (sw >= 0) good = wait_event(p, sw, (int32_t)(p.epoch * (uint32_t)p.evcount[sw]), cur, *sm.deadline) ? 1 : 0;
        else
          for (int i = 0; good && i < t->in_n; ++i) {
            const int word = i < 4 ? t->in_word[i] : p.inwords[t->in_off + i];
            good = wait_event(p, word, (int32_t)(p.epoch * (uint32_t)p.evcount[word]), cur, *sm.deadline) ? 1 : 0;
          }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) break;
    } else if (ld_relaxed(p.ctrl) != 0) {
      break;
    }
    const GemvTask gt = gemv_task(body, *pa, t->c0);
    if (gt.n > 0 && body != 3) gemv_routing<LEAN, SH>(*pa, sm.prod, (float*)(sm.prod + 16));
    ok = produce_task<SH>(body, *pa, gt, sm.prod, n, sm, cur, p.trace ? p.trace + 8 * (size_t)t->id : nullptr);
  }
  // Nothing is left in flight on a normal exit (the consumers waited for every stage).  When the step was abandoned,
  // wait (bounded) for the copies already issued before the CTA's shared memory goes away.
  if (ld_relaxed(p.ctrl) != 0 && lane == 0) {
    const uint32_t issued = n < ETXB_NSTAGE ? n : ETXB_NSTAGE;
    for (uint32_t k = 0; k < issued; ++k) {
      const uint32_t m = n - 1 - k, st = m % ETXB_NSTAGE, par = (m / ETXB_NSTAGE) & 1;
      for (int spin = 0; spin < 2000000 && !mbar_try_wait(sm.full + st, par); ++spin) {}
    }
  }
}

template <int GQV, bool XCH = false>
__global__ void __launch_bounds__(ETXB_THREADS, 1) etxb_megakernel(const __grid_constant__ etxb_params p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_stop;
  __shared__ unsigned long long s_deadline;
  __shared__ __align__(8) TcShared s_tc;                           // (used by the full kernel of a batched plan only)
  constexpr bool TC = GQV == 0 && !XCH;
  Smem sm;
  sm.ring = smem_raw;
  sm.xs = (float*)(smem_raw + ETXB_RING_BYTES);
  sm.scr = (float*)(smem_raw + ETXB_RING_BYTES + ETXB_GEN_BYTES);
  sm.full = (uint64_t*)(smem_raw + ETXB_RING_BYTES + ETXB_GEN_BYTES + ETXB_SCR_FLOATS * 4);
  sm.empty = sm.full + ETXB_NSTAGE;
  sm.prod = (int32_t*)(sm.empty + ETXB_NSTAGE);
  sm.deadline = &s_deadline;
  sm.ctrl = p.ctrl;
  sm.stop = &s_stop;
  sm.tr = nullptr;
  sm.tc = &s_tc;
  sm.epoch = p.epoch;
  sm.cur = 0;
  if (threadIdx.x == 0) {
    s_stop = 0;
    s_deadline = globaltimer() + p.timeout_ns;
    for (int i = 0; i < ETXB_NSTAGE; ++i) { mbar_init(sm.full + i, 1); mbar_init(sm.empty + i, ETXB_CONSUMER_WARPS); }
    if constexpr (TC) {
      for (int i = 0; i < ETXB_TC_MAXSTAGE; ++i) { mbar_init(s_tc.full + i, 1); mbar_init(s_tc.empty + i, 1); s_tc.lu[i] = 0; s_tc.mu[i] = 0; }
      for (int i = 0; i < 2; ++i) { mbar_init(s_tc.acc_full + i, 1); mbar_init(s_tc.acc_free + i, 4); s_tc.nfull[i] = 0; s_tc.nfree[i] = 0; }
      s_tc.tmem = 0;
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if ((int)blockIdx.x >= p.n_workers) return;
  const int q0 = p.qbegin[blockIdx.x], q1 = p.qbegin[blockIdx.x + 1];
  if (threadIdx.x >= ETXB_CONSUMERS) {
    producer_loop<GQV != 0, GQV == 0 || GQV == ETXB_VARIANT_MLA>(p, sm, q0, q1);
    return;
  }
  TaskCtx* ctx = (TaskCtx*)(smem_raw + ETXB_RING_BYTES + ETXB_GEN_BYTES + ETXB_SCR_FLOATS * 4 + 512);
  const bool fetcher = threadIdx.x >= ETXB_CONSUMERS - 32;          // the last consumer warp keeps the contexts coming
  if constexpr (TC) {
    // tensor memory for the tensor-core tiles of a batched plan: allocated once per launch by warp 0 (one CTA per SM, so
    // the columns are always there), freed by the same warp after the last task on every path out of the loop below
    if (p.tc_on != 0u && threadIdx.x < 32) tc_alloc(&s_tc.tmem);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  }
  if (fetcher && q0 < q1) {
    fetch_ctx(p, ctx, q0, q0, -1);
    fetch_ctx(p, ctx, q0, q0 + 1 < q1 ? q0 + 1 : -1, -1);
    cp_async_wait_all();
    __syncwarp();
    fetch_ctx(p, ctx, q0, -1, q0);
    cp_async_wait_all();
  }
  csync();
  uint32_t n = 0;                                                  // stages consumed so far (same count the producer keeps)
  for (int cur = q0; cur < q1; ++cur) {
    const TaskCtx* c = ctx + ((cur - q0) & (ETXB_CTX_SLOTS - 1));
    if (threadIdx.x == 0) {
      const int in_n = c->r.in_n;
      if (p.trace) p.trace[8 * (size_t)c->r.id] = globaltimer();
      bool ok = true;                                              // wait_event polls the abort word itself
      for (int i = 0; ok && i < in_n; ++i) {
        int word, cnt;
        if (i < 4) { word = c->r.in_word[i]; cnt = c->r.in_cnt[i]; }
        else { word = p.inwords[c->r.in_off + i]; cnt = p.evcount[word]; }
        ok = wait_event(p, word, (int32_t)(p.epoch * (uint32_t)cnt), cur, s_deadline);
      }
      if (!ok) s_stop = 1;
      if (p.trace) p.trace[8 * (size_t)c->r.id + 1] = globaltimer();
    }
    csync();
    if (s_stop) break;
    if (fetcher) fetch_ctx(p, ctx, q0, cur + 2 < q1 ? cur + 2 : -1, cur + 1 < q1 ? cur + 1 : -1);   // asynchronous
    sm.tr = p.trace ? p.trace + 8 * (size_t)c->r.id : nullptr;
    if constexpr (XCH) sm.cur = cur;
    run_body<GQV, XCH>(p, c, cur, sm, n);
    if (fetcher) cp_async_wait_all();
    csync();                                                       // every consumer thread's stores are issued, the next contexts landed
    // Sharded model: warp 1 publishes the bf16 rows this task wrote as flagged words (value | this step's flag) into the
    // grid's block of every rank's exchange region, its own included -- plain 4-byte stores, over NVLink for the peers.
    // Value and flag travel in one word, so nothing has to be ordered: no fence, no barrier, no remote counter; the
    // arrival below only tells this rank's consumers that the local phase is over, the folds then poll the flags.
    const uint32_t mirror = XCH ? c->r.mirror : 0u;                  // 0 unless the grid is exchanged
    if (XCH && mirror != 0u && s_stop == 0 && (threadIdx.x >> 5) == 1) {   // (an abandoned body publishes nothing)
      const etxb_gemv_args& d = *(const etxb_gemv_args*)c->args;
      const int r0 = (c->r.body == 3 ? c->r.c0 : c->r.c0 % d.tpe) * d.rpt;
      const unsigned short* src = (const unsigned short*)d.out + r0;
      const uint32_t off = mirror & 0x3fffffu, len = mirror >> 22, fl = row_flag(p.epoch);
      for (uint32_t i = threadIdx.x & 31; i < len; i += 32) {
        const uint32_t v = (uint32_t)__ldcg(src + i) | fl;
        for (int q = 0; q < p.n_peers; ++q) st_flagged((uint32_t*)p.xpeer[q] + off + i, v);
        st_flagged((uint32_t*)p.xbase + off + i, v);
      }
    }
    if (threadIdx.x == 0) {
      const int out_n = c->r.out_n, id = c->r.id;
      if (s_stop == 0)                                             // (set when a stage wait gave up inside the body: no arrivals then)
        for (int i = 0; i < out_n; ++i) {                          // release: orders the CTA's stores (seen through the barrier) before the count
          const int word = i < 4 ? c->r.out_word[i] : p.outwords[c->r.out_off + i];
          red_release_add(p.events + (size_t)word * ETXB_EV_STRIDE, 1);
        }
      if (p.trace) { p.trace[8 * (size_t)id + 2] = globaltimer(); p.trace[8 * (size_t)id + 3] = blockIdx.x; }
      if (p.exec_count) atomicAdd(p.exec_count + id, 1);
    }
  }
  if constexpr (TC) {
    if (p.tc_on != 0u) {
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      csync();                                                     // nobody reads an accumulator any more
      if (threadIdx.x < 32) tc_dealloc(s_tc.tmem);
    }
  }
}

}  // namespace etxb
