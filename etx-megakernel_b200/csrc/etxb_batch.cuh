// Batched decode (several sequences per step) inside the persistent kernel: the tiles that take more than one activation
// column per weight read.
//
// What they take over from the reference: the column-batched dense GEMV (`dsl_gemv_rows_nb`, etx/ops/gemv.py:40-73,
// 176-289: NB activation columns served from one weight read, column b at ptr + b * stride) and whole-layer request
// batching (examples/vllm_llm/model.py:194-211: dense nodes batched, attention per sequence, top-k one column per
// wave, expert tasks per (request, slot)).  The reference stops at one column per expert task and notes the union
// de-duplication as the further step; here the expert tiles are EXPERT-GROUPED: a routing tile builds, per expert, the
// list of (sequence, slot) pairs that selected it, and an expert's rows are read once for all of its tokens.
//
// With several tokens per weight row the product is a real (rows x K) . (K x tokens) contraction, so these tiles run on
// the tensor cores: mma.sync m16n8k16 with 16 weight rows as the A operand loaded straight from global memory (16 bytes
// per thread and row, streamed past L1) and up to 8 tokens as the B operand from shared memory, fp32 accumulation,
// partial tiles of the K slices added in slice order (reproducible).  More than 8 tokens are served in passes of 8
// over a block of at most 128 rows: the block's weights come from HBM once and from L2 for the later passes.  They do
// not use the weight ring (the producer warp skips them): that ring stages whole rows for one activation vector.
// Measured on B200 for sizing: a tcgen05.mma (cta_group::1, kind::f16) costs 156 clocks whatever its shape, so with the
// weight rows of a task as its N operand it only pays from about 128 rows per task up (26 bytes/clock/SM at N = 128,
// where HBM needs 22.5); the 14 .. 42 rows a projection leaves per SM run faster on this path.
#pragma once
#include "etxb_gemv.cuh"
#include "etxb_gemv_nb.cuh"

namespace etxb {

#define ETXB_NBC 8                     // tokens per pass (the n of m16n8k16)
#define ETXB_NB_ROWS 128               // weight rows per block
#define ETXB_NBX_BYTES 40960           // shared memory for the tokens' activation vectors of a pass
#define ETXB_NBP_OFF 40960             // partial tiles: 32 units x 128 floats
#define ETXB_NBP_UNITS 32
#define ETXB_NBR_OFF 57344             // result tiles: 2 x [128 rows][8 tokens] floats

// tokens a pass can hold for rows of K elements (their vectors, 64 bytes apart in the banks, must fit ETXB_NBX_BYTES)
__device__ __forceinline__ int nb_cols_per_pass(int K) { return min(ETXB_NBC, ETXB_NBX_BYTES / (K * 2 + ETXB_NB_PAD)); }

// res[q * 8 + n] = W_row(q) . x_n for q < nrows (<= 128), n < 8 (columns >= ncols give 0).  rowptr(q): address of row q.
// xs: the tokens' vectors in shared memory, `xstride` bytes apart.  All consumer threads call; ends with a barrier.
template <typename RowPtr>
__device__ __forceinline__ void nb_block(RowPtr rowptr, int nrows, int K, const unsigned char* xsm, int xstride, int ncols, float* part, float* res) {
  const int tid = tidx(), lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int nblk = (nrows + 15) >> 4, steps = (K + 31) >> 5;       // blocks of 16 rows; k32 steps per row
  int ks = 1;                                                      // K slices per block: enough units for two per warp
  while (nblk * ks < 2 * ETXB_CONSUMER_WARPS && steps / (ks * 2) >= 8 && nblk * ks * 2 <= ETXB_NBP_UNITS) ks *= 2;
  const unsigned char* xs = xsm + (size_t)g * xstride + 16 * t;
  for (int u = warp; u < nblk * ks; u += ETXB_CONSUMER_WARPS) {
    const int b = u / ks, s = u - b * ks;
    const unsigned char* wa = rowptr(min(16 * b + g, nrows - 1)) + 16 * t;       // rows past the block repeat its last row
    const unsigned char* wb = rowptr(min(16 * b + g + 8, nrows - 1)) + 16 * t;
    const int s0 = s * steps / ks, s1 = (s + 1) * steps / ks;
    float da[4] = {0.f, 0.f, 0.f, 0.f}, db[4] = {0.f, 0.f, 0.f, 0.f};
    constexpr int U = 8;                                           // k32 steps in flight: 16 independent 16-byte loads per thread
    for (int k = s0; k < s1; k += U) {
      uint4 va[U], vb[U];
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const bool in = k + j < s1 && 32 * (k + j) + 8 * t < K;    // K % 8 == 0: a 16-byte piece is all inside or all outside
        va[j] = in ? ld_stream(wa + 64 * (k + j)) : make_uint4(0u, 0u, 0u, 0u);
        vb[j] = in ? ld_stream(wb + 64 * (k + j)) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < U; ++j) {
        const bool in = k + j < s1 && 32 * (k + j) + 8 * t < K;
        const uint4 x = in && g < ncols ? *(const uint4*)(xs + 64 * (k + j)) : make_uint4(0u, 0u, 0u, 0u);
        mma_bf16_16x8x16(da, va[j].x, vb[j].x, va[j].y, vb[j].y, x.x, x.y);
        mma_bf16_16x8x16(db, va[j].z, vb[j].z, va[j].w, vb[j].w, x.z, x.w);
      }
    }
    float* p = part + (size_t)u * 128;                             // D[row g][token 2t, 2t + 1] in (0, 1), D[row g + 8][...] in (2, 3)
    p[g * 8 + 2 * t] = __fadd_rn(da[0], db[0]); p[g * 8 + 2 * t + 1] = __fadd_rn(da[1], db[1]);
    p[(g + 8) * 8 + 2 * t] = __fadd_rn(da[2], db[2]); p[(g + 8) * 8 + 2 * t + 1] = __fadd_rn(da[3], db[3]);
  }
  csync();
  for (int i = tid; i < nrows * ETXB_NBC; i += ETXB_CONSUMERS) {     // slices added in slice order
    const int q = i >> 3, n = i & 7;
    const float* p = part + (size_t)((q >> 4) * ks) * 128 + (q & 15) * 8 + n;
    float v = p[0];
    for (int s = 1; s < ks; ++s) v = __fadd_rn(v, p[(size_t)s * 128]);
    res[i] = v;
  }
  csync();
}

// `nc` token vectors of K bf16 values -> shared memory; vector n comes from src(n).  Ends with a barrier.
template <typename Src>
__device__ __forceinline__ void nb_stage_x(Src src, int nc, int K, unsigned char* xsm, int xstride) {
  const int nv = K >> 3;
  for (int i = tidx(); i < nc * nv; i += ETXB_CONSUMERS) {
    const int n = i / nv, v = i - n * nv;
    *(uint4*)(xsm + (size_t)n * xstride + 16 * v) = ld_act16((const __nv_bfloat16*)src(n) + 8 * v);
  }
  csync();
}

// ---------------------------------------------------------------------------------------------- norm of one column
// Task blk = column b of the batch: z = bf16(resid_in[b] + the R rows of column b added one by one in bf16 in ascending
// id order), x[b] = rmsnorm(z) * ln, resid_out[b] = z.  The GEMV block's fields with the column strides of the
// reference's batched form: x + b * sx, rows + b * srows (R rows of K each), resid_in + b * srin, resid_out + b * srout,
// ids + b * R.  For the expert combine R = top-k, rows = the slots' down outputs, ids = the column's expert ids.
__device__ __forceinline__ void tile_norm_col(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks || blk >= d.nb) return;
  const size_t b = (size_t)blk;
  const __nv_bfloat16* rows = d.rows ? (const __nv_bfloat16*)d.rows + b * d.srows : nullptr;
  stage_norm_col<false>(rows, (const __nv_bfloat16*)d.resid_in + b * d.srin, d.resid_out ? (__nv_bfloat16*)d.resid_out + b * d.srout : nullptr,
                        (__nv_bfloat16*)d.x + b * d.sx, d.ln, d.ids ? d.ids + b * d.R : nullptr, d.R, d.K, d.eps, sm.xs, smem_xb(sm), sm.scr, true);
}

// ---------------------------------------------------------------------------------------------- batched dense GEMV
// out[b * sout + r] = bf16(W[r,:] . x[b] (+ bias[r])) for the nb columns b, rows [blk * rpt, ...) of W [M, K].
__device__ __forceinline__ void tile_gemv_nb(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int r0 = blk * d.rpt, r1 = min(d.M, r0 + d.rpt), K = d.K;
  if (r0 >= r1) return;
  unsigned char* xsm = (unsigned char*)sm.xs;
  float* part = (float*)((unsigned char*)sm.xs + ETXB_NBP_OFF);
  float* res = (float*)((unsigned char*)sm.xs + ETXB_NBR_OFF);
  const int xstride = K * 2 + ETXB_NB_PAD, cpp = nb_cols_per_pass(K);
  const unsigned char* W = (const unsigned char*)d.W;
  const __nv_bfloat16* bias = (d.mode & ETXB_MODE_BIAS) ? (const __nv_bfloat16*)d.wts : nullptr;
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  for (int c0 = r0; c0 < r1; c0 += ETXB_NB_ROWS) {                  // a block of rows: from HBM for the first pass, from L2 after
    const int nr = min(ETXB_NB_ROWS, r1 - c0);
    for (int b0 = 0; b0 < d.nb; b0 += cpp) {
      const int nc = min(cpp, d.nb - b0);
      nb_stage_x([&](int n) { return (const __nv_bfloat16*)d.x + (size_t)(b0 + n) * d.sx; }, nc, K, xsm, xstride);
      nb_block([&](int q) { return W + (size_t)(c0 + q) * K * 2; }, nr, K, xsm, xstride, nc, part, res);
      for (int i = tidx(); i < nr * nc; i += ETXB_CONSUMERS) {
        const int n = i / nr, q = i - n * nr;                      // consecutive threads -> consecutive rows of one column
        const float v = res[q * ETXB_NBC + n];
        out[(size_t)(b0 + n) * d.sout + c0 + q] = __float2bfloat16_rn(bias ? __fadd_rn(v, __bfloat162float(bias[c0 + q])) : v);
      }
      csync();
    }
  }
}

// ---------------------------------------------------------------------------------------------- routing of a batch
// One task: softmax top-k of every column (a warp per column), then the per-expert token lists: elist[e][0 .. ecount[e])
// holds the (column << 8 | slot) pairs that selected expert e, in ascending (column, slot) order.  With elist == null the
// grid has one task per column, which only writes its column's ids / wts (the share-scheduled expert tiles build
// their lists themselves).
struct etxb_route_args {
  const void* logits; float* wts; int32_t* ids; int32_t* ecount; int32_t* elist;      // 0..39
  int32_t* active;                                                                    // 40..47: optional counter, += the experts with a non-empty list (the byte ledger of a batched step)
  int32_t E, K, mode, nb, cap, pad;                                                   // 48..71: mode as the top-k tile (bit0 renormalise, 0x100 bf16 weights); cap = entries per expert
  uint32_t grid[3], nblocks;                                                          // 72..87
};
__device__ __forceinline__ void tile_route(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_route_args& d = *(const etxb_route_args*)a;
  const int warp = tidx() >> 5, lane = tidx() & 31;
  if (d.elist == nullptr) {
    if (blk < d.nb && warp == 0)
      warp_topk<false>((const __nv_bfloat16*)d.logits + (size_t)blk * d.E, d.E, d.K, (d.mode & 0xff) == 1, (d.mode & ETXB_MODE_BF16_WTS) != 0,
                       d.ids + (size_t)blk * d.K, d.wts + (size_t)blk * d.K, nullptr);
    return;
  }
  if (blk != 0) return;
  int32_t* sids = (int32_t*)sm.xs;                                 // [nb][K]
  float* swts = sm.xs + 2048;
  for (int b = warp; b < d.nb; b += ETXB_CONSUMER_WARPS) {
    warp_topk<false>((const __nv_bfloat16*)d.logits + (size_t)b * d.E, d.E, d.K, (d.mode & 0xff) == 1, (d.mode & ETXB_MODE_BF16_WTS) != 0,
                     sids + b * d.K, swts + b * d.K, nullptr);
    if (lane < d.K) { d.ids[b * d.K + lane] = sids[b * d.K + lane]; d.wts[b * d.K + lane] = swts[b * d.K + lane]; }
  }
  csync();
  for (int e = tidx(); e < d.E; e += ETXB_CONSUMERS) {
    int cnt = 0;
    for (int i = 0; i < d.nb * d.K; ++i)
      if (sids[i] == e && cnt < d.cap) d.elist[(size_t)e * d.cap + cnt++] = ((i / d.K) << 8) | (i % d.K);
    d.ecount[e] = cnt;
    if (cnt > 0 && d.active != nullptr) atomicAdd(d.active, 1);
  }
}

// ---------------------------------------------------------------------------------------------- expert-grouped gate+up / down
// The GEMV block's fields, read this way: W, estride, M, K, rpt, tpe as in the one-token tiles; task blk = expert
// blk / tpe, row chunk blk % tpe; `rows` = elist, `resid_in` = ecount, nb = cap (entries per expert), R = top-k;
// gate+up: x[b * sx ..] the columns' normed vectors, out = act [nb][R][M]; down: x = act [nb][R][K], wts [nb][R] the
// routing weights, out = y [nb][R][M].
struct GroupTask { int e, r0, nr, cnt; const int32_t* list; };
__device__ __forceinline__ GroupTask group_task(const etxb_gemv_args& d, int blk) {
  GroupTask t;
  t.e = blk / d.tpe; t.r0 = (blk - t.e * d.tpe) * d.rpt; t.nr = min(d.M, t.r0 + d.rpt) - t.r0;
  t.cnt = blk < (int)d.nblocks ? min(__ldcg((const int32_t*)d.resid_in + t.e), d.nb) : 0;
  t.list = (const int32_t*)d.rows + (size_t)t.e * d.nb;
  return t;
}

__device__ __forceinline__ void tile_moe_up_g(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  const GroupTask t = group_task(d, blk);
  if (t.cnt <= 0 || t.nr <= 0) return;
  unsigned char* xsm = (unsigned char*)sm.xs;
  float* part = (float*)((unsigned char*)sm.xs + ETXB_NBP_OFF);
  float* rg = (float*)((unsigned char*)sm.xs + ETXB_NBR_OFF);
  float* ru = rg + ETXB_NB_ROWS * ETXB_NBC;
  int32_t* ent = (int32_t*)(sm.scr + 96);
  const int K = d.K, xstride = K * 2 + ETXB_NB_PAD, cpp = nb_cols_per_pass(K);
  const unsigned char* We = (const unsigned char*)d.W + (size_t)t.e * d.estride * 2;
  for (int c0 = 0; c0 < t.nr; c0 += ETXB_NB_ROWS) {
    const int nr = min(ETXB_NB_ROWS, t.nr - c0);
    for (int p0 = 0; p0 < t.cnt; p0 += cpp) {
      const int nc = min(cpp, t.cnt - p0);
      if (tidx() < nc) ent[tidx()] = __ldcg(t.list + p0 + tidx());
      csync();
      nb_stage_x([&](int n) { return (const __nv_bfloat16*)d.x + (size_t)(ent[n] >> 8) * d.sx; }, nc, K, xsm, xstride);
      nb_block([&](int q) { return We + (size_t)(t.r0 + c0 + q) * K * 2; }, nr, K, xsm, xstride, nc, part, rg);          // gate rows
      nb_block([&](int q) { return We + (size_t)(d.M + t.r0 + c0 + q) * K * 2; }, nr, K, xsm, xstride, nc, part, ru);  // up rows follow the M gate rows
      for (int i = tidx(); i < nr * nc; i += ETXB_CONSUMERS) {
        const int n = i / nr, q = i - n * nr, b = ent[n] >> 8, s = ent[n] & 0xff;
        const float gv = bfr(rg[q * ETXB_NBC + n]), uv = bfr(ru[q * ETXB_NBC + n]);
        ((__nv_bfloat16*)d.out)[((size_t)b * d.R + s) * d.M + t.r0 + c0 + q] = __float2bfloat16_rn(__fmul_rn(bfr(silu_f(gv)), uv));
      }
      csync();
    }
  }
}

__device__ __forceinline__ void tile_moe_down_g(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  const GroupTask t = group_task(d, blk);
  if (t.cnt <= 0 || t.nr <= 0) return;
  unsigned char* xsm = (unsigned char*)sm.xs;
  float* part = (float*)((unsigned char*)sm.xs + ETXB_NBP_OFF);
  float* res = (float*)((unsigned char*)sm.xs + ETXB_NBR_OFF);
  int32_t* ent = (int32_t*)(sm.scr + 96);
  float* wt = sm.scr + 112;
  const int K = d.K, xstride = K * 2 + ETXB_NB_PAD, cpp = nb_cols_per_pass(K);
  const unsigned char* We = (const unsigned char*)d.W + (size_t)t.e * d.estride * 2;
  for (int c0 = 0; c0 < t.nr; c0 += ETXB_NB_ROWS) {
    const int nr = min(ETXB_NB_ROWS, t.nr - c0);
    for (int p0 = 0; p0 < t.cnt; p0 += cpp) {
      const int nc = min(cpp, t.cnt - p0);
      if (tidx() < nc) {
        const int en = __ldcg(t.list + p0 + tidx());
        ent[tidx()] = en;
        wt[tidx()] = d.wts ? __ldcg(d.wts + (size_t)(en >> 8) * d.R + (en & 0xff)) : 1.f;
      }
      csync();
      nb_stage_x([&](int n) { return (const __nv_bfloat16*)d.x + ((size_t)(ent[n] >> 8) * d.R + (ent[n] & 0xff)) * K; }, nc, K, xsm, xstride);
      nb_block([&](int q) { return We + (size_t)(t.r0 + c0 + q) * K * 2; }, nr, K, xsm, xstride, nc, part, res);
      for (int i = tidx(); i < nr * nc; i += ETXB_CONSUMERS) {
        const int n = i / nr, q = i - n * nr, b = ent[n] >> 8, s = ent[n] & 0xff;
        const float y = bfr(res[q * ETXB_NBC + n]);
        ((__nv_bfloat16*)d.out)[((size_t)b * d.R + s) * d.M + t.r0 + c0 + q] = __float2bfloat16_rn(d.wts ? bfr(__fmul_rn(y, wt[n])) : y);
      }
      csync();
    }
  }
}

// ---------------------------------------------------------------------------------------------- per-column prologue
// Columns of a batched step: token_in / token_out are [step][nb]; every column is at the step's position; column b owns
// the cache slots [b * slot_span, (b + 1) * slot_span) of the shared block pool.
// `zero`: optional, ETXB_SPLITK_COUNTERS int32 counters that column 0's prologue task clears (the arrival counters of the
// split-K dense grids: they return to a multiple of the split in every completed step, and an abandoned step must not
// leave them off one).
#define ETXB_SPLITK_COUNTERS 768
struct etxb_batch_args { int32_t nb, slot_span; int32_t* zero; uint32_t grid[3], nblocks; };
__device__ __forceinline__ void tile_prologue_nb(const unsigned char* a, int b, const etxb_stepv& S) {
  const etxb_batch_args& d = *(const etxb_batch_args*)a;
  if (b >= d.nb) return;
  const int t = S.tok;
  if (tidx() == 0) {
    if (S.token_time && b == 0) S.token_time[2 * t] = globaltimer();
    S.positions[b] = S.pos; S.seq_lens[b] = S.pos + 1; S.slot_mapping[b] = (long long)b * d.slot_span + S.pos;
  }
  if (b == 0 && d.zero != nullptr)
    for (int i = tidx(); i < ETXB_SPLITK_COUNTERS; i += ETXB_CONSUMERS) d.zero[i] = 0;
  const int id = __ldcg(S.token_in + (size_t)t * d.nb + b);
  const uint4* src = (const uint4*)((const __nv_bfloat16*)S.embed + (size_t)id * S.H);
  uint4* dst = (uint4*)((__nv_bfloat16*)S.resid + (size_t)b * S.H);
  for (int i = tidx(); i < S.H / 8; i += ETXB_CONSUMERS) dst[i] = __ldg(src + i);
}

}  // namespace etxb
