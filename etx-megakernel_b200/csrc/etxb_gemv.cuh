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
// Streaming: one warp owns a row (or a K segment of a row when a task has fewer rows than warps: split-K),
// every lane keeps up to 8 independent 16-byte non-temporal weight loads in flight (64 KB per SM), fp32 FMA on
// unpacked bf16, xor-butterfly across lanes, K segments added left to right: the summation order is fixed.
#pragma once
#include "etxb_prims.cuh"

namespace etxb {

struct Smem {
  float* xs;       // ETXB_XS_FLOATS staged activations (nb columns, KS floats apart)
  float* scr;      // ETXB_SCRATCH_FLOATS
};

// ---------------------------------------------------------------------------------------------- staging
// nb columns of K bf16 values -> floats in shared memory; column b at xs + b * KS.  K % 8 == 0.
__device__ __forceinline__ void stage_x(const void* x, int K, int sx, int nb, int KS, float* xs) {
  const int nv = K >> 3;
  for (int b = 0; b < nb; ++b) {
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x + (size_t)b * sx;
    float* dst = xs + (size_t)b * KS;
    for (int i = tidx(); i < nv; i += blockDim.x) {
      const uint4 v = ld_act16(xb + 8 * i);
      *(float4*)(dst + 8 * i) = make_float4(bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y));
      *(float4*)(dst + 8 * i + 4) = make_float4(bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w));
    }
  }
  __syncthreads();
}

// Norm fold of one column: z = bf16(resid_in + acc), acc = the R rows added one by one in bf16 in ascending id order
// (R == 1: the row itself; rows == null: z = resid_in), then x = bf16(ln * bf16(z * r)), r = 1 / sqrt(mean(z^2) + eps)
// with the mean summed in numpy's order.  `store`: this task also writes resid_out (z) and xout (x).
__device__ __forceinline__ void stage_norm_col(const void* rows, const void* rin, void* rout, void* xout, const void* ln,
                                               const int32_t* ids, int R, int K, float eps, float* xs, float* scr, bool store) {
  int* order = (int*)(scr + 64);
  if (R > 1) {
    if (tidx() < R) {
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
    __syncthreads();
  }
  const int nv = K >> 3;
  for (int i = tidx(); i < nv; i += blockDim.x) {
    float z[8];
    const uint4 ri = ld_act16((const __nv_bfloat16*)rin + 8 * i);
    const float rf[8] = {bf_lo(ri.x), bf_hi(ri.x), bf_lo(ri.y), bf_hi(ri.y), bf_lo(ri.z), bf_hi(ri.z), bf_lo(ri.w), bf_hi(ri.w)};
    if (rows == nullptr || R == 0) {
#pragma unroll
      for (int j = 0; j < 8; ++j) z[j] = rf[j];
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
    *(float4*)(xs + 8 * i) = make_float4(z[0], z[1], z[2], z[3]);
    *(float4*)(xs + 8 * i + 4) = make_float4(z[4], z[5], z[6], z[7]);
    if (store && rout != nullptr)
      *(uint4*)((__nv_bfloat16*)rout + 8 * i) = make_uint4(pack_bf(z[0], z[1]), pack_bf(z[2], z[3]), pack_bf(z[4], z[5]), pack_bf(z[6], z[7]));
  }
  __syncthreads();
  const float ss = sumsq_numpy_order(xs, K, scr);
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)K), eps)));
  __syncthreads();
  for (int i = tidx(); i < nv; i += blockDim.x) {
    const uint4 w = __ldg((const uint4*)((const __nv_bfloat16*)ln + 8 * i));
    const float wf[8] = {bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y), bf_lo(w.z), bf_hi(w.z), bf_lo(w.w), bf_hi(w.w)};
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = bfr(__fmul_rn(wf[j], bfr(__fmul_rn(xs[8 * i + j], r))));
    *(float4*)(xs + 8 * i) = make_float4(v[0], v[1], v[2], v[3]);
    *(float4*)(xs + 8 * i + 4) = make_float4(v[4], v[5], v[6], v[7]);
    if (store && xout != nullptr)
      *(uint4*)((__nv_bfloat16*)xout + 8 * i) = make_uint4(pack_bf(v[0], v[1]), pack_bf(v[2], v[3]), pack_bf(v[4], v[5]), pack_bf(v[6], v[7]));
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------- the stream
template <int NB>
__device__ __forceinline__ void fma8(const uint4 w, const float* xp, int KS, float* acc) {
  const float wf[8] = {bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y), bf_lo(w.z), bf_hi(w.z), bf_lo(w.w), bf_hi(w.w)};
#pragma unroll
  for (int b = 0; b < NB; ++b) {
    const float4 xa = *(const float4*)(xp + (size_t)b * KS), xb = *(const float4*)(xp + (size_t)b * KS + 4);
    float a = acc[b];
    a = __fmaf_rn(wf[0], xa.x, a); a = __fmaf_rn(wf[1], xa.y, a); a = __fmaf_rn(wf[2], xa.z, a); a = __fmaf_rn(wf[3], xa.w, a);
    a = __fmaf_rn(wf[4], xb.x, a); a = __fmaf_rn(wf[5], xb.y, a); a = __fmaf_rn(wf[6], xb.z, a); a = __fmaf_rn(wf[7], xb.w, a);
    acc[b] = a;
  }
}

// rows q = 0 .. nrows-1 of bf16 weights, row q at rowptr(q), K elements each (K % 8 == 0); activations xs (NB columns,
// KS floats apart).  epi(q, v) is called once per row with the NB dot products by one thread.  part: scratch of at
// least ETXB_NWARPS * NB floats.  All threads of the CTA call; contains __syncthreads().
template <int NB, typename RowPtr, typename Epi>
__device__ __forceinline__ void gemv_rows(int nrows, int K, RowPtr rowptr, const float* xs, int KS, float* part, Epi epi) {
  const int lane = tidx() & 31, warp = tidx() >> 5;
  const int nvec = K >> 3;
  int ks = 1;                                                    // split-K factor: power of two, >= 32 vectors per segment
  while (nrows * ks * 2 <= ETXB_NWARPS && (nvec / (ks * 2)) >= 32) ks *= 2;
  const int segn = (((nvec + ks - 1) / ks) + 31) & ~31;           // vectors per segment, whole lanes-rounds
  const int vpl = segn >> 5;                                      // vectors per lane per segment
  const int units = nrows * ks;
  constexpr int U = NB >= 4 ? 4 : 8;                              // independent 16-byte loads in flight per lane

  if (ks == 1) {
    if (vpl > 4) {
      for (int q = warp; q < nrows; q += ETXB_NWARPS) {
        const __nv_bfloat16* wr = rowptr(q);
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) acc[b] = 0.f;
        for (int v0 = 0; v0 < vpl; v0 += U) {
          uint4 w[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int v = (v0 + u) * 32 + lane;
            if (v0 + u < vpl && v < nvec) w[u] = ld_stream(wr + 8 * v);
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int v = (v0 + u) * 32 + lane;
            if (v0 + u < vpl && v < nvec) fma8<NB>(w[u], xs + 8 * v, KS, acc);
          }
        }
        float out[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) out[b] = warp_sum(acc[b]);
        if (lane == 0) epi(q, out);
      }
    } else {                                                       // short rows: two rows per warp trip, <= 4 vectors each
      for (int q0 = warp * 2; q0 < nrows; q0 += ETXB_NWARPS * 2) {
        const bool two = q0 + 1 < nrows;
        const __nv_bfloat16* wa = rowptr(q0);
        const __nv_bfloat16* wb = two ? rowptr(q0 + 1) : wa;
        uint4 w[2][4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = u * 32 + lane;
          if (u < vpl && v < nvec) { w[0][u] = ld_stream(wa + 8 * v); if (two) w[1][u] = ld_stream(wb + 8 * v); }
        }
        float acc[2][NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) { acc[0][b] = 0.f; acc[1][b] = 0.f; }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int v = u * 32 + lane;
          if (u < vpl && v < nvec) { fma8<NB>(w[0][u], xs + 8 * v, KS, acc[0]); if (two) fma8<NB>(w[1][u], xs + 8 * v, KS, acc[1]); }
        }
        float o0[NB], o1[NB];
#pragma unroll
        for (int b = 0; b < NB; ++b) { o0[b] = warp_sum(acc[0][b]); o1[b] = warp_sum(acc[1][b]); }
        if (lane == 0) { epi(q0, o0); if (two) epi(q0 + 1, o1); }
      }
    }
    return;
  }
  // split-K: unit u = (row, segment); partials to shared memory, summed left to right
  __syncthreads();
  for (int u = warp; u < units; u += ETXB_NWARPS) {
    const int q = u / ks, seg = u - q * ks;
    const __nv_bfloat16* wr = rowptr(q);
    float acc[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) acc[b] = 0.f;
    for (int v0 = 0; v0 < vpl; v0 += U) {
      uint4 w[U];
#pragma unroll
      for (int t = 0; t < U; ++t) {
        const int v = seg * segn + (v0 + t) * 32 + lane;
        if (v0 + t < vpl && v < nvec) w[t] = ld_stream(wr + 8 * v);
      }
#pragma unroll
      for (int t = 0; t < U; ++t) {
        const int v = seg * segn + (v0 + t) * 32 + lane;
        if (v0 + t < vpl && v < nvec) fma8<NB>(w[t], xs + 8 * v, KS, acc);
      }
    }
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      const float s = warp_sum(acc[b]);
      if (lane == 0) part[u * NB + b] = s;
    }
  }
  __syncthreads();
  if (tidx() < nrows) {
    float out[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float s = 0.f;
      for (int seg = 0; seg < ks; ++seg) s = __fadd_rn(s, part[(tidx() * ks + seg) * NB + b]);
      out[b] = s;
    }
    epi(tidx(), out);
  }
}

// ---------------------------------------------------------------------------------------------- top-k
// softmax over E bf16 logits (fp32), K rounds of argmax with the lower index winning ties, optional renormalisation
// over the selected weights (numpy's summation order for <= 16 values), optional bf16 rounding of the weights.
// One warp; E <= 256.  ids / wts / tei may point to shared or global memory; lane t stores result t.
__device__ __forceinline__ void warp_topk(const void* logits, int E, int K, bool renorm, bool bf16w,
                                          int32_t* ids, float* wts, int32_t* tei) {
  const int lane = tidx() & 31;
  float p[8]; bool taken[8];
  float m = -INFINITY;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int e = lane + 32 * k;
    p[k] = e < E ? ld_bf(logits, e) : -INFINITY;
    taken[k] = e >= E;
    m = fmaxf(m, p[k]);
  }
  m = warp_max(m);
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) { p[k] = taken[k] ? 0.f : expf(__fsub_rn(p[k], m)); s = __fadd_rn(s, p[k]); }
  s = warp_sum(s);
#pragma unroll
  for (int k = 0; k < 8; ++k) p[k] = __fdiv_rn(p[k], s);
  float myw = 0.f; int myid = 0x7fffffff;
  for (int t = 0; t < K; ++t) {
    float bv = -1.f; int bi = 0x7fffffff;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (!taken[k] && p[k] > bv) { bv = p[k]; bi = lane + 32 * k; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) taken[k] = taken[k] || (lane + 32 * k == bi);
    if (lane == t) { myw = bv; myid = bi; }
  }
  if (renorm) {
    float sel[16];
    const int n = K < 16 ? K : 16;
    for (int t = 0; t < n; ++t) sel[t] = __shfl_sync(0xffffffffu, myw, t);
    const float tot = sum_small_numpy_order(sel, n);
    myw = __fdiv_rn(myw, tot);
  }
  if (bf16w) myw = bfr(myw);
  if (lane < K) { ids[lane] = myid; wts[lane] = myw; if (tei) tei[lane] = lane; }
}

__device__ __forceinline__ void tile_topk(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_topk_args& d = *(const etxb_topk_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int nb = (d.nbsv & 0xff) ? (d.nbsv & 0xff) : 1, sv = d.nbsv >> 8;
  const int w = tidx() >> 5;
  if (w >= nb) return;
  warp_topk((const __nv_bfloat16*)d.logits + (size_t)w * d.E, d.E, d.K, (d.mode & 0xff) == 1, (d.mode & ETXB_MODE_BF16_WTS) != 0,
            d.ids + (size_t)w * sv, d.wts + (size_t)w * sv, d.tei ? d.tei + (size_t)w * sv : nullptr);
}

// ---------------------------------------------------------------------------------------------- plain / folded GEMV
template <int NB>
__device__ __forceinline__ void gemv_plain_nb(const etxb_gemv_args& d, int blk, const Smem& sm) {
  const int r0 = blk * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 >= r1) return;
  const int KS = (d.K + 7) & ~7;
  if ((d.mode & 0xff) == ETXB_MODE_NORM) {
#pragma unroll 1
    for (int b = 0; b < NB; ++b)
      stage_norm_col(d.rows ? (const __nv_bfloat16*)d.rows + (size_t)b * d.srows : nullptr,
                     (const __nv_bfloat16*)d.resid_in + (size_t)b * d.srin,
                     d.resid_out ? (__nv_bfloat16*)d.resid_out + (size_t)b * d.srout : nullptr,
                     d.x ? (__nv_bfloat16*)d.x + (size_t)b * d.sx : nullptr, d.ln,
                     d.ids ? d.ids + (size_t)b * d.R : nullptr, d.R, d.K, d.eps, sm.xs + (size_t)b * KS, sm.scr, blk == 0);
  } else {
    stage_x(d.x, d.K, d.sx, NB, KS, sm.xs);
  }
  const __nv_bfloat16* W = (const __nv_bfloat16*)d.W;
  const __nv_bfloat16* bias = (d.mode & ETXB_MODE_BIAS) ? (const __nv_bfloat16*)d.wts : nullptr;
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  const int K = d.K, sout = d.sout;
  gemv_rows<NB>(r1 - r0, K, [&](int q) { return W + (size_t)(r0 + q) * K; }, sm.xs, KS, sm.scr + 128,
                [&](int q, const float* v) {
                  const float bv = bias ? __bfloat162float(bias[r0 + q]) : 0.f;
#pragma unroll
                  for (int b = 0; b < NB; ++b) out[(size_t)b * sout + r0 + q] = __float2bfloat16_rn(bias ? __fadd_rn(v[b], bv) : v[b]);
                });
}

__device__ __forceinline__ void tile_gemv(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  switch (d.nb <= 1 ? 1 : d.nb) {
    case 1: gemv_plain_nb<1>(d, blk, sm); break;
    case 2: gemv_plain_nb<2>(d, blk, sm); break;
    case 4: gemv_plain_nb<4>(d, blk, sm); break;
    case 8: gemv_plain_nb<8>(d, blk, sm); break;
    default: break;                                                // rejected on the host
  }
}

// ---------------------------------------------------------------------------------------------- MoE gate+up
// task blk: slot s = blk / tpe, row chunk j = blk % tpe; expert e = ids[s] (ids == null and no fold: expert 0, the
// dense SwiGLU MLP); act[s][r] = bf16(bf16(silu(bf16 g)) * bf16 u), g = W_e[r,:].x, u = W_e[M + r,:].x.
__device__ __forceinline__ void tile_moe_up(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int s = blk / d.tpe, j = blk - s * d.tpe;
  const int r0 = j * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 >= r1) return;
  const int n = r1 - r0;
  int* lids = (int*)(sm.scr + 96); float* lwts = sm.scr + 112;
  const int fold = d.mode & 0xff;
  if (fold >= 2) {
    if (tidx() < 32) warp_topk(d.logits, d.E, d.R, fold == 3, (d.mode & ETXB_MODE_BF16_WTS) != 0, lids, lwts, nullptr);
    __syncthreads();
    if (j == 0 && tidx() == 0) {                              // the slot's first chunk publishes the routing
      if (d.ids) ((int32_t*)d.ids)[s] = lids[s];
      if (d.wts) ((float*)d.wts)[s] = lwts[s];
    }
  }
  const int e = fold >= 2 ? lids[s] : (d.ids ? __ldcg(d.ids + s) : 0);
  const __nv_bfloat16* We = (const __nv_bfloat16*)d.W + (size_t)e * d.estride;
  const int K = d.K, M = d.M, KS = (K + 7) & ~7;
  if (fold == ETXB_MODE_NORM)                                      // dense MLP: the post-attention norm folded in
    stage_norm_col(d.rows, d.resid_in, d.resid_out, (void*)d.x, d.ln, nullptr, d.R, K, d.eps, sm.xs, sm.scr, blk == 0);
  else
    stage_x(d.x, K, 0, 1, KS, sm.xs);
  float* g = sm.scr + 1024;                                        // 2 * n floats (n <= 2048)
  gemv_rows<1>(2 * n, K, [&](int q) { return We + (size_t)(q < n ? r0 + q : M + r0 + q - n) * K; }, sm.xs, KS, sm.scr + 128,
               [&](int q, const float* v) { g[q] = bfr(v[0]); });
  __syncthreads();
  __nv_bfloat16* act = (__nv_bfloat16*)d.out + (size_t)s * M;
  for (int r = tidx(); r < n; r += blockDim.x) act[r0 + r] = __float2bfloat16_rn(__fmul_rn(bfr(silu_f(g[r])), g[n + r]));
}

// ---------------------------------------------------------------------------------------------- MoE down
// out[s][r] = bf16(bf16(W_e[r,:] . act_s) * wts[s]); wts == null (dense MLP): out[s][r] = bf16(W_e[r,:] . act_s).
__device__ __forceinline__ void tile_moe_down(const unsigned char* a, int blk, const Smem& sm) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int s = blk / d.tpe, j = blk - s * d.tpe;
  const int r0 = j * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 >= r1) return;
  int* lids = (int*)(sm.scr + 96); float* lwts = sm.scr + 112;
  const int fold = d.mode & 0xff;
  if (fold >= 2) {
    if (tidx() < 32) warp_topk(d.logits, d.E, d.R, fold == 3, (d.mode & ETXB_MODE_BF16_WTS) != 0, lids, lwts, nullptr);
    __syncthreads();
  }
  const int e = fold >= 2 ? lids[s] : (d.ids ? __ldcg(d.ids + s) : 0);
  const bool scaled = fold >= 2 || d.wts != nullptr;
  const float ws = fold >= 2 ? lwts[s] : (d.wts ? __ldcg(d.wts + s) : 1.f);
  const __nv_bfloat16* We = (const __nv_bfloat16*)d.W + (size_t)e * d.estride;
  const int K = d.K, KS = (K + 7) & ~7;
  stage_x((const __nv_bfloat16*)d.x + (size_t)s * K, K, 0, 1, KS, sm.xs);
  __nv_bfloat16* out = (__nv_bfloat16*)d.out + (size_t)s * d.M;
  gemv_rows<1>(r1 - r0, K, [&](int q) { return We + (size_t)(r0 + q) * K; }, sm.xs, KS, sm.scr + 128,
               [&](int q, const float* v) {
                 const float y = bfr(v[0]);
                 out[r0 + q] = __float2bfloat16_rn(scaled ? __fmul_rn(y, ws) : y);
               });
}

}  // namespace etxb
