// The attention phase of a decode step, the form tuned for head_dim 128 and 16-position cache blocks: one task per
// (128-position partition, group of GQ q heads that share a kv head).  Same work as the general fused tile
// (etxb_attn_fused.cuh: q/k RMSNorm + neox rotary, the new position's k / v rows into the paged cache, split-KV
// attention, merge by the last task to finish) with two differences that shorten its critical path:
//   * the partition's K and V go from the cache straight into registers (each thread keeps the 64 + 64 bytes it will
//     multiply), no shared-memory staging;
//   * a task covers few q heads and many positions, so the merge that the last task runs reads GQ * parts partial
//     rows (2 * 9 at a 1K context) instead of G * parts of 32 positions (8 * 34): one round of loads.
// The groups of one kv head read the same K / V (through L2); the first group of the kv head writes the cache slot.
// The new position never comes from the cache: its k / v rows are taken from shared memory as one extra position.
//
// It stands where the reference runs dsl_attnprep (etx/ops/attnprep.py:86-211), vLLM's paged attention and its reduce
// kernel (etx/importer/spec.py:243-244; grids examples/vllm_llm/model.py:78-84, 358-362); numerics follow
// examples/llm/ref_numpy.py:113-129 (fp32 scores and sums over bf16 q, k, v; bf16 output).
#pragma once
#include "etxb_attn_fused.cuh"

namespace etxb {

#define ETXB_GQ_PART 128   // positions per task
#define ETXB_GQ_STAGE_BYTES 65536  // whole-sequence form: a partition's K and V pieces in shared memory (512 threads x 4 x 16 bytes each)
#define ETXB_GQ_WHOLE (1 << 24)   // part_len bit: one task per (sequence, q group) walks all partitions (plans without streamed tiles)
#define ETXB_GQ_PW 136     // 8-byte (value, flag) pairs a task publishes per q head and partition: 128 outputs, max, sum, padding

// Partial results travel as FLAGGED PAIRS: every fp32 value is stored together with a 32-bit flag derived from the step
// (one aligned 8-byte store: value and flag become visible together), into `tmp_out` viewed as
// [NH][max_parts][ETXB_GQ_PW] pairs.  The merge is run by a task that is known beforehand -- the one of the context's LAST
// partition (the partition of the new position: it has the fewest cached positions, so it is the first to finish and
// polls while the others work) -- which re-reads a pair until its flag is this step's.  No counter, no election, no
// fence: the producers only store, the merger's loads are its wait.  Nothing has to be reset between steps or after an
// abandoned step; a buffer that was zeroed once never shows a current flag by accident (flags are never 0, differ
// from grid to grid within a step and grow with the step).  Bounded like every wait: on a give-up the step is abandoned with the timeout status.
// The flag names the step AND the grid: the layers of a step share the partial buffers, and a merger must not take the
// previous layer's partials of the same step for its own.  The grid's tag travels in the upper half of the block's
// part_len word (the builder puts the layer index there).
__device__ __forceinline__ uint32_t pair_flag(uint32_t epoch, int part_len) { return ((epoch << 8) | (((uint32_t)part_len >> 16) & 0xffu)) | 0x80000000u; }
__device__ __forceinline__ void st_pair(uint2* p, float v, uint32_t fl) {
  asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(fl) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
  uint2 v;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
  return v;
}
// value of the pair at `p` once its flag is `fl`; gives up (step abandoned, 0 returned) at the deadline or on an abort
__device__ __forceinline__ float poll_pair(const uint2* p, uint32_t fl, const Smem& sm) {
  uint32_t spins = 0;
  for (;;) {
    const uint2 v = ld_pair(p);
    if (v.y == fl) return __uint_as_float(v.x);
    if ((++spins & 63u) == 0) {
      if (ld_relaxed(sm.ctrl) != 0) { *(volatile int*)sm.stop = 1; return 0.f; }
      if ((spins & 1023u) == 0 && globaltimer() > *sm.deadline) {
        if (atomicOr(sm.ctrl, ETXB_CTRL_TIMEOUT) == 0) { sm.ctrl[1] = sm.cur; sm.ctrl[2] = -3; sm.ctrl[3] = (int32_t)v.y; sm.ctrl[4] = (int32_t)fl; }
        *(volatile int*)sm.stop = 1;
        return 0.f;
      }
      __nanosleep(32);
    }
  }
}

template <int GQ>
struct GqSmem {
  static constexpr int HD = 128, PL = ETXB_GQ_PART;
  float* raw;   // [GQ + 2][HD] raw q rows, new k row, new v row
  float* cw;    // [3][HD] cos | sin row, q norm weight, k norm weight
  float* qs;    // [GQ][HD] normed + roped q
  float* knew;  // [HD] normed + roped new k (bf16 values)
  float* vnew;  // [HD] new v (bf16 values)
  float* ph;    // [4][GQ][PL] quarter dot products
  float* sc;    // [GQ][PL] probabilities
  float* st;    // [GQ] max, [GQ] sum, [GQ] probability of the new position
  float* po;    // [4][GQ][HD] partial outputs
  __device__ explicit GqSmem(float* b) {
    raw = b; cw = raw + (GQ + 2) * HD; qs = cw + 3 * HD; knew = qs + GQ * HD; vnew = knew + HD;
    ph = vnew + HD; sc = ph + 4 * GQ * PL; st = sc + GQ * PL; po = st + 32;
  }
};
#ifndef ETXB_LAYOUT_EXPERIMENT
static_assert(((8 + 2) + 3 + 8 + 2 + 32 + 8 + 32) * 128 * 4 + 128 <= ETXB_GEN_BYTES, "GQ = 8 layout fits the general region");
#endif

// out[hq][:] = bf16(sum_p w_p * tmp[p][:] / sum_p w_p * l_p), w_p = exp(m_p - max m), for q heads hq0 .. hq0 + GQ - 1.
// Run by the task of the last partition; polls the flagged partials the other CTAs publish (L2).  GQ * np <= 4096.
// The statistics AND the partial outputs are requested in one round (up to ETXB_GQ_NPR partitions out of registers), so the
// tail of the attention phase is one L2 round trip after the slowest partition has published.
template <int GQ>
__device__ __noinline__ void attn_gq_merge(const etxb_attnf_args& d, const Smem& sm, int hq0, int np, uint32_t fl) {
#ifndef ETXB_GQ_NPR
#define ETXB_GQ_NPR 12               // partitions merged out of registers in one round (a 1.5K context); measured against 16: 0.8 % faster
#endif
  constexpr int HD = 128, NPR = ETXB_GQ_NPR, NR = (GQ * HD + ETXB_CONSUMERS - 1) / ETXB_CONSUMERS;   // output values per thread
  const int lane = tidx() & 31, warp = tidx() >> 5;
  float* wl = sm.xs;                                              // [GQ][np] max logits, then weights
  float* es = sm.xs + 4096;                                       // [GQ][np] exp sums
  float* red = sm.scr + 200;                                      // [GQ] denominators
  const uint2* pw = (const uint2*)d.tmp_out;
  const int idx0 = tidx();                                        // this thread's output values (GQ * HD <= 1024: one or two)
  float pv[NR][NPR];
  const bool in_regs = np <= NPR;
  if (in_regs) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int idx = idx0 + r * ETXB_CONSUMERS;
      if (idx < GQ * HD) {
        const int g = idx >> 7, dd = idx & (HD - 1);
        const uint2* tp = pw + (size_t)(hq0 + g) * d.max_parts * ETXB_GQ_PW + dd;
        uint2 first[NPR];
#pragma unroll
        for (int u = 0; u < NPR; ++u) first[u] = ld_pair(tp + (size_t)min(u, np - 1) * ETXB_GQ_PW);   // all requests in flight at once
#pragma unroll
        for (int u = 0; u < NPR; ++u)
          pv[r][u] = (u >= np || first[u].y == fl) ? __uint_as_float(first[u].x) : poll_pair(tp + (size_t)u * ETXB_GQ_PW, fl, sm);
      }
    }
  }
  for (int i = tidx(); i < GQ * np; i += ETXB_CONSUMERS) {
    const int g = i / np, pp = i - g * np;
    const uint2* st = pw + ((size_t)(hq0 + g) * d.max_parts + pp) * ETXB_GQ_PW + HD;
    wl[i] = poll_pair(st, fl, sm);
    es[i] = poll_pair(st + 1, fl, sm);
  }
  csync();
  mark(sm, 0);
  if (warp < GQ) {
    const int g = warp;
    float m = -INFINITY;
    for (int pp = lane; pp < np; pp += 32) m = fmaxf(m, wl[g * np + pp]);
    m = warp_max(m);
    float L = 0.f;
    for (int pp = lane; pp < np; pp += 32) {
      const float w = expf(__fsub_rn(wl[g * np + pp], m));
      wl[g * np + pp] = w;
      L = __fmaf_rn(w, es[g * np + pp], L);
    }
    L = warp_sum(L);
    if (lane == 0) red[g] = L;
  }
  csync();
  mark(sm, 1);
  if (in_regs) {
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      const int idx = idx0 + r * ETXB_CONSUMERS;
      if (idx < GQ * HD) {
        const int g = idx >> 7;
        const float* wg = wl + g * np;
        float o = 0.f;
#pragma unroll
        for (int u = 0; u < NPR; ++u) o = __fmaf_rn(u < np ? wg[u] : 0.f, u < np ? pv[r][u] : 0.f, o);   // partitions in ascending order
        ((__nv_bfloat16*)d.out)[(size_t)hq0 * HD + idx] = __float2bfloat16_rn(__fdiv_rn(o, red[g]));
      }
    }
  } else {
    // a long context: the partials in rounds of NPR requests per output value, partitions still in ascending order
    for (int idx = tidx(); idx < GQ * HD; idx += ETXB_CONSUMERS) {
      const int g = idx >> 7, dd = idx & (HD - 1);
      const uint2* tp = pw + (size_t)(hq0 + g) * d.max_parts * ETXB_GQ_PW + dd;
      const float* wg = wl + g * np;
      float o = 0.f;
      for (int p0 = 0; p0 < np; p0 += NPR) {
        uint2 first[NPR];
#pragma unroll
        for (int u = 0; u < NPR; ++u) first[u] = ld_pair(tp + (size_t)min(p0 + u, np - 1) * ETXB_GQ_PW);
#pragma unroll
        for (int u = 0; u < NPR; ++u)
          if (p0 + u < np)
            o = __fmaf_rn(wg[p0 + u], first[u].y == fl ? __uint_as_float(first[u].x) : poll_pair(tp + (size_t)(p0 + u) * ETXB_GQ_PW, fl, sm), o);
      }
      ((__nv_bfloat16*)d.out)[(size_t)(hq0 + g) * HD + dd] = __float2bfloat16_rn(__fdiv_rn(o, red[g]));
    }
  }
  mark(sm, 2);
}

template <int GQ>
__device__ __noinline__ void attn_gq_impl(const etxb_attnf_args& d, int blk, const Smem& sm, const etxb_stepv& S) {
  constexpr int HD = 128, BS = 16, X = 8, PL = ETXB_GQ_PART, HV = HD / 8;
  const int NKV = d.NKV, G = d.NH / NKV, NQG = d.NH / GQ;
  const int part = blk / NQG, qg = blk - part * NQG;
  const int hq0 = qg * GQ, h = hq0 / G;                           // first q head of the group, its kv head
  const bool writer = hq0 - h * G == 0;                           // the kv head's first group stores the new k / v rows
  // the step's own buffers hold what the prologue wrote from the step parameters: take the values from there
  const long long pos = (const void*)d.positions == (const void*)S.positions ? (long long)S.pos : __ldcg((const long long*)d.positions);
  const long long slot = (const void*)d.slot_mapping == (const void*)S.slot_mapping ? (long long)S.pos : __ldcg((const long long*)d.slot_mapping);
  const int seq = (const void*)d.seq_lens == (const void*)S.seq_lens ? S.pos + 1 : __ldcg(d.seq_lens);
  const int t0 = part * PL;
  const int tid = tidx(), lane = tid & 31, warp = tid >> 5;
  const uint32_t fl = pair_flag(sm.epoch, d.part_len);
  if (t0 < seq) {
    const GqSmem<GQ> s(sm.xs);
    const bool owner = pos >= t0 && pos < t0 + PL;                // this partition holds the position being written
    const int tpos = owner ? (int)(pos - t0) : -1;
    const int ntok = min(PL, seq - t0);
    // positions taken from the cache: all of the partition's but the new one (its slot is stale until this step's write)
    auto cached = [&](int tt) { return tt < ntok && tt != tpos; };
    const int t = tid & (PL - 1), qr = tid >> 7;                  // K: position t, dims [32 qr, 32 qr + 32);  V: dim t, blocks 2 qr, 2 qr + 1
    // ---- K and V of the partition: cache -> registers (nothing here depends on this step's q)
    uint4 kreg[4], vreg[4];
    {
      const int lb = t0 / BS + (t >> 4);
      const bool live = lb * BS < seq;
      const long long pb = live ? __ldg(d.block_tables + lb) : 0;
      const __nv_bfloat16* kp = (const __nv_bfloat16*)d.kc + ((((size_t)pb * NKV + h) * HV + qr * 4) * BS + (t & 15)) * X;
#pragma unroll
      for (int j = 0; j < 4; ++j) kreg[j] = live ? ld_act16(kp + (size_t)j * BS * X) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int lv = t0 / BS + 2 * qr + u;
        const bool lv_live = lv * BS < seq;
        const long long pv = lv_live ? __ldg(d.block_tables + lv) : 0;
        const __nv_bfloat16* vp = (const __nv_bfloat16*)d.vc + (((size_t)pv * NKV + h) * HD + t) * BS;
        vreg[2 * u] = lv_live ? ld_act16(vp) : make_uint4(0u, 0u, 0u, 0u);
        vreg[2 * u + 1] = lv_live ? ld_act16(vp + 8) : make_uint4(0u, 0u, 0u, 0u);
      }
    }
    // ---- this step's rows: raw q heads, (owner) new k and v rows; rotary row and norm weights
    {
      const __nv_bfloat16* qkv = (const __nv_bfloat16*)d.qkv;
      const int nq = GQ * HV, nrow = nq + (owner ? 2 * HV : 0);
      for (int i = tid; i < nrow + 3 * HV; i += ETXB_CONSUMERS) {
        if (i < nrow) {
          const __nv_bfloat16* src = i < nq ? qkv + (size_t)hq0 * HD + 8 * i
                                            : (i < nq + HV ? qkv + (size_t)(d.NH + h) * HD + 8 * (i - nq)
                                                           : qkv + (size_t)(d.NH + NKV + h) * HD + 8 * (i - nq - HV));
          unpack8(ld_act16(src), s.raw + (i < nq ? 8 * i : GQ * HD + 8 * (i - nq)));
        } else {
          const int c = i - nrow, which = c / HV, v = c - which * HV;
          const __nv_bfloat16* src = which == 0 ? (const __nv_bfloat16*)d.cos_sin + (size_t)pos * HD
                                                : (const __nv_bfloat16*)(which == 1 ? d.qw : d.kw);
          if (src != nullptr) unpack8(__ldg((const uint4*)src + v), s.cw + which * HD + 8 * v);
        }
      }
    }
    csync();
    mark(sm, 0);
    // ---- norm + rope of the q heads (warps 0..GQ-1), of the new k row (warp GQ); the new v row (warp GQ + 1)
    if (warp < GQ) {
      float o[8];
      head_norm_rope_s<128>(s.raw + warp * HD, d.qw ? s.cw + HD : nullptr, s.cw, HD, d.eps, o);
#pragma unroll
      for (int j = 0; j < 4; ++j) s.qs[warp * HD + lane * 4 + j] = o[j];
    } else if (warp == GQ && owner) {
      float o[8];
      head_norm_rope_s<128>(s.raw + GQ * HD, d.kw ? s.cw + 2 * HD : nullptr, s.cw, HD, d.eps, o);
      const long long cb = slot / BS; const int off = (int)(slot % BS);
      __nv_bfloat16* kc = (__nv_bfloat16*)d.kc;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int dd = lane * 4 + j;
        s.knew[dd] = o[j];
        if (writer) kc[((((size_t)cb * NKV + h) * HV + dd / X) * BS + off) * X + dd % X] = __float2bfloat16_rn(o[j]);
      }
    } else if (warp == GQ + 1 && owner) {
      const long long cb = slot / BS; const int off = (int)(slot % BS);
      __nv_bfloat16* vc = (__nv_bfloat16*)d.vc;
      for (int dd = lane; dd < HD; dd += 32) {
        const float v = s.raw[(GQ + 1) * HD + dd];
        s.vnew[dd] = v;
        if (writer) vc[(((size_t)cb * NKV + h) * HD + dd) * BS + off] = __float2bfloat16_rn(v);
      }
    }
    csync();
    mark(sm, 1);
    // ---- scores: thread (qr, t) holds 32 dims of position t; quarter sums to shared memory
    {
      float acc[GQ];
#pragma unroll
      for (int g = 0; g < GQ; ++g) acc[g] = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float kf[8];
        unpack8(kreg[j], kf);
#pragma unroll
        for (int g = 0; g < GQ; ++g) {
          const float4 qa = *(const float4*)(s.qs + g * HD + (qr * 4 + j) * 8), qb = *(const float4*)(s.qs + g * HD + (qr * 4 + j) * 8 + 4);
          acc[g] = __fmaf_rn(kf[0], qa.x, acc[g]); acc[g] = __fmaf_rn(kf[1], qa.y, acc[g]);
          acc[g] = __fmaf_rn(kf[2], qa.z, acc[g]); acc[g] = __fmaf_rn(kf[3], qa.w, acc[g]);
          acc[g] = __fmaf_rn(kf[4], qb.x, acc[g]); acc[g] = __fmaf_rn(kf[5], qb.y, acc[g]);
          acc[g] = __fmaf_rn(kf[6], qb.z, acc[g]); acc[g] = __fmaf_rn(kf[7], qb.w, acc[g]);
        }
      }
#pragma unroll
      for (int g = 0; g < GQ; ++g) s.ph[(qr * GQ + g) * PL + t] = acc[g];
    }
    csync();
    // ---- softmax statistics: one warp per q head, lane holds positions lane + 32 k
    if (warp < GQ) {
      const int g = warp;
      float sv[4], m = -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int tt = lane + 32 * k;
        const float dot = __fadd_rn(__fadd_rn(__fadd_rn(s.ph[g * PL + tt], s.ph[(GQ + g) * PL + tt]), s.ph[(2 * GQ + g) * PL + tt]), s.ph[(3 * GQ + g) * PL + tt]);
        sv[k] = cached(tt) ? __fmul_rn(dot, d.scale) : -INFINITY;
        m = fmaxf(m, sv[k]);
      }
      float snew = -INFINITY;
      if (owner) {                                                 // the new position: q . k_new from shared memory
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) a = __fmaf_rn(s.qs[g * HD + lane * 4 + j], s.knew[lane * 4 + j], a);
        snew = __fmul_rn(warp_sum(a), d.scale);
      }
      m = fmaxf(warp_max(m), snew);
      float l = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float pr = cached(lane + 32 * k) ? expf(__fsub_rn(sv[k], m)) : 0.f;
        s.sc[g * PL + lane + 32 * k] = pr;
        l = __fadd_rn(l, pr);
      }
      l = warp_sum(l);
      const float pn = owner ? expf(__fsub_rn(snew, m)) : 0.f;
      if (lane == 0) { s.st[g] = m; s.st[GQ + g] = __fadd_rn(l, pn); s.st[2 * GQ + g] = pn; }
    }
    csync();
    mark(sm, 2);
    // ---- output: thread (qr, dd = t) multiplies its two blocks of 16 positions; quarter sums to shared memory
    {
      float acc[GQ];
#pragma unroll
      for (int g = 0; g < GQ; ++g) acc[g] = 0.f;
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int tb = (2 * qr + u) * BS;
        if (tb < ntok) {
          float f[16];
          unpack8(vreg[2 * u], f); unpack8(vreg[2 * u + 1], f + 8);
#pragma unroll
          for (int o = 0; o < 16; ++o) f[o] = cached(tb + o) ? f[o] : 0.f;   // stale slots may hold anything: never multiply them
#pragma unroll
          for (int g = 0; g < GQ; ++g) {
#pragma unroll
            for (int o4 = 0; o4 < 4; ++o4) {
              const float4 pr = *(const float4*)(s.sc + g * PL + tb + 4 * o4);
              acc[g] = __fmaf_rn(pr.x, f[4 * o4], acc[g]); acc[g] = __fmaf_rn(pr.y, f[4 * o4 + 1], acc[g]);
              acc[g] = __fmaf_rn(pr.z, f[4 * o4 + 2], acc[g]); acc[g] = __fmaf_rn(pr.w, f[4 * o4 + 3], acc[g]);
            }
          }
        }
      }
#pragma unroll
      for (int g = 0; g < GQ; ++g) s.po[(qr * GQ + g) * HD + t] = acc[g];
    }
    csync();
    for (int idx = tid; idx < GQ * HD; idx += ETXB_CONSUMERS) {
      const int g = idx >> 7, dd = idx & (HD - 1);
      float o = __fadd_rn(__fadd_rn(__fadd_rn(s.po[g * HD + dd], s.po[(GQ + g) * HD + dd]), s.po[(2 * GQ + g) * HD + dd]), s.po[(3 * GQ + g) * HD + dd]);
      if (owner) o = __fmaf_rn(s.st[2 * GQ + g], s.vnew[dd], o);
      uint2* pw = (uint2*)d.tmp_out + ((size_t)(hq0 + g) * d.max_parts + part) * ETXB_GQ_PW;
      st_pair(pw + dd, o, fl);
      if (dd == 0) { st_pair(pw + HD, s.st[g], fl); st_pair(pw + HD + 1, s.st[GQ + g], fl); }
    }
  }
  mark(sm, 3);
  // the context's last partition merges (never past the partitions the grid computed, whatever seq_lens says)
  const int np = min((seq + PL - 1) / PL, d.max_parts);
  if (part == np - 1) {
    csync();                                                       // every thread is done with the tile's shared memory
    attn_gq_merge<GQ>(d, sm, hq0, np, fl);
  }
}

// ---------------------------------------------------------------------------------------------- a whole sequence per task
// The same attention with one task per (sequence, group of GQ q heads): the task walks the context's partitions itself,
// keeps every partition's partial output and statistics in shared memory and merges them at the end with the merge's
// arithmetic (same partition boundaries, same order of sums: the results are those of the one-partition-per-task form bit
// for bit).  This is the form of a batched step with enough sequences to fill the workers (sequences x kv heads x groups
// tasks): the q rows are prepared once per sequence instead of once per partition, the next partition's K (then V) is
// copied asynchronously into shared memory while the current one is being worked on, so the cache latency hides behind
// the softmax and the output sums, and nothing is published, polled or merged through global memory.
// The partials live in the weight ring, which is idle in a batched plan (no streamed tiles): part_len bit 24 selects
// this form, and only builders of plans without streamed tiles may set it.  (64 KB of K / V pieces + np * GQ * 130 floats <= the ring.)
// D += A (16 x 16, row-major) * B (16 x 8, column-major), bf16 operands, fp32 accumulators (the warp-level tensor-core form)
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int GQ>
__device__ __noinline__ void attn_gq_seq(const etxb_attnf_args& d, int blk, const Smem& sm, const etxb_stepv& S) {
  constexpr int HD = 128, BS = 16, X = 8, PL = ETXB_GQ_PART, HV = HD / 8;
  const int NKV = d.NKV, G = d.NH / NKV;
  const int hq0 = blk * GQ, h = hq0 / G;
  const bool writer = hq0 - h * G == 0;
  const long long pos = (const void*)d.positions == (const void*)S.positions ? (long long)S.pos : __ldcg((const long long*)d.positions);
  const long long slot = (const void*)d.slot_mapping == (const void*)S.slot_mapping ? (long long)S.pos : __ldcg((const long long*)d.slot_mapping);
  const int seq = (const void*)d.seq_lens == (const void*)S.seq_lens ? S.pos + 1 : __ldcg(d.seq_lens);
  const int np = min(min((seq + PL - 1) / PL, d.max_parts), (ETXB_RING_BYTES - ETXB_GQ_STAGE_BYTES) / (GQ * (HD + 2) * 4));
  if (np < 1) return;
  const int tid = tidx(), lane = tid & 31, warp = tid >> 5;
  const GqSmem<GQ> s(sm.xs);
  // the weight ring: [4][512] 16-byte K pieces, [4][512] V pieces (piece j of thread tid at [j][tid]: every thread copies
  // and reads only its own), then the partitions' partial outputs and statistics
  uint4* KB = (uint4*)sm.ring;
  uint4* VB = KB + 4 * ETXB_CONSUMERS;
  // bf16 operands of the tensor-core products, rows padded to 68 words (bank-conflict-free fragment loads): the q heads,
  // and a partition's probabilities split into a bf16 value and the bf16 of what that rounding lost
  uint32_t* QB = (uint32_t*)(s.po + 4 * GQ * HD);                  // [8][68] words = [8 heads][136] bf16 (heads >= GQ: zero)
  uint32_t* PH = QB + 8 * 68;                                      // [8][68] high parts of the probabilities
  uint32_t* PLo = PH + 8 * 68;                                     // [8][68] low parts
  for (int i = tid; i < 3 * 8 * 68; i += ETXB_CONSUMERS) QB[i] = 0u;
  float* PO = (float*)(sm.ring + ETXB_GQ_STAGE_BYTES);            // [np][GQ][HD] partial outputs
  float* PS = PO + (size_t)np * GQ * HD;                           // [np][GQ][2] max logit, exp sum
  const int t = tid & (PL - 1), qr = tid >> 7;                     // K: position t, dims [32 qr, 32 qr + 32);  V: dim t, blocks 2 qr, 2 qr + 1
  // Asynchronous copies (cp.async, 16 bytes each, zero-filled where the context ends) bring a partition's K and V pieces
  // from the cache to shared memory while the previous partition is being worked on: K of the next partition as soon as
  // the scores have consumed this one's, V of the next as soon as the output sums have.  One commit group per request, in
  // that order, so "all but the latest group" is always the piece about to be read.  Nothing waits in registers: a
  // 17-warp CTA has 96 of them per thread, and a partition of K and V ahead would take 32.
  // (the block-table entries a request needs are fetched a phase earlier: tab[0] the block of the thread's K position,
  // tab[1], tab[2] the blocks of its V positions, of the partition that is requested next)
  int tab[3];
  auto fetch_tab = [&](int part) {
    const int lb = part * (PL / BS) + (t >> 4), lv = part * (PL / BS) + 2 * qr;
    tab[0] = part < np && lb * BS < seq ? __ldg(d.block_tables + lb) : 0;
    tab[1] = part < np && lv * BS < seq ? __ldg(d.block_tables + lv) : 0;
    tab[2] = part < np && (lv + 1) * BS < seq ? __ldg(d.block_tables + lv + 1) : 0;
  };
  auto request_k = [&](int part) {
    if (part < np) {
      const int lb = part * (PL / BS) + (t >> 4);
      const bool live = lb * BS < seq;
      const long long pb = tab[0];
      const __nv_bfloat16* kp = (const __nv_bfloat16*)d.kc + ((((size_t)pb * NKV + h) * HV + qr * 4) * BS + (t & 15)) * X;
#pragma unroll
      for (int j = 0; j < 4; ++j) cp_async16(KB + j * ETXB_CONSUMERS + tid, kp + (size_t)j * BS * X, live);
    }
    cp_async_commit();
  };
  auto request_v = [&](int part) {
    if (part < np) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int lv = part * (PL / BS) + 2 * qr + u;
        const bool live = lv * BS < seq;
        const long long pv = tab[1 + u];
        const __nv_bfloat16* vp = (const __nv_bfloat16*)d.vc + (((size_t)pv * NKV + h) * HD + t) * BS;
        cp_async16(VB + (2 * u) * ETXB_CONSUMERS + tid, vp, live);
        cp_async16(VB + (2 * u + 1) * ETXB_CONSUMERS + tid, vp + 8, live);
      }
    }
    cp_async_commit();
  };
  fetch_tab(0);
  request_k(0);
  request_v(0);
  // ---- this step's rows: raw q heads, new k and v rows; rotary row and norm weights
  {
    const __nv_bfloat16* qkv = (const __nv_bfloat16*)d.qkv;
    const int nq = GQ * HV, nrow = nq + 2 * HV;
    for (int i = tid; i < nrow + 3 * HV; i += ETXB_CONSUMERS) {
      if (i < nrow) {
        const __nv_bfloat16* src = i < nq ? qkv + (size_t)hq0 * HD + 8 * i
                                          : (i < nq + HV ? qkv + (size_t)(d.NH + h) * HD + 8 * (i - nq)
                                                         : qkv + (size_t)(d.NH + NKV + h) * HD + 8 * (i - nq - HV));
        unpack8(ld_act16(src), s.raw + (i < nq ? 8 * i : GQ * HD + 8 * (i - nq)));
      } else {
        const int c = i - nrow, which = c / HV, v = c - which * HV;
        const __nv_bfloat16* src = which == 0 ? (const __nv_bfloat16*)d.cos_sin + (size_t)pos * HD
                                              : (const __nv_bfloat16*)(which == 1 ? d.qw : d.kw);
        if (src != nullptr) unpack8(__ldg((const uint4*)src + v), s.cw + which * HD + 8 * v);
      }
    }
  }
  csync();
  mark(sm, 0);
  if (warp < GQ) {
    float o[8];
    head_norm_rope_s<128>(s.raw + warp * HD, d.qw ? s.cw + HD : nullptr, s.cw, HD, d.eps, o);
#pragma unroll
    for (int j = 0; j < 4; ++j) s.qs[warp * HD + lane * 4 + j] = o[j];
    QB[warp * 68 + 2 * lane] = pack_bf(o[0], o[1]);                // (the rotated q values are bf16 values already)
    QB[warp * 68 + 2 * lane + 1] = pack_bf(o[2], o[3]);
  } else if (warp == GQ) {
    float o[8];
    head_norm_rope_s<128>(s.raw + GQ * HD, d.kw ? s.cw + 2 * HD : nullptr, s.cw, HD, d.eps, o);
    const long long cb = slot / BS; const int off = (int)(slot % BS);
    __nv_bfloat16* kc = (__nv_bfloat16*)d.kc;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int dd = lane * 4 + j;
      s.knew[dd] = o[j];
      if (writer) kc[((((size_t)cb * NKV + h) * HV + dd / X) * BS + off) * X + dd % X] = __float2bfloat16_rn(o[j]);
    }
  } else if (warp == GQ + 1) {
    const long long cb = slot / BS; const int off = (int)(slot % BS);
    __nv_bfloat16* vc = (__nv_bfloat16*)d.vc;
    for (int dd = lane; dd < HD; dd += 32) {
      const float v = s.raw[(GQ + 1) * HD + dd];
      s.vnew[dd] = v;
      if (writer) vc[(((size_t)cb * NKV + h) * HD + dd) * BS + off] = __float2bfloat16_rn(v);
    }
  }
  csync();
  mark(sm, 1);
  for (int part = 0; part < np; ++part) {
    const int t0 = part * PL;
    const bool owner = pos >= t0 && pos < t0 + PL;
    const int tpos = owner ? (int)(pos - t0) : -1;
    const int ntok = min(PL, seq - t0);
    auto cached = [&](int tt) { return tt < ntok && tt != tpos; };
    fetch_tab(part + 1);
    // ---- scores on the tensor cores: S[position][head] = K[position][:] . q[head][:].  Warp = (16 positions, half of the
    //      128 dims): four m16n8k16 steps; A fragments straight from the staged K pieces (piece of dims chunk c and
    //      position p sits at [c & 3][c >> 2][p]), B fragments from the bf16 q rows.  The two halves go to s.ph.
    cp_async_wait1();                                              // this thread's K pieces have landed (its V may still travel)
    csync();                                                       // .. and everybody else's: the fragments cross threads
    {
      const int mt = warp & 7, kh = warp >> 3, g8 = lane >> 2, t4 = lane & 3;
      const uint32_t* KW = (const uint32_t*)KB;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      const int p0 = 16 * mt + g8;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int ks = 4 * kh + q, c0 = 2 * ks, c1 = 2 * ks + 1;
        const uint32_t a0 = KW[(((c0 & 3) * ETXB_CONSUMERS + (c0 >> 2) * PL + p0) << 2) + t4];
        const uint32_t a1 = KW[(((c0 & 3) * ETXB_CONSUMERS + (c0 >> 2) * PL + p0 + 8) << 2) + t4];
        const uint32_t a2 = KW[(((c1 & 3) * ETXB_CONSUMERS + (c1 >> 2) * PL + p0) << 2) + t4];
        const uint32_t a3 = KW[(((c1 & 3) * ETXB_CONSUMERS + (c1 >> 2) * PL + p0 + 8) << 2) + t4];
        mma16816(c, a0, a1, a2, a3, QB[g8 * 68 + 8 * ks + t4], QB[g8 * 68 + 8 * ks + 4 + t4]);
      }
      const int h0 = 2 * t4;
      if (h0 < GQ) { s.ph[(kh * GQ + h0) * PL + p0] = c[0]; s.ph[(kh * GQ + h0) * PL + p0 + 8] = c[2]; }
      if (h0 + 1 < GQ) { s.ph[(kh * GQ + h0 + 1) * PL + p0] = c[1]; s.ph[(kh * GQ + h0 + 1) * PL + p0 + 8] = c[3]; }
    }
    csync();
    request_k(part + 1);                                           // every warp is done with the K pieces: the next partition's may land
    // ---- softmax statistics: one warp per q head, lane holds positions lane + 32 k
    if (warp < GQ) {
      const int g = warp;
      float sv[4], m = -INFINITY;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int tt = lane + 32 * k;
        const float dot = __fadd_rn(s.ph[g * PL + tt], s.ph[(GQ + g) * PL + tt]);
        sv[k] = cached(tt) ? __fmul_rn(dot, d.scale) : -INFINITY;
        m = fmaxf(m, sv[k]);
      }
      float snew = -INFINITY;
      if (owner) {
        float a = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) a = __fmaf_rn(s.qs[g * HD + lane * 4 + j], s.knew[lane * 4 + j], a);
        snew = __fmul_rn(warp_sum(a), d.scale);
      }
      m = fmaxf(warp_max(m), snew);
      float l = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float pr = cached(lane + 32 * k) ? expf(__fsub_rn(sv[k], m)) : 0.f;
        const __nv_bfloat16 hi = __float2bfloat16_rn(pr), lo = __float2bfloat16_rn(__fsub_rn(pr, __bfloat162float(hi)));
        ((__nv_bfloat16*)PH)[g * 136 + lane + 32 * k] = hi;
        ((__nv_bfloat16*)PLo)[g * 136 + lane + 32 * k] = lo;
        l = __fadd_rn(l, pr);
      }
      l = warp_sum(l);
      const float pn = owner ? expf(__fsub_rn(snew, m)) : 0.f;
      if (lane == 0) { s.st[g] = m; s.st[GQ + g] = __fadd_rn(l, pn); s.st[2 * GQ + g] = pn; }
    }
    // ---- output on the tensor cores: O[dim][head] = sum_pos V[dim][pos] P[head][pos].  Warp = (16 dims, half of the
    //      partition's eight cache blocks): per block one m16n8k16 step for the high and one for the low part of the
    //      probabilities; A fragments straight from the staged V pieces (block b, positions 8 v .. of dim d at
    //      [2 (b & 1) + v][b >> 1][d]).  Slots that are not cached yet (last partition only) are zeroed first: a
    //      probability of 0 does not neutralise whatever bits a stale slot holds.
    cp_async_wait1();                                              // this thread's V pieces have landed (the next K may still travel)
    if (part == np - 1) {
      __nv_bfloat16* vb = (__nv_bfloat16*)VB;
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int v = 0; v < 2; ++v) {
          const int base = (2 * qr + u) * BS + 8 * v;
          if (base + 8 > ntok || (tpos >= base && tpos < base + 8))
#pragma unroll
            for (int o = 0; o < 8; ++o)
              if (!cached(base + o)) vb[(((2 * u + v) * ETXB_CONSUMERS + tid) << 3) + o] = __float2bfloat16_rn(0.f);
        }
    }
    csync();                                                       // the probabilities and everybody's V pieces are in place
    {
      const int mt = warp & 7, kh = warp >> 3, g8 = lane >> 2, t4 = lane & 3;
      const uint32_t* VW = (const uint32_t*)VB;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      const int d0 = 16 * mt + g8;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int b = 4 * kh + q;
        if (b * BS < ntok) {
          const int pu = 2 * (b & 1), pq = (b >> 1) * PL;
          const uint32_t a0 = VW[((pu * ETXB_CONSUMERS + pq + d0) << 2) + t4];
          const uint32_t a1 = VW[((pu * ETXB_CONSUMERS + pq + d0 + 8) << 2) + t4];
          const uint32_t a2 = VW[(((pu + 1) * ETXB_CONSUMERS + pq + d0) << 2) + t4];
          const uint32_t a3 = VW[(((pu + 1) * ETXB_CONSUMERS + pq + d0 + 8) << 2) + t4];
          mma16816(c, a0, a1, a2, a3, PH[g8 * 68 + 8 * b + t4], PH[g8 * 68 + 8 * b + 4 + t4]);
          mma16816(c, a0, a1, a2, a3, PLo[g8 * 68 + 8 * b + t4], PLo[g8 * 68 + 8 * b + 4 + t4]);
        }
      }
      const int h0 = 2 * t4;
      if (h0 < GQ) { s.po[(kh * GQ + h0) * HD + d0] = c[0]; s.po[(kh * GQ + h0) * HD + d0 + 8] = c[2]; }
      if (h0 + 1 < GQ) { s.po[(kh * GQ + h0 + 1) * HD + d0] = c[1]; s.po[(kh * GQ + h0 + 1) * HD + d0 + 8] = c[3]; }
    }
    csync();
    request_v(part + 1);                                           // every warp is done with the V pieces
    for (int idx = tid; idx < GQ * HD; idx += ETXB_CONSUMERS) {
      const int g = idx >> 7, dd = idx & (HD - 1);
      float o = __fadd_rn(s.po[g * HD + dd], s.po[(GQ + g) * HD + dd]);
      if (owner) o = __fmaf_rn(s.st[2 * GQ + g], s.vnew[dd], o);
      PO[((size_t)part * GQ + g) * HD + dd] = o;
      if (dd == 0) { PS[(part * GQ + g) * 2] = s.st[g]; PS[(part * GQ + g) * 2 + 1] = s.st[GQ + g]; }
    }
    // (the next partition's score sums go to s.ph, its statistics to s.sc / s.st only after the barrier that follows them:
    // nothing this loop still reads is overwritten early)
  }
  csync();
  mark(sm, 2);
  // ---- merge, with the arithmetic of attn_gq_merge: weights exp(m_p - max m), sums in ascending partition order
  float* wl = s.ph;                                                // [GQ][np]
  float* red = s.st + 24;                                          // [GQ]
  if (warp < GQ) {
    const int g = warp;
    float m = -INFINITY;
    for (int pp = lane; pp < np; pp += 32) m = fmaxf(m, PS[(pp * GQ + g) * 2]);
    m = warp_max(m);
    float L = 0.f;
    for (int pp = lane; pp < np; pp += 32) {
      const float w = expf(__fsub_rn(PS[(pp * GQ + g) * 2], m));
      wl[g * np + pp] = w;
      L = __fmaf_rn(w, PS[(pp * GQ + g) * 2 + 1], L);
    }
    L = warp_sum(L);
    if (lane == 0) red[g] = L;
  }
  csync();
  for (int idx = tid; idx < GQ * HD; idx += ETXB_CONSUMERS) {
    const int g = idx >> 7, dd = idx & (HD - 1);
    float o = 0.f;
    for (int pp = 0; pp < np; ++pp) o = __fmaf_rn(wl[g * np + pp], PO[((size_t)pp * GQ + g) * HD + dd], o);
    ((__nv_bfloat16*)d.out)[(size_t)(hq0 + g) * HD + dd] = __float2bfloat16_rn(__fdiv_rn(o, red[g]));
  }
  mark(sm, 3);
  cp_async_wait0();
  csync();                                                         // the next task may overwrite the partials
}

// The grouped forms (gq > 0 in the argument block; head_dim 128, cache blocks of 16, partitions of 128): one task per
// partition, or (part_len bit 24) one task per sequence and q group.
__device__ __forceinline__ void tile_attn_gq(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_attnf_args& d = *(const etxb_attnf_args*)a;
  if (blk >= (int)d.nblocks || d.gq <= 0) return;
  if (d.part_len & ETXB_GQ_WHOLE) {
    switch (d.gq) {
      case 1: attn_gq_seq<1>(d, blk, sm, S); break;
      case 2: attn_gq_seq<2>(d, blk, sm, S); break;
      case 4: attn_gq_seq<4>(d, blk, sm, S); break;
      default: attn_gq_seq<8>(d, blk, sm, S); break;
    }
    return;
  }
  switch (d.gq) {
    case 1: attn_gq_impl<1>(d, blk, sm, S); break;
    case 2: attn_gq_impl<2>(d, blk, sm, S); break;
    case 4: attn_gq_impl<4>(d, blk, sm, S); break;
    default: attn_gq_impl<8>(d, blk, sm, S); break;
  }
}

// Fused attention, either form: gq > 0 in the argument block selects the grouped forms above, else the general tile.
__device__ __forceinline__ void tile_attn_any(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_attnf_args& d = *(const etxb_attnf_args*)a;
  if (d.gq == 0) { tile_attn_fused(a, blk, sm, S); return; }
  tile_attn_gq(a, blk, sm, S);
}

}  // namespace etxb
