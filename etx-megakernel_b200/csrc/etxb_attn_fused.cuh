// The attention phase of a decode step as ONE tile per (32-position partition, kv head): q/k RMSNorm + neox rotary, the
// new position's k / v rows into the paged cache, split-KV GQA attention over the partition, and the merge of the
// partitions by the last task of each kv head to finish (a monotonic counter per kv head elects it).
//
// It stands where the reference runs three phases: dsl_attnprep (etx/ops/attnprep.py:86-211), vLLM's paged attention
// and its reduce kernel (call recipe etx/importer/spec.py:243-244; grids examples/vllm_llm/model.py:78-84, 358-362).
// Numerics are those of the separate tiles (etxb_attn.cuh), i.e. of examples/llm/ref_numpy.py:113-129.
//
// HDT / BST: head_dim and cache block size as compile-time constants (0 = read them from the argument block); the
// 128 / 16 instantiation is the one every bundled model takes, and with constants the index arithmetic folds away.
#pragma once
#include "etxb_attn.cuh"

namespace etxb {

// One head row in shared memory (xh, HD floats; d = lane * epl + j held by lane): optional RMSNorm with weight nw, then
// neox rotary with the cos | sin row cs (both as floats in shared memory).  o[j] = the bf16-rounded results.  One warp.
template <int HDT>
__device__ __noinline__ void head_norm_rope_s(const float* xh, const float* nw, const float* cs, int HDr, float eps, float* o) {
  const int HD = HDT ? HDT : HDr;                                  // HDT: head_dim as a compile-time constant (0: read it)
  const int lane = tidx() & 31, half = HD >> 1, epl = HD >> 5;
  constexpr int EPL = HDT ? HDT / 32 : 8;
  float v[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) v[j] = j < epl ? xh[lane * epl + j] : 0.f;
  if (nw != nullptr) {
    const float ss = HDT == 128 ? sumsq128_numpy_order_warp(xh) : head_sumsq(xh, HD);
    const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)HD), eps)));
#pragma unroll
    for (int j = 0; j < EPL; ++j)
      if (j < epl) v[j] = bfr(__fmul_rn(nw[lane * epl + j], bfr(__fmul_rn(v[j], r))));
  }
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);    // element d +- HD/2 lives 16 lanes away
    if (j < epl) {
      const int dd = lane * epl + j;
      const float rot = dd < half ? -other : other;
      const int k = dd < half ? dd : dd - half;
      o[j] = bfr(__fadd_rn(bfr(__fmul_rn(v[j], cs[k])), bfr(__fmul_rn(rot, cs[half + k]))));
    }
  }
}

__device__ __forceinline__ void unpack8(const uint4 v, float* f) {
  f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
  f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}

// Shared-memory layout of the tile (G * HD <= 2048, HD <= 256: 60.7 KB of the 64 KB general region)
struct AttnSmem {
  float* qs; __nv_bfloat16* ks; __nv_bfloat16* vs; float* sc; float* st; float* ph; float* raw; float* cw;
};
__device__ __forceinline__ AttnSmem attn_smem(float* base, int G, int HD) {
  constexpr int P = ETXB_ATTN_PART;
  AttnSmem s;
  s.qs = base;                                    // [G][HD] normed + roped q
  s.ks = (__nv_bfloat16*)(s.qs + G * HD);         // [P / BS][HD / 8][BS][8]
  s.vs = s.ks + P * HD;                           // [P / BS][HD][BS]
  s.sc = (float*)(s.vs + P * HD);                 // [16][P] scores, then probabilities
  s.st = s.sc + 16 * P;                           // per head: max, sum
  s.ph = s.st + 64;                               // [2][16 * P] half dot products
  s.raw = s.ph + 2 * 16 * P;                      // [G + 2][HD] raw q rows, k row, v row
  s.cw = s.raw + (G + 2) * HD;                    // cos | sin row, q norm weight, k norm weight
  return s;
}

// Loads that depend on nothing but the step's position: the partition's cached K / V blocks, the rotary row and the
// norm weights; then the raw q rows (and the new k, v rows for the partition that holds the new position).
template <int HDT, int BST>
__device__ __forceinline__ void attn_fused_load(const etxb_attnf_args& d, const AttnSmem& s, int part, int h, int seq, long long pos, bool owner) {
  const int HD = HDT ? HDT : d.HD, BS = BST ? BST : d.BS;
  const int NH = d.NH, NKV = d.NKV, G = NH / NKV, P = ETXB_ATTN_PART;
  const int t0 = part * P, nblk = P / BS, vec_per_blk = HD * BS / 8;
  for (int i = tidx(); i < nblk * vec_per_blk; i += ETXB_CONSUMERS) {
    const int b = i / vec_per_blk, r = i - b * vec_per_blk;
    const int lb = t0 / BS + b;
    if (lb * BS < seq) {
      const long long pb = __ldg(d.block_tables + lb);
      const size_t base = ((size_t)pb * NKV + h) * HD * BS;
      *(uint4*)(s.ks + (size_t)b * HD * BS + 8 * r) = ld_act16((const __nv_bfloat16*)d.kc + base + 8 * r);
      *(uint4*)(s.vs + (size_t)b * HD * BS + 8 * r) = ld_act16((const __nv_bfloat16*)d.vc + base + 8 * r);
    }
  }
  const int hv = HD / 8;                                          // 16-byte vectors per head row
  for (int i = tidx(); i < 3 * hv; i += ETXB_CONSUMERS) {          // cos | sin, q weight, k weight
    const int which = i / hv, v = i - which * hv;
    const __nv_bfloat16* src = which == 0 ? (const __nv_bfloat16*)d.cos_sin + (size_t)pos * HD
                                          : (const __nv_bfloat16*)(which == 1 ? d.qw : d.kw);
    if (src != nullptr) unpack8(__ldg((const uint4*)src + v), s.cw + which * HD + 8 * v);
  }
  const __nv_bfloat16* qkv = (const __nv_bfloat16*)d.qkv;
  const int nq = G * hv;
  for (int i = tidx(); i < nq + (owner ? 2 * hv : 0); i += ETXB_CONSUMERS) {
    const __nv_bfloat16* src = i < nq ? qkv + (size_t)h * G * HD + 8 * i
                                      : (i < nq + hv ? qkv + (size_t)(NH + h) * HD + 8 * (i - nq)
                                                     : qkv + (size_t)(NH + NKV + h) * HD + 8 * (i - nq - hv));
    unpack8(ld_act16(src), s.raw + 8 * i);
  }
}

// norm + rope of the q heads (warps 0..G-1), of the new k row (warp G) and the new v row (warp G+1); the new rows go
// to the paged cache and over the stale slot of the shared tiles.
template <int HDT, int BST>
__device__ __forceinline__ void attn_fused_prep(const etxb_attnf_args& d, const AttnSmem& s, int part, int h, long long pos, long long slot, bool owner) {
  const int HD = HDT ? HDT : d.HD, BS = BST ? BST : d.BS;
  constexpr int X = 8, P = ETXB_ATTN_PART;
  const int NKV = d.NKV, G = d.NH / NKV;
  const int lane = tidx() & 31, warp = tidx() >> 5, epl = HD >> 5;
  const long long cb = slot / BS; const int off = (int)(slot % BS);
  const int lb_new = (int)(pos / BS) - part * P / BS, lo_new = (int)(pos % BS);
  if (warp < G) {
    float o[8];
    head_norm_rope_s<0>(s.raw + warp * HD, d.qw ? s.cw + HD : nullptr, s.cw, HD, d.eps, o);
#pragma unroll
    for (int j = 0; j < 8; ++j) if (j < epl) s.qs[warp * HD + lane * epl + j] = o[j];
  } else if (warp == G && owner) {
    float o[8];
    head_norm_rope_s<0>(s.raw + G * HD, d.kw ? s.cw + 2 * HD : nullptr, s.cw, HD, d.eps, o);
    __nv_bfloat16* kc = (__nv_bfloat16*)d.kc;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (j < epl) {
        const int dd = lane * epl + j;
        const __nv_bfloat16 kb = __float2bfloat16_rn(o[j]);
        kc[(((size_t)cb * NKV + h) * (HD / X) + dd / X) * BS * X + (size_t)off * X + dd % X] = kb;
        s.ks[(size_t)lb_new * HD * BS + ((size_t)(dd / X) * BS + lo_new) * X + dd % X] = kb;
      }
  } else if (warp == G + 1 && owner) {
    __nv_bfloat16* vc = (__nv_bfloat16*)d.vc;
    for (int dd = lane; dd < HD; dd += 32) {
      const __nv_bfloat16 vb = __float2bfloat16_rn(s.raw[(G + 1) * HD + dd]);
      vc[(((size_t)cb * NKV + h) * HD + dd) * BS + off] = vb;
      s.vs[(size_t)lb_new * HD * BS + (size_t)dd * BS + lo_new] = vb;
    }
  }
}

// scores, softmax statistics and the unnormalised output of the partition -> the partial buffers in global memory
template <int HDT, int BST>
__device__ __forceinline__ void attn_fused_core(const etxb_attnf_args& d, const AttnSmem& s, int part, int h, int ntok) {
  const int HD = HDT ? HDT : d.HD, BS = BST ? BST : d.BS;
  constexpr int X = 8, P = ETXB_ATTN_PART;
  const int G = d.NH / d.NKV, nblk = P / BS, hx = HD / X;
  const int lane = tidx() & 31, warp = tidx() >> 5;
  for (int idx = tidx(); idx < G * 2 * P; idx += ETXB_CONSUMERS) {  // idx -> (g, half of the head dimension, t)
    const int t = idx % P, hf = (idx / P) & 1, g = idx / (2 * P);
    float acc = 0.f;
    if (t < ntok) {
      const int b = t / BS, o = t % BS;
      const __nv_bfloat16* kb = s.ks + (size_t)b * HD * BS;
      const float* qg = s.qs + g * HD;
#pragma unroll 2
      for (int dg = hf * (hx / 2); dg < (hf + 1) * (hx / 2); ++dg) {
        const uint4 kv = *(const uint4*)(kb + ((size_t)dg * BS + o) * X);
        const float4 qa = *(const float4*)(qg + dg * X), qb = *(const float4*)(qg + dg * X + 4);
        acc = __fmaf_rn(bf_lo(kv.x), qa.x, acc); acc = __fmaf_rn(bf_hi(kv.x), qa.y, acc);
        acc = __fmaf_rn(bf_lo(kv.y), qa.z, acc); acc = __fmaf_rn(bf_hi(kv.y), qa.w, acc);
        acc = __fmaf_rn(bf_lo(kv.z), qb.x, acc); acc = __fmaf_rn(bf_hi(kv.z), qb.y, acc);
        acc = __fmaf_rn(bf_lo(kv.w), qb.z, acc); acc = __fmaf_rn(bf_hi(kv.w), qb.w, acc);
      }
    }
    s.ph[hf * 16 * P + g * P + t] = acc;
  }
  csync();
  for (int g = warp; g < G; g += ETXB_NWARPS) {                      // one warp per q head, lane = position (P == 32)
    const float sv = lane < ntok ? __fmul_rn(__fadd_rn(s.ph[g * P + lane], s.ph[16 * P + g * P + lane]), d.scale) : -INFINITY;
    const float m = warp_max(sv);
    const float pr = lane < ntok ? expf(__fsub_rn(sv, m)) : 0.f;
    const float l = warp_sum(pr);
    s.sc[g * P + lane] = pr;
    if (lane == 0) { s.st[2 * g] = m; s.st[2 * g + 1] = l; }
  }
  csync();
  for (int idx = tidx(); idx < G * HD; idx += ETXB_CONSUMERS) {      // idx -> (g, dd): o = sum_t p[t] * V[t][dd], t ascending
    const int dd = idx % HD, g = idx / HD;
    float acc = 0.f;
    for (int b = 0; b < nblk; ++b) {
      if (b * BS >= ntok) break;
      const __nv_bfloat16* vb = s.vs + ((size_t)b * HD + dd) * BS;
      const float* pg = s.sc + g * P + b * BS;
      const int lim = min(BS, ntok - b * BS);
      if (BST == 16) {                                             // a 32-byte row: two vector reads; positions past ntok have p = 0
        float f[16];
        unpack8(*(const uint4*)vb, f); unpack8(*(const uint4*)(vb + 8), f + 8);
#pragma unroll
        for (int o = 0; o < 16; ++o) if (o < lim) acc = __fmaf_rn(pg[o], f[o], acc);
      } else {
        for (int o = 0; o < lim; ++o) acc = __fmaf_rn(pg[o], __bfloat162float(vb[o]), acc);
      }
    }
    const int hq = h * G + g;
    d.tmp_out[((size_t)hq * d.max_parts + part) * HD + dd] = acc;
    if (dd == 0) {
      d.max_logits[(size_t)hq * d.max_parts + part] = s.st[2 * g];
      d.exp_sums[(size_t)hq * d.max_parts + part] = s.st[2 * g + 1];
    }
  }
}

// out[hq][:] = bf16(sum_p w_p * tmp[p][:] / sum_p w_p * l_p), w_p = exp(m_p - max m), for the G q heads of kv head h.
// Run by the last task of the kv head; reads the partials the other CTAs wrote (L2).  G * np <= 8192.
__device__ __noinline__ void attn_fused_merge(const etxb_attnf_args& d, const Smem& sm, int h, int np, int HD) {
  const int G = d.NH / d.NKV, lane = tidx() & 31, warp = tidx() >> 5;
  float* wl = sm.xs;                                              // [G][np] max logits, then weights
  float* es = sm.xs + 8192;                                       // [G][np] exp sums
  float* red = sm.scr + 200;                                      // [G] denominators
  for (int i = tidx(); i < G * np; i += ETXB_CONSUMERS) {
    const int g = i / np, pp = i - g * np;
    wl[i] = __ldcg(d.max_logits + (size_t)(h * G + g) * d.max_parts + pp);
    es[i] = __ldcg(d.exp_sums + (size_t)(h * G + g) * d.max_parts + pp);
  }
  csync();
  mark(sm, 0);
  for (int g = warp; g < G; g += ETXB_NWARPS) {
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
  // weighted sum of the partials: a thread owns four consecutive output values (16-byte loads) and every groups-th
  // partition; the groups' sums are then added left to right.  A fixed order, so the result is reproducible.
  const int quads = G * HD / 4, groups = ETXB_CONSUMERS / quads > 0 ? ETXB_CONSUMERS / quads : 1;
  float* part = sm.xs + 12288;                                    // [groups][G * HD] = 2048 floats, over the exp sums (dead by now)
  for (int item = tidx(); item < quads * groups; item += ETXB_CONSUMERS) {
    const int qd = item % quads, grp = item / quads;
    const int g = (4 * qd) / HD, dd = 4 * qd - g * HD;
    const float* tp = d.tmp_out + (size_t)(h * G + g) * d.max_parts * HD + dd;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p0 = grp; p0 < np; p0 += 4 * groups) {
      float4 v[4]; float w[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int pp = p0 + u * groups;
        const int pc = pp < np ? pp : np - 1;                      // clamped: the weight of a padded load is zero
        v[u] = __ldcg((const float4*)(tp + (size_t)pc * HD));
        w[u] = pp < np ? wl[g * np + pp] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        o.x = __fmaf_rn(w[u], v[u].x, o.x); o.y = __fmaf_rn(w[u], v[u].y, o.y);
        o.z = __fmaf_rn(w[u], v[u].z, o.z); o.w = __fmaf_rn(w[u], v[u].w, o.w);
      }
    }
    *(float4*)(part + (size_t)grp * G * HD + 4 * qd) = o;
  }
  csync();
  mark(sm, 2);
  for (int idx = tidx(); idx < G * HD; idx += ETXB_CONSUMERS) {
    const int g = idx / HD;
    float o = 0.f;
    for (int grp = 0; grp < groups; ++grp) o = __fadd_rn(o, part[(size_t)grp * G * HD + idx]);
    ((__nv_bfloat16*)d.out)[(size_t)h * G * HD + idx] = __float2bfloat16_rn(__fdiv_rn(o, red[g]));
  }
}

template <int HDT, int BST>
__device__ __noinline__ void attn_fused_impl(const etxb_attnf_args& d, int blk, const Smem& sm, const etxb_stepv& S) {
  const int HD = HDT ? HDT : d.HD;
  const int NKV = d.NKV, G = d.NH / NKV, P = ETXB_ATTN_PART;
  const int part = blk / NKV, h = blk - part * NKV;
  // the step's own buffers hold what the prologue wrote from the step parameters: take the values from there
  const long long pos = (const void*)d.positions == (const void*)S.positions ? (long long)S.pos : __ldcg((const long long*)d.positions);
  const long long slot = (const void*)d.slot_mapping == (const void*)S.slot_mapping ? (long long)S.pos : __ldcg((const long long*)d.slot_mapping);
  const int seq = (const void*)d.seq_lens == (const void*)S.seq_lens ? S.pos + 1 : __ldcg(d.seq_lens);
  const int t0 = part * P;
  int* flag = (int*)(sm.scr + 130);
  if (t0 < seq) {
    const AttnSmem s = attn_smem(sm.xs, G, HD);
    const bool owner = pos >= t0 && pos < t0 + P;                 // this partition holds the position being written
    attn_fused_load<HDT, BST>(d, s, part, h, seq, pos, owner);
    csync();
    mark(sm, 0);
    attn_fused_prep<HDT, BST>(d, s, part, h, pos, slot, owner);
    csync();
    mark(sm, 1);
    attn_fused_core<HDT, BST>(d, s, part, h, min(P, seq - t0));
  }
  csync();                                                         // the partials of this task are issued
  mark(sm, 2);
  if (tidx() == 0) {
    __threadfence();
    const int old = atomicAdd(d.counters + h, 1);                  // monotonic: max_parts arrivals per step and kv head
    *flag = ((old + 1) % d.max_parts) == 0;
    if (*flag) __threadfence();
  }
  csync();
  mark(sm, 3);
  // partitions that were computed: never more than the grid holds, whatever seq_lens says (a context past
  // max_parts * 32 positions is the caller's error: the positions beyond are left out, nothing is read past the partials)
  if (*flag) attn_fused_merge(d, sm, h, min((seq + P - 1) / P, d.max_parts), HD);
}

__device__ __forceinline__ void tile_attn_fused(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_attnf_args& d = *(const etxb_attnf_args*)a;
  if (blk >= (int)d.nblocks) return;
  if (d.HD == 128 && d.BS == 16) attn_fused_impl<128, 16>(d, blk, sm, S);
  else attn_fused_impl<0, 0>(d, blk, sm, S);
}

}  // namespace etxb
