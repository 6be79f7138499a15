// Attention side of the decode step: q/k RMSNorm + rotary + paged KV-cache write of one kv head, split-KV paged GQA
// decode attention over ETXB_ATTN_PART positions per task, and the merge of the partitions.
//
// Reference functions these take over:
//   dsl_attnprep                       etx/ops/attnprep.py:86-211 (task = kv head, in place on qkv, cache layout
//                                      key [blocks][NKV][HD/X][BS][X], value [blocks][NKV][HD][BS], attnprep.py:3-6, 146-165)
//   paged attention + reduce           imported vLLM kernels, call recipe etx/importer/spec.py:243-244,
//                                      grid examples/vllm_llm/model.py:78-84, 358-362
// Numerics follow examples/llm/ref_numpy.py:113-129: RMSNorm rounded twice, each rotary product rounded and their sum
// rounded, scores and softmax in fp32 over the whole context, one bf16 rounding of the attention output.
#pragma once
#include "etxb_prims.cuh"
#include "etxb_gemv.cuh"

namespace etxb {

// sum of squares of one head (n = 64, 128 or 256 values in shared memory) in numpy's pairwise order; one warp.
__device__ __forceinline__ float head_sumsq(const float* x, int n) {
  const int lane = tidx() & 31;
  if (n != 64 && n != 128 && n != 256) {
    float s = 0.f;
    for (int i = lane; i < n; i += 32) s = __fmaf_rn(x[i], x[i], s);
    return warp_sum(s);
  }
  const int iters = (n < 128 ? n : 128) >> 3, nacc = n <= 128 ? 8 : n >> 4;
  float r = 0.f;
  if (lane < nacc) {
    const float* b = x + (lane >> 3) * 128 + (lane & 7);
    r = __fmul_rn(b[0], b[0]);
    for (int i = 1; i < iters; ++i) r = __fadd_rn(r, __fmul_rn(b[8 * i], b[8 * i]));
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, o));
  return r;
}

// task h = kv head: warps 0..G-1 do the q heads h*G + w, warp G the k head (both in place on qkv; k also into the
// cache), warp G+1 copies the v row into the cache.  G + 2 <= 16, HD a multiple of 32 and <= 256.
__device__ __noinline__ void tile_attnprep(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_attnprep_args& d = *(const etxb_attnprep_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int h = blk, NH = d.NH, NKV = d.NKV, HD = d.HD, G = NH / NKV, BS = d.BS, X = d.X;
  const int lane = tidx() & 31, warp = tidx() >> 5;
  // the step's own buffers hold what the prologue wrote from the step parameters: take the values from there
  const long long pos = (const void*)d.positions == (const void*)S.positions ? (long long)S.pos : __ldcg((const long long*)d.positions);
  const long long slot = (const void*)d.slot_mapping == (const void*)S.slot_mapping ? (long long)S.pos : __ldcg((const long long*)d.slot_mapping);
  const long long cb = slot / BS; const int off = (int)(slot % BS);
  __nv_bfloat16* qkv = (__nv_bfloat16*)d.qkv;
  const int half = HD >> 1, epl = HD >> 5;                       // elements per lane, contiguous
  if (warp <= G) {
    const bool isk = warp == G;
    __nv_bfloat16* row = qkv + (size_t)(isk ? NH + h : h * G + warp) * HD;
    const __nv_bfloat16* nw = (const __nv_bfloat16*)(isk ? d.kw : d.qw);
    float* xh = sm.xs + warp * 256;
    float v[8];
    for (int j = 0; j < epl; ++j) { v[j] = ld_bf(row, lane * epl + j); xh[lane * epl + j] = v[j]; }
    __syncwarp();
    if (nw != nullptr) {
      const float ss = head_sumsq(xh, HD);
      const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)HD), d.eps)));
      for (int j = 0; j < epl; ++j) v[j] = bfr(__fmul_rn(__bfloat162float(nw[lane * epl + j]), bfr(__fmul_rn(v[j], r))));
    }
    const __nv_bfloat16* cs = (const __nv_bfloat16*)d.cos_sin + (size_t)pos * HD;
    float o[8];
    for (int j = 0; j < epl; ++j) {
      const int dd = lane * epl + j;
      const float other = __shfl_xor_sync(0xffffffffu, v[j], 16);  // element dd +- HD/2 lives 16 lanes away
      const float rot = dd < half ? -other : other;
      const float c = __bfloat162float(cs[dd % half]), s = __bfloat162float(cs[half + dd % half]);
      o[j] = bfr(__fadd_rn(bfr(__fmul_rn(v[j], c)), bfr(__fmul_rn(rot, s))));
    }
    for (int j = 0; j < epl; ++j) row[lane * epl + j] = __float2bfloat16_rn(o[j]);
    if (isk) {
      __nv_bfloat16* kc = (__nv_bfloat16*)d.kc;
      for (int j = 0; j < epl; ++j) {
        const int dd = lane * epl + j;
        kc[(((size_t)cb * NKV + h) * (HD / X) + dd / X) * BS * X + (size_t)off * X + dd % X] = __float2bfloat16_rn(o[j]);
      }
    }
  } else if (warp == G + 1) {
    const __nv_bfloat16* row = qkv + (size_t)(NH + NKV + h) * HD;
    __nv_bfloat16* vc = (__nv_bfloat16*)d.vc;
    for (int dd = lane; dd < HD; dd += 32)
      vc[(((size_t)cb * NKV + h) * HD + dd) * BS + off] = __float2bfloat16_rn(ld_bf(row, dd));
  }
}

// task blk = part * NKV + h: positions [part*32, part*32 + 32) of kv head h against its G q heads.
// Writes, per q head, the partition's max logit, exp sum and unnormalised output (fp32).  HD <= 256, HD % 8 == 0,
// BS 16 or 32, X 8.
__device__ __noinline__ void tile_attn(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_attn_args& d = *(const etxb_attn_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int NKV = d.NKV, HD = d.HD, G = d.NH / NKV, BS = d.BS, X = d.X, P = ETXB_ATTN_PART;
  const int part = blk / NKV, h = blk - part * NKV;
  const int seq = (const void*)d.seq_lens == (const void*)S.seq_lens ? S.pos + 1 : __ldcg(d.seq_lens);
  const int t0 = part * P;
  if (t0 >= seq) return;
  const int ntok = min(P, seq - t0);
  const int nblk = P / BS;
  float* qs = sm.xs;                                              // [G][HD] floats
  __nv_bfloat16* ks = (__nv_bfloat16*)(sm.xs + 16 * 256);         // [nblk][HD/X][BS][X]
  __nv_bfloat16* vs = ks + P * 256;                               // [nblk][HD][BS]
  float* sc = (float*)(vs + P * 256);                             // [G][P]
  float* st = sc + 16 * P;                                        // per head: max, sum
  // q rows
  const __nv_bfloat16* q = (const __nv_bfloat16*)d.q;
  for (int i = tidx(); i < G * HD; i += ETXB_CONSUMERS) qs[i] = ld_bf(q, (size_t)h * G * HD + i);
  // K and V blocks: HD * BS bf16 each, contiguous per (block, head)
  const int vec_per_blk = HD * BS / 8;
  for (int i = tidx(); i < nblk * vec_per_blk; i += ETXB_CONSUMERS) {
    const int b = i / vec_per_blk, r = i - b * vec_per_blk;
    const int lb = t0 / BS + b;
    if (lb * BS < seq) {
      const long long pb = __ldg(d.block_tables + lb);
      const size_t base = ((size_t)pb * NKV + h) * HD * BS;
      *(uint4*)(ks + (size_t)b * HD * BS + 8 * r) = ld_act16((const __nv_bfloat16*)d.kc + base + 8 * r);
      *(uint4*)(vs + (size_t)b * HD * BS + 8 * r) = ld_act16((const __nv_bfloat16*)d.vc + base + 8 * r);
    }
  }
  csync();
  // scores: idx -> (g, half, t); the two halves of the head dimension are added left to right, then scaled
  const int hx = HD / X;                                          // 8-element groups per head
  float* ph = st + 64;                                            // [2][16 * P] half dot products
  for (int idx = tidx(); idx < G * 2 * P; idx += ETXB_CONSUMERS) {
    const int t = idx % P, hf = (idx / P) & 1, g = idx / (2 * P);
    float acc = 0.f;
    if (t < ntok) {
      const int b = t / BS, o = t % BS;
      const __nv_bfloat16* kb = ks + (size_t)b * HD * BS;
      for (int dg = hf * (hx / 2); dg < (hf + 1) * (hx / 2); ++dg) {
        const uint4 kv = *(const uint4*)(kb + ((size_t)dg * BS + o) * X);
        const float* qq = qs + g * HD + dg * X;
        acc = __fmaf_rn(bf_lo(kv.x), qq[0], acc); acc = __fmaf_rn(bf_hi(kv.x), qq[1], acc);
        acc = __fmaf_rn(bf_lo(kv.y), qq[2], acc); acc = __fmaf_rn(bf_hi(kv.y), qq[3], acc);
        acc = __fmaf_rn(bf_lo(kv.z), qq[4], acc); acc = __fmaf_rn(bf_hi(kv.z), qq[5], acc);
        acc = __fmaf_rn(bf_lo(kv.w), qq[6], acc); acc = __fmaf_rn(bf_hi(kv.w), qq[7], acc);
      }
    }
    ph[hf * 16 * P + g * P + t] = acc;
  }
  csync();
  for (int i = tidx(); i < G * P; i += ETXB_CONSUMERS)
    sc[i] = (i % P) < ntok ? __fmul_rn(__fadd_rn(ph[i], ph[16 * P + i]), d.scale) : -INFINITY;
  csync();
  // softmax statistics per q head (one warp per head, P == 32 lanes)
  for (int g = tidx() >> 5; g < G; g += ETXB_NWARPS) {
    const int lane = tidx() & 31;
    const float s = sc[g * P + lane];
    const float m = warp_max(s);
    const float p = lane < ntok ? expf(__fsub_rn(s, m)) : 0.f;
    const float l = warp_sum(p);
    sc[g * P + lane] = p;
    if (lane == 0) { st[2 * g] = m; st[2 * g + 1] = l; }
  }
  csync();
  // output: idx -> (g, dd); o = sum_t p[t] * V[t][dd], positions in ascending order
  for (int idx = tidx(); idx < G * HD; idx += ETXB_CONSUMERS) {
    const int dd = idx % HD, g = idx / HD;
    float acc = 0.f;
    for (int b = 0; b < nblk; ++b) {
      if (b * BS >= ntok) break;
      const __nv_bfloat16* vb = vs + ((size_t)b * HD + dd) * BS;
      const int lim = min(BS, ntok - b * BS);
      for (int o = 0; o < lim; ++o) acc = __fmaf_rn(sc[g * P + b * BS + o], __bfloat162float(vb[o]), acc);
    }
    const int hq = h * G + g;
    d.tmp_out[((size_t)hq * d.max_parts + part) * HD + dd] = acc;
    if (dd == 0) {
      d.max_logits[(size_t)hq * d.max_parts + part] = st[2 * g];
      d.exp_sums[(size_t)hq * d.max_parts + part] = st[2 * g + 1];
    }
  }
}

// task blk = q head: out[hq][:] = bf16(sum_p w_p * tmp[p][:] / sum_p w_p * l_p), w_p = exp(m_p - max m).
__device__ __noinline__ void tile_attn_reduce(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_attn_args& d = *(const etxb_attn_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int HD = d.HD, hq = blk, P = ETXB_ATTN_PART;
  const int seq = (const void*)d.seq_lens == (const void*)S.seq_lens ? S.pos + 1 : __ldcg(d.seq_lens);
  const int np = (seq + P - 1) / P;
  float* wp = sm.xs;                                              // [np] max logits, then weights
  float* es = sm.xs + 4096;                                       // [np] exp sums
  float* acc4 = sm.xs + 8192;                                     // [groups][HD]
  float* red = sm.scr;
  const int lane = tidx() & 31;
  for (int p = tidx(); p < np; p += ETXB_CONSUMERS) {
    wp[p] = __ldcg(d.max_logits + (size_t)hq * d.max_parts + p);
    es[p] = __ldcg(d.exp_sums + (size_t)hq * d.max_parts + p);
  }
  csync();
  if (tidx() < 32) {
    float m = -INFINITY;
    for (int p = lane; p < np; p += 32) m = fmaxf(m, wp[p]);
    m = warp_max(m);
    if (lane == 0) red[41] = m;
  }
  csync();
  const float m = red[41];
  for (int p = tidx(); p < np; p += ETXB_CONSUMERS) wp[p] = expf(__fsub_rn(wp[p], m));
  csync();
  if (tidx() < 32) {
    float L = 0.f;
    for (int p = lane; p < np; p += 32) L = __fmaf_rn(wp[p], es[p], L);
    L = warp_sum(L);
    if (lane == 0) red[40] = L;
  }
  const int groups = ETXB_CONSUMERS / HD > 0 ? ETXB_CONSUMERS / HD : 1;
  const int dd = tidx() % HD, pg = tidx() / HD;
  if (pg < groups) {
    float o = 0.f;
    for (int p = pg; p < np; p += groups) o = __fmaf_rn(wp[p], __ldcg(d.tmp_out + ((size_t)hq * d.max_parts + p) * HD + dd), o);
    acc4[pg * HD + dd] = o;
  }
  csync();
  if (tidx() < HD) {
    float o = 0.f;
    for (int g2 = 0; g2 < groups; ++g2) o = __fadd_rn(o, acc4[g2 * HD + tidx()]);
    ((__nv_bfloat16*)d.out)[(size_t)hq * HD + tidx()] = __float2bfloat16_rn(__fdiv_rn(o, red[40]));
  }
}

}  // namespace etxb
