// Absorbed multi-head latent attention (DeepSeek-V2 family), one decode step, one task per head.
//
// The latent cache holds ONE row per position, shared by all heads: c (kv_lora values, RMS-normed) | k_pe (qk_rope
// values, rotated).  W_UK is folded into the query and W_UV into the output:
//   q_c[h] = q_nope[h] W_UK[h];   s[h][t] = scale (q_c[h] . c[t] + q_pe[h] . k_pe[t]);   p = softmax_t(s);
//   o_c[h] = sum_t p[t] c[t];     out[h] = W_UV[h] o_c[h]
// It stands where the reference's DeepSeek-V2-Lite graph runs the tasks q_absorb, attention (16 heads x 16 KV chunks),
// merge_uv (examples/dsv2lite/graph.py:98-209); the arithmetic follows the archived NumPy reference of that model,
// attention_absorbed (examples/dsv2lite/results/2026-10-14-k1/b_alld4r0l1kvs_stamps/fleet_src/host/reference_decode.py:207-253):
// bf16 q / kv_a rows, RMSNorm rounded twice on the latent, interleave-then-rotate rope with fp32 YaRN tables rounded to
// bf16 after the rotation, fp32 scores / softmax / sums, bf16 output.
//
// A task (head h) does everything for its head over the whole context: the new position's latent row is computed by
// every task from the kv_a row (576 values: cheaper than a phase of its own) and used from shared memory, head 0 also
// stores it into the cache; the cached rows come from L2 (16 heads read the same 1152-byte rows).  16 tasks leave most
// SMs idle during this phase: the phase is short (the cache of a 1K context is 1.2 MB) and a partitioned form with a
// merge is the known next step.
#pragma once
#include "etxb_gemv.cuh"

namespace etxb {

#define ETXB_MLA_MAXCTX 8192   // positions whose scores fit the tile's shared memory

struct etxb_mla_args {
  const void* qkv;             // 0   bf16 [NH * (DN + DR) + C + DR]: the q heads (nope | rope part each), then the kv_a row (c | k_pe)
  const void* kvln;            // 8   bf16 [C]: weight of the latent's RMSNorm
  const void* cos_sin;         // 16  fp32 [maxlen][2 * DR]: cos | sin rows of the rotary table (YaRN: already scaled)
  const void* wkvb;            // 24  bf16 [NH * (DN + DV)][C]: per head DN rows of W_UK, then DV rows of W_UV
  void* cache;                 // 32  bf16 [maxlen][C + DR]: the layer's latent cache
  const int64_t* positions;    // 40
  void* out;                   // 48  bf16 [NH * DV]
  int32_t NH, C, DN, DR, DV, maxlen;   // 56..79
  float scale, eps;            // 80..87
  int32_t pad[2];              // 88..95
  uint32_t grid[3], nblocks;   // 96..111
};

__device__ __noinline__ void tile_mla_attn(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_mla_args& d = *(const etxb_mla_args*)a;
  if (blk >= (int)d.nblocks || blk >= d.NH) return;
  const int h = blk, C = d.C, DN = d.DN, DR = d.DR, DV = d.DV, QH = DN + DR, ROW = C + DR;
  const long long pos = (const void*)d.positions == (const void*)S.positions ? (long long)S.pos : __ldcg((const long long*)d.positions);
  if (pos < 0 || pos >= d.maxlen || pos >= ETXB_MLA_MAXCTX) return;
  const int seq = (int)pos + 1;
  const int tid = tidx(), lane = tid & 31, warp = tid >> 5;
  float* qf = sm.xs;            // [QH <= 256] this head's q row
  float* kvf = qf + 256;        // [ROW <= 640] the raw kv_a row
  float* cn = kvf + 640;        // [C <= 512] the new position's latent (bf16 values)
  float* kpn = cn + 512;        // [DR <= 64] its rotated k_pe (bf16 values)
  float* qpe = kpn + 64;        // [DR] this head's rotated q_pe (bf16 values)
  float* cs = qpe + 64;         // [2 DR] cos | sin of the position
  float* qc = cs + 128;         // [C] q_nope W_UK
  float* oc = qc + 512;         // [2][C] softmax-weighted latent, two halves of the positions
  float* red = oc + 1024;       // [64]
  float* sc = red + 64;         // [seq] scores, then probabilities
  const __nv_bfloat16* qkv = (const __nv_bfloat16*)d.qkv;
  for (int i = tid; i < QH + ROW + 2 * DR; i += ETXB_CONSUMERS) {
    if (i < QH) qf[i] = ld_bf(qkv, (size_t)h * QH + i);
    else if (i < QH + ROW) kvf[i - QH] = ld_bf(qkv, (size_t)d.NH * QH + (i - QH));
    else cs[i - QH - ROW] = __ldg((const float*)d.cos_sin + (size_t)pos * 2 * DR + (i - QH - ROW));
  }
  csync();
  // ---- the new position's cache row: latent = rmsnorm(kv_a[:C]) (rounded twice), k_pe = rope(kv_a[C:]); this head's q_pe
  const float ss = sumsq_numpy_order(kvf, C, red);
  const float r = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(ss, (float)C), d.eps)));
  for (int i = tid; i < C; i += ETXB_CONSUMERS)
    cn[i] = bfr(__fmul_rn(bfr(__fmul_rn(kvf[i], r)), __bfloat162float(__ldg((const __nv_bfloat16*)d.kvln + i))));
  if (tid < 2 * DR) {
    // de-interleave (even elements first, then odd), then the half rotation: y cos + rot(y) sin
    const int i = tid < DR ? tid : tid - DR, half = DR >> 1;
    const float* x = tid < DR ? kvf + C : qf + DN;
    const float y = i < half ? x[2 * i] : x[2 * (i - half) + 1];
    const float rot = i < half ? -x[2 * i + 1] : x[2 * (i - half)];
    const float v = bfr(__fadd_rn(__fmul_rn(y, cs[i]), __fmul_rn(rot, cs[DR + i])));
    (tid < DR ? kpn : qpe)[i] = v;
  }
  csync();
  if (h == 0) {
    __nv_bfloat16* row = (__nv_bfloat16*)d.cache + (size_t)pos * ROW;
    for (int i = tid; i < ROW; i += ETXB_CONSUMERS) row[i] = __float2bfloat16_rn(i < C ? cn[i] : kpn[i - C]);
  }
  // ---- q_c[j] = sum_i q_nope[i] W_UK[h][i][j]: thread pairs of columns, rows in ascending order
  const __nv_bfloat16* wuk = (const __nv_bfloat16*)d.wkvb + (size_t)h * (DN + DV) * C;
  for (int j2 = tid; j2 < (C >> 1); j2 += ETXB_CONSUMERS) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
    for (int i = 0; i < DN; ++i) {
      const uint32_t w = __ldg((const uint32_t*)(wuk + (size_t)i * C) + j2);
      a0 = __fmaf_rn(qf[i], bf_lo(w), a0);
      a1 = __fmaf_rn(qf[i], bf_hi(w), a1);
    }
    qc[2 * j2] = a0; qc[2 * j2 + 1] = a1;
  }
  csync();
  // ---- scores: one warp per position, a lane takes element pairs 2 lane + 64 k of the row (latent part against q_c,
  //      rope part against q_pe); the new position's row comes from shared memory
  const __nv_bfloat16* cache = (const __nv_bfloat16*)d.cache;
  const int npair = ROW >> 1;
  for (int t = warp; t < seq; t += ETXB_CONSUMER_WARPS) {
    float acc = 0.f;
    if (t == (int)pos) {
      for (int e = 2 * lane; e < ROW; e += 64) {
        const float x0 = e < C ? cn[e] : kpn[e - C], x1 = e + 1 < C ? cn[e + 1] : kpn[e + 1 - C];
        acc = __fmaf_rn(x0, e < C ? qc[e] : qpe[e - C], acc);
        acc = __fmaf_rn(x1, e + 1 < C ? qc[e + 1] : qpe[e + 1 - C], acc);
      }
    } else {
      const uint32_t* row = (const uint32_t*)(cache + (size_t)t * ROW);
      uint32_t w[10];
#pragma unroll
      for (int k = 0; k < 10; ++k) w[k] = lane + 32 * k < npair ? __ldcg(row + lane + 32 * k) : 0u;
#pragma unroll
      for (int k = 0; k < 10; ++k) {
        const int e = 2 * lane + 64 * k;
        if (e < ROW) {
          acc = __fmaf_rn(bf_lo(w[k]), e < C ? qc[e] : qpe[e - C], acc);
          acc = __fmaf_rn(bf_hi(w[k]), e + 1 < C ? qc[e + 1] : qpe[e + 1 - C], acc);
        }
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) sc[t] = __fmul_rn(acc, d.scale);
  }
  csync();
  // ---- softmax over the positions
  float m = -INFINITY;
  for (int t = tid; t < seq; t += ETXB_CONSUMERS) m = fmaxf(m, sc[t]);
  m = warp_max(m);
  if (lane == 0) red[warp] = m;
  csync();
  m = red[0];
  for (int w = 1; w < ETXB_CONSUMER_WARPS; ++w) m = fmaxf(m, red[w]);
  csync();
  float l = 0.f;
  for (int t = tid; t < seq; t += ETXB_CONSUMERS) { const float e = expf(__fsub_rn(sc[t], m)); sc[t] = e; l = __fadd_rn(l, e); }
  l = block_sum(l, red);
  for (int t = tid; t < seq; t += ETXB_CONSUMERS) sc[t] = __fdiv_rn(sc[t], l);
  csync();
  // ---- o_c[j] = sum_t p[t] c[t][j]: threads 0..255 take the even positions, 256..511 the odd ones, a column pair each
  {
    const int half = tid >> 8, j2 = tid & 255;
    float a0 = 0.f, a1 = 0.f;
    if (j2 < (C >> 1)) {
#pragma unroll 4
      for (int t = half; t < seq; t += 2) {
        float x0, x1;
        if (t == (int)pos) { x0 = cn[2 * j2]; x1 = cn[2 * j2 + 1]; }
        else { const uint32_t w = __ldcg((const uint32_t*)(cache + (size_t)t * ROW) + j2); x0 = bf_lo(w); x1 = bf_hi(w); }
        a0 = __fmaf_rn(sc[t], x0, a0);
        a1 = __fmaf_rn(sc[t], x1, a1);
      }
      oc[half * 512 + 2 * j2] = a0; oc[half * 512 + 2 * j2 + 1] = a1;
    }
  }
  csync();
  for (int j = tid; j < C; j += ETXB_CONSUMERS) oc[j] = __fadd_rn(oc[j], oc[512 + j]);
  csync();
  // ---- out[v] = W_UV[h][v] . o_c: a warp per output row, lanes over the columns
  const __nv_bfloat16* wuv = wuk + (size_t)DN * C;
  for (int v = warp; v < DV; v += ETXB_CONSUMER_WARPS) {
    float acc = 0.f;
    for (int j = 8 * lane; j < C; j += 256) {
      const uint4 w = __ldg((const uint4*)(wuv + (size_t)v * C + j));
      const float wf[8] = {bf_lo(w.x), bf_hi(w.x), bf_lo(w.y), bf_hi(w.y), bf_lo(w.z), bf_hi(w.z), bf_lo(w.w), bf_hi(w.w)};
#pragma unroll
      for (int u = 0; u < 8; ++u) acc = __fmaf_rn(wf[u], oc[j + u], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) ((__nv_bfloat16*)d.out)[(size_t)h * DV + v] = __float2bfloat16_rn(acc);
  }
  csync();
}

}  // namespace etxb
