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
// A task is (head h, partition of 128 positions): 16 heads x 9 partitions fill the SMs at a 1K context (one task per head
// over the whole context took 73 us per layer; this form takes a quarter of that).  Every task computes the new
// position's latent row from the kv_a row (576 values: cheaper than a phase of its own) and uses it from shared
// memory -- the task (head 0, last partition) also stores it into the cache --, folds W_UK into its head's query, and
// produces its partition's softmax statistics and weighted latent.  The partials travel as flagged (value, step) pairs
// like those of the grouped GQA tile (etxb_attn_gq.cuh); four finishing tasks per head, placed after the partition tasks
// in the grid, poll them, merge them in ascending partition order and apply a quarter of W_UV's rows each.  The cached
// rows come from L2 (all heads read the same rows).
#pragma once
#include "etxb_attn_gq.cuh"

namespace etxb {

#define ETXB_MLA_MAXCTX 8192   // longest context (64 partitions)
#define ETXB_MLA_PART 128      // positions per task
#define ETXB_MLA_FIN 4         // finishing tasks per head: each merges the head's partials and applies a quarter of W_UV's rows

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
  void* tmp;                   // 88  (value, flag) pairs [NH][max_parts][C + 8]: weighted latent, then max logit and exp sum
  int32_t max_parts, tag;      // 96, 100: partitions the grid covers (tasks = (max_parts + 4) * NH: partitions, then finishing tasks); tag tells the layers that share tmp apart
  int32_t pad[2];              // 104..111
  uint32_t grid[3], nblocks;   // 112..127
};

// A finishing task of head h: waits (bounded) for the head's np partials, merges them -- weights exp(m_p - max m),
// partitions in ascending order -- and applies rows [f * DV / FIN, ..) of W_UV.  The finishing tasks come after the
// partition tasks in the grid, so whatever they wait for runs on another worker or ran before them on their own; the
// partition tasks never wait.  Four tasks per head instead of one cut the tail of the phase (merge + all of W_UV by the
// last partition's task: 15 us) to a third.
__device__ __forceinline__ void mla_finish(const etxb_mla_args& d, const Smem& sm, int h, int f, int np) {
  const int C = d.C, DN = d.DN, DV = d.DV, PW = C + 8;
  const int tid = tidx(), lane = tid & 31, warp = tid >> 5;
  const uint32_t fl = pair_flag(sm.epoch, d.tag << 16);
  float* oc = sm.xs;                                               // [C] merged, normalised latent
  float* wl = oc + 512;                                            // [np <= 64] max logits, then weights
  float* es = wl + 64;                                             // [np] exp sums
  float* red = es + 64;
  const __nv_bfloat16* wuv = (const __nv_bfloat16*)d.wkvb + ((size_t)h * (DN + DV) + DN) * C;
  const int v_lo = f * ((DV + ETXB_MLA_FIN - 1) / ETXB_MLA_FIN), v_hi = min(DV, v_lo + (DV + ETXB_MLA_FIN - 1) / ETXB_MLA_FIN);
  // this task's rows of W_UV travel while it waits for the partials
  uint4 w[2][2];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int v = v_lo + warp + r * ETXB_CONSUMER_WARPS, j = 8 * lane + 256 * k;
      w[r][k] = (v < v_hi && j < C) ? __ldg((const uint4*)(wuv + (size_t)v * C + j)) : make_uint4(0u, 0u, 0u, 0u);
    }
  const uint2* ph = (const uint2*)d.tmp + (size_t)h * d.max_parts * PW;
  for (int q = tid; q < np; q += ETXB_CONSUMERS) {
    wl[q] = poll_pair(ph + (size_t)q * PW + C, fl, sm);
    es[q] = poll_pair(ph + (size_t)q * PW + C + 1, fl, sm);
  }
  csync();
  if (warp == 0) {
    float mm = -INFINITY;
    for (int q = lane; q < np; q += 32) mm = fmaxf(mm, wl[q]);
    mm = warp_max(mm);
    float L = 0.f;
    for (int q = lane; q < np; q += 32) {
      const float wq = expf(__fsub_rn(wl[q], mm));
      wl[q] = wq;
      L = __fmaf_rn(wq, es[q], L);
    }
    L = warp_sum(L);
    if (lane == 0) red[0] = L;
  }
  csync();
  for (int j = tid; j < C; j += ETXB_CONSUMERS) {
    float o = 0.f;
    for (int q0 = 0; q0 < np; q0 += 8) {                             // eight partitions' pairs requested at once
      uint2 first[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) first[u] = ld_pair(ph + (size_t)min(q0 + u, np - 1) * PW + j);
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (q0 + u < np) o = __fmaf_rn(wl[q0 + u], first[u].y == fl ? __uint_as_float(first[u].x) : poll_pair(ph + (size_t)(q0 + u) * PW + j, fl, sm), o);
    }
    oc[j] = __fdiv_rn(o, red[0]);
  }
  csync();
  // ---- out[v] = W_UV[h][v] . o_c: a warp per output row, lanes over the columns
  for (int r = 0; r < 2; ++r) {
    const int v = v_lo + warp + r * ETXB_CONSUMER_WARPS;
    float acc = 0.f;
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int j = 8 * lane + 256 * k;
      if (j < C) {
        const uint4 x = w[r][k];
        const float wf[8] = {bf_lo(x.x), bf_hi(x.x), bf_lo(x.y), bf_hi(x.y), bf_lo(x.z), bf_hi(x.z), bf_lo(x.w), bf_hi(x.w)};
#pragma unroll
        for (int u = 0; u < 8; ++u) acc = __fmaf_rn(wf[u], oc[j + u], acc);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0 && v < v_hi) ((__nv_bfloat16*)d.out)[(size_t)h * DV + v] = __float2bfloat16_rn(acc);
  }
  for (int v0 = v_lo + 2 * ETXB_CONSUMER_WARPS; v0 < v_hi; v0 += ETXB_CONSUMER_WARPS) {   // (more than 32 rows per finishing task: DV > 128)
    const int v = v0 + warp;
    float acc = 0.f;
    if (v < v_hi)
      for (int j = 8 * lane; j < C; j += 256) {
        const uint4 x = __ldg((const uint4*)(wuv + (size_t)v * C + j));
        const float wf[8] = {bf_lo(x.x), bf_hi(x.x), bf_lo(x.y), bf_hi(x.y), bf_lo(x.z), bf_hi(x.z), bf_lo(x.w), bf_hi(x.w)};
#pragma unroll
        for (int u = 0; u < 8; ++u) acc = __fmaf_rn(wf[u], oc[j + u], acc);
      }
    acc = warp_sum(acc);
    if (lane == 0 && v < v_hi) ((__nv_bfloat16*)d.out)[(size_t)h * DV + v] = __float2bfloat16_rn(acc);
  }
  csync();
}

__device__ __noinline__ void tile_mla_attn(const unsigned char* a, int blk, const Smem& sm, const etxb_stepv& S) {
  const etxb_mla_args& d = *(const etxb_mla_args*)a;
  if (blk >= (int)d.nblocks || blk >= d.NH * (d.max_parts + ETXB_MLA_FIN)) return;
  const int part_i = blk / d.NH, h = blk - part_i * d.NH;            // part_i >= max_parts: finishing task part_i - max_parts of the head
  const int C = d.C, DN = d.DN, DR = d.DR, DV = d.DV, QH = DN + DR, ROW = C + DR, PW = C + 8;
  const long long pos = (const void*)d.positions == (const void*)S.positions ? (long long)S.pos : __ldcg((const long long*)d.positions);
  if (pos < 0 || pos >= d.maxlen || pos >= ETXB_MLA_MAXCTX) return;
  const int seq_all = (int)pos + 1;
  const int np = min((seq_all + ETXB_MLA_PART - 1) / ETXB_MLA_PART, d.max_parts);
  if (part_i >= d.max_parts) { mla_finish(d, sm, h, part_i - d.max_parts, np); return; }
  if (part_i >= np) return;
  const int tbase = part_i * ETXB_MLA_PART;                        // first position of this task
  const int seq = min(seq_all - tbase, ETXB_MLA_PART);               // its positions: tbase .. tbase + seq - 1
  const bool owner = pos >= tbase && pos < tbase + ETXB_MLA_PART;    // the new position falls into this partition
  const int lpos = owner ? (int)pos - tbase : -1;
  const uint32_t fl = pair_flag(sm.epoch, d.tag << 16);
  const int tid = tidx(), lane = tid & 31, warp = tid >> 5;
  float* qf = sm.xs;            // [QH <= 256] this head's q row
  float* kvf = qf + 256;        // [ROW <= 640] the raw kv_a row
  float* cn = kvf + 640;        // [C <= 512] the new position's latent (bf16 values)
  float* kpn = cn + 512;        // [DR <= 64] its rotated k_pe (bf16 values)
  float* qpe = kpn + 64;        // [DR] this head's rotated q_pe (bf16 values)
  float* cs = qpe + 64;         // [2 DR] cos | sin of the position
  float* qc = cs + 128;         // [C] q_nope W_UK
  float* part = qc + 512;       // [8][C] partial sums of the eight thread groups (q_c, then o_c)
  float* red = part + 4096;     // [64]
  float* sc = red + 64;         // [128] the partition's scores, then exp(s - m); the merge keeps its weights and sums here
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
  if (h == 0 && owner) {
    __nv_bfloat16* row = (__nv_bfloat16*)d.cache + (size_t)pos * ROW;
    for (int i = tid; i < ROW; i += ETXB_CONSUMERS) row[i] = __float2bfloat16_rn(i < C ? cn[i] : kpn[i - C]);
  }
  // Every loop below keeps eight 16-byte loads per thread in flight before it uses the first: the rows come from L2 (a
  // microsecond away) and a thread that consumed each load before issuing the next spent the phase waiting.
  // ---- q_c[j] = sum_i q_nope[i] W_UK[h][i][j]: thread = (group of DN / 8 rows, 8 columns); groups added in ascending order
  const __nv_bfloat16* wuk = (const __nv_bfloat16*)d.wkvb + (size_t)h * (DN + DV) * C;
  const int nocts = C >> 3, grp = tid >> 6, oct = tid & 63;
  {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const int per = (DN + 7) >> 3, i0 = grp * per, i1 = min(DN, i0 + per);
    if (oct < nocts) {
      for (int ib = i0; ib < i1; ib += 8) {
        uint4 w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = ib + u < i1 ? __ldg((const uint4*)(wuk + (size_t)(ib + u) * C) + oct) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float q = ib + u < i1 ? qf[ib + u] : 0.f;
          acc[0] = __fmaf_rn(q, bf_lo(w[u].x), acc[0]); acc[1] = __fmaf_rn(q, bf_hi(w[u].x), acc[1]);
          acc[2] = __fmaf_rn(q, bf_lo(w[u].y), acc[2]); acc[3] = __fmaf_rn(q, bf_hi(w[u].y), acc[3]);
          acc[4] = __fmaf_rn(q, bf_lo(w[u].z), acc[4]); acc[5] = __fmaf_rn(q, bf_hi(w[u].z), acc[5]);
          acc[6] = __fmaf_rn(q, bf_lo(w[u].w), acc[6]); acc[7] = __fmaf_rn(q, bf_hi(w[u].w), acc[7]);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) part[grp * 512 + 8 * oct + u] = acc[u];
    }
  }
  csync();
  for (int j = tid; j < C; j += ETXB_CONSUMERS) {
    float v = part[j];
#pragma unroll
    for (int g = 1; g < 8; ++g) v = __fadd_rn(v, part[g * 512 + j]);
    qc[j] = v;
  }
  csync();
  // ---- scores: four lanes per position (lane q of the four takes the 16-byte pieces q, q + 4, ..), eight positions per
  //      warp and round; the new position's row comes from shared memory
  const __nv_bfloat16* cache = (const __nv_bfloat16*)d.cache + (size_t)tbase * ROW;    // (positions below are relative to the partition)
  const int npiece = ROW >> 3, quad = lane >> 2, ql = lane & 3;
  for (int t0 = warp * 8; t0 < seq; t0 += ETXB_CONSUMER_WARPS * 8) {
    const int t = t0 + quad;
    float acc = 0.f;
    if (t < seq) {
      const uint4* row = (const uint4*)(cache + (size_t)t * ROW);
      for (int p0 = ql; p0 < npiece; p0 += 32) {
        uint4 w[8];
        if (t == lpos) {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int e = 8 * (p0 + 4 * u);
            if (e < ROW) {
              const float* src = e < C ? cn + e : kpn + (e - C);
              w[u] = make_uint4(pack_bf(src[0], src[1]), pack_bf(src[2], src[3]), pack_bf(src[4], src[5]), pack_bf(src[6], src[7]));
            } else w[u] = make_uint4(0u, 0u, 0u, 0u);
          }
        } else {
#pragma unroll
          for (int u = 0; u < 8; ++u) w[u] = p0 + 4 * u < npiece ? __ldcg(row + p0 + 4 * u) : make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int e = 8 * (p0 + 4 * u);
          if (e < ROW) {
            const float* qv = e < C ? qc + e : qpe + (e - C);
            acc = __fmaf_rn(bf_lo(w[u].x), qv[0], acc); acc = __fmaf_rn(bf_hi(w[u].x), qv[1], acc);
            acc = __fmaf_rn(bf_lo(w[u].y), qv[2], acc); acc = __fmaf_rn(bf_hi(w[u].y), qv[3], acc);
            acc = __fmaf_rn(bf_lo(w[u].z), qv[4], acc); acc = __fmaf_rn(bf_hi(w[u].z), qv[5], acc);
            acc = __fmaf_rn(bf_lo(w[u].w), qv[6], acc); acc = __fmaf_rn(bf_hi(w[u].w), qv[7], acc);
          }
        }
      }
    }
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 1));
    acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, 2));
    if (ql == 0 && t < seq) sc[t] = __fmul_rn(acc, d.scale);
  }
  csync();
  // ---- softmax statistics of the partition: m = max score, e_t = exp(s_t - m) (kept unnormalised), l = sum e_t
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
  csync();
  // ---- o_c[j] = sum_t e_t c[t][j]: thread = (group g of eight: cached positions g, g + 8, .., 8 columns); the new
  //      position's term is added by group 0 from shared memory; groups added in ascending order
  {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (oct < nocts) {
      const int ncached = owner ? lpos : seq;                      // the partition's rows that come from the cache (the new one is its last)
      for (int tb = grp; tb < ncached; tb += 64) {
        uint4 w[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) w[u] = tb + 8 * u < ncached ? __ldcg((const uint4*)(cache + (size_t)(tb + 8 * u) * ROW) + oct) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float pr = tb + 8 * u < ncached ? sc[tb + 8 * u] : 0.f;
          acc[0] = __fmaf_rn(pr, bf_lo(w[u].x), acc[0]); acc[1] = __fmaf_rn(pr, bf_hi(w[u].x), acc[1]);
          acc[2] = __fmaf_rn(pr, bf_lo(w[u].y), acc[2]); acc[3] = __fmaf_rn(pr, bf_hi(w[u].y), acc[3]);
          acc[4] = __fmaf_rn(pr, bf_lo(w[u].z), acc[4]); acc[5] = __fmaf_rn(pr, bf_hi(w[u].z), acc[5]);
          acc[6] = __fmaf_rn(pr, bf_lo(w[u].w), acc[6]); acc[7] = __fmaf_rn(pr, bf_hi(w[u].w), acc[7]);
        }
      }
      if (grp == 0 && owner) {
        const float pr = sc[lpos];
#pragma unroll
        for (int u = 0; u < 8; ++u) acc[u] = __fmaf_rn(pr, cn[8 * oct + u], acc[u]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) part[grp * 512 + 8 * oct + u] = acc[u];
    }
  }
  csync();
  // ---- publish the partition's partial as flagged pairs: weighted latent [C], then max and sum
  uint2* pw = (uint2*)d.tmp + ((size_t)h * d.max_parts + part_i) * PW;
  for (int j = tid; j < C; j += ETXB_CONSUMERS) {
    float v = part[j];
#pragma unroll
    for (int g = 1; g < 8; ++g) v = __fadd_rn(v, part[g * 512 + j]);
    st_pair(pw + j, v, fl);
  }
  if (tid == 0) { st_pair(pw + C, m, fl); st_pair(pw + C + 1, l, fl); }
}

}  // namespace etxb
