// Stand-alone batched bf16 GEMV (nb = 2, 4 or 8 activation columns per weight read): the column-batched form of
// dsl_gemv (etx/ops/gemv.py:40-73, 176-289 `dsl_gemv_rows_nb`), used for the GEMV sweep.  One warp owns a row, every
// lane keeps 4-8 independent 16-byte non-temporal weight loads in flight, fp32 FMA on unpacked bf16 against fp32
// activations staged in shared memory, xor-butterfly across lanes: the summation order is fixed.  It is its own
// (non-persistent) kernel: inside the persistent task loop its register need (nb accumulators x loads in flight)
// spills.
#pragma once
#include "etxb_prims.cuh"

namespace etxb {

// ---------------------------------------------------------------------------------------------- staging
// nb columns of K bf16 values -> floats in shared memory; column b at xs + b * KS.  K % 8 == 0.
__device__ __forceinline__ void stage_x(const void* x, int K, int sx, int nb, int KS, float* xs) {
  const int nv = K >> 3;
  for (int b = 0; b < nb; ++b) {
    const __nv_bfloat16* xb = (const __nv_bfloat16*)x + (size_t)b * sx;
    float* dst = xs + (size_t)b * KS;
    for (int i = (int)threadIdx.x; i < nv; i += blockDim.x) {
      const uint4 v = ld_act16(xb + 8 * i);
      *(float4*)(dst + 8 * i) = make_float4(bf_lo(v.x), bf_hi(v.x), bf_lo(v.y), bf_hi(v.y));
      *(float4*)(dst + 8 * i + 4) = make_float4(bf_lo(v.z), bf_hi(v.z), bf_lo(v.w), bf_hi(v.w));
    }
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
// least 16 * NB floats.  All threads of the CTA call; contains __syncthreads().
template <int NB, typename RowPtr, typename Epi>
__device__ __forceinline__ void gemv_rows(int nrows, int K, RowPtr rowptr, const float* xs, int KS, float* part, Epi epi) {
  const int lane = (int)threadIdx.x & 31, warp = (int)threadIdx.x >> 5;
  const int nvec = K >> 3;
  int ks = 1;                                                    // split-K factor: power of two, >= 32 vectors per segment
  while (nrows * ks * 2 <= 16 && (nvec / (ks * 2)) >= 32) ks *= 2;
  const int segn = (((nvec + ks - 1) / ks) + 31) & ~31;           // vectors per segment, whole lanes-rounds
  const int vpl = segn >> 5;                                      // vectors per lane per segment
  const int units = nrows * ks;
  constexpr int U = NB >= 4 ? 4 : 8;                              // independent 16-byte loads in flight per lane

  if (ks == 1) {
    if (vpl > 4) {
      for (int q = warp; q < nrows; q += 16) {
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
      for (int q0 = warp * 2; q0 < nrows; q0 += 16 * 2) {
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
  for (int u = warp; u < units; u += 16) {
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
  if ((int)threadIdx.x < nrows) {
    float out[NB];
#pragma unroll
    for (int b = 0; b < NB; ++b) {
      float s = 0.f;
      for (int seg = 0; seg < ks; ++seg) s = __fadd_rn(s, part[((int)threadIdx.x * ks + seg) * NB + b]);
      out[b] = s;
    }
    epi((int)threadIdx.x, out);
  }
}


template <int NB>
__global__ void __launch_bounds__(512, 1) etxb_gemv_nb_kernel(const etxb_gemv_args d) {
  extern __shared__ __align__(16) float nb_xs[];
  const int blk = blockIdx.x;
  if (blk >= (int)d.nblocks) return;
  const int r0 = blk * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 >= r1) return;
  const int K = d.K, KS = (K + 7) & ~7, sout = d.sout;
  stage_x(d.x, K, d.sx, NB, KS, nb_xs);
  const __nv_bfloat16* W = (const __nv_bfloat16*)d.W;
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  gemv_rows<NB>(r1 - r0, K, [&](int q) { return W + (size_t)(r0 + q) * K; }, nb_xs, KS, nb_xs + ETXB_NB_XS_FLOATS,
                [&](int q, const float* v) {
#pragma unroll
                  for (int b = 0; b < NB; ++b) out[(size_t)b * sout + r0 + q] = __float2bfloat16_rn(v[b]);
                });
}

}  // namespace etxb
