// Stand-alone batched bf16 GEMV (nb = 2 .. 8 activation columns per weight read): the column-batched form of dsl_gemv
// (etx/ops/gemv.py:40-73, 176-289 `dsl_gemv_rows_nb`), used for the GEMV sweep.  With several tokens per weight row the
// product is a (rows x K) . (K x 8) contraction, so it runs on the tensor cores: mma.sync m16n8k16, 16 weight rows as
// the A operand straight from global memory (each thread loads 16 bytes of rows g and g + 8 -- no shared-memory
// staging of weights), the tokens' activations as the B operand from shared memory, fp32 accumulators.  The k order
// inside a 32-group is permuted identically on both operands (a thread's 16 bytes are 8 consecutive k), which a dot
// product does not notice.  An fp32 FMA loop over unpacked bf16 was bound by the unpacking (14 % of the HBM roofline
// at 8 tokens); here the stream is bound by memory.
//
// A task (CTA) covers rows [blk * rpt, ...): blocks of 16 rows x ks slices of K, one unit per warp trip; the slices'
// 16 x 8 partial tiles go through shared memory and are added in slice order (fixed order: reproducible).
// It is its own (non-persistent) kernel: the persistent kernel's tiles are built for one token.
#pragma once
#include "etxb_prims.cuh"

namespace etxb {

#define ETXB_NB_THREADS 512
#define ETXB_NB_PAD 64                 // bytes between the tokens' activation rows in shared memory (bank spread)
#define ETXB_NB_PART_FLOATS 8192       // partial tiles: units * 128 floats

__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(ETXB_NB_THREADS, 1) etxb_gemv_nb_kernel(const etxb_gemv_args d) {
  extern __shared__ __align__(128) unsigned char nb_smem[];
  const int blk = blockIdx.x;
  if (blk >= (int)d.nblocks) return;
  const int r0 = blk * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 >= r1) return;
  const int K = d.K, nb = d.nb, nrows = r1 - r0;
  const int tid = (int)threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
  const int xstride = K * 2 + ETXB_NB_PAD;                         // bytes; token n < nb at nb_smem + n * xstride
  float* part = (float*)(nb_smem + (size_t)nb * xstride);
  // ---- the tokens' activations -> shared memory (bf16 as they are); the columns of absent tokens multiply zeros
  for (int i = tid; i < nb * (K >> 3); i += ETXB_NB_THREADS) {
    const int n = i / (K >> 3), v = i - n * (K >> 3);
    *(uint4*)(nb_smem + (size_t)n * xstride + 16 * v) = ld_act16((const __nv_bfloat16*)d.x + (size_t)n * d.sx + 8 * v);
  }
  __syncthreads();
  // ---- units: (block of 16 rows, slice of K); ks = slices per block, a power of two
  const int nblk = (nrows + 15) >> 4, steps = (K + 31) >> 5;       // k32 steps per row
  int ks = 1;
  while (nblk * ks < 2 * 16 && steps / (ks * 2) >= 8 && (nblk * ks * 2) * 128 <= ETXB_NB_PART_FLOATS) ks *= 2;
  const unsigned char* W = (const unsigned char*)d.W;
  const unsigned char* xs = nb_smem + (size_t)g * xstride + 16 * t;
  for (int u = warp; u < nblk * ks; u += 16) {
    const int b = u / ks, s = u - b * ks;
    const int ra = r0 + min(16 * b + g, nrows - 1), rb = r0 + min(16 * b + g + 8, nrows - 1);   // rows past the task repeat its last row
    const unsigned char* wa = W + (size_t)ra * K * 2 + 16 * t;
    const unsigned char* wb = W + (size_t)rb * K * 2 + 16 * t;
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
        const uint4 x = in && g < nb ? *(const uint4*)(xs + 64 * (k + j)) : make_uint4(0u, 0u, 0u, 0u);
        mma_bf16_16x8x16(da, va[j].x, vb[j].x, va[j].y, vb[j].y, x.x, x.y);
        mma_bf16_16x8x16(db, va[j].z, vb[j].z, va[j].w, vb[j].w, x.z, x.w);
      }
    }
    // D[row g][token 2t, 2t + 1] in (0, 1), D[row g + 8][...] in (2, 3)
    float* p = part + (size_t)u * 128;
    p[g * 8 + 2 * t] = __fadd_rn(da[0], db[0]); p[g * 8 + 2 * t + 1] = __fadd_rn(da[1], db[1]);
    p[(g + 8) * 8 + 2 * t] = __fadd_rn(da[2], db[2]); p[(g + 8) * 8 + 2 * t + 1] = __fadd_rn(da[3], db[3]);
  }
  __syncthreads();
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  for (int i = tid; i < nrows * nb; i += ETXB_NB_THREADS) {
    const int n = i / nrows, q = i - n * nrows;                    // consecutive threads -> consecutive rows of one token
    const float* p = part + (size_t)((q >> 4) * ks) * 128 + (q & 15) * 8 + n;
    float v = p[0];
    for (int s = 1; s < ks; ++s) v = __fadd_rn(v, p[(size_t)s * 128]);
    out[(size_t)n * d.sout + r0 + q] = __float2bfloat16_rn(v);
  }
}

}  // namespace etxb
