// Batched decode on the Blackwell tensor cores: tcgen05.mma with the tokens as the M side (A operand, shared memory,
// SWIZZLE_128B K-major), 128 weight rows as the N side (B operand, loaded by TMA tensor copies -- cp.async.bulk.tensor.2d
// with SWIZZLE_128B, one tensor map per weight tensor, box 64 k x 128 rows) and fp32 accumulators in tensor memory, read
// back with tcgen05.ld for the epilogue.
//
// These tiles serve the same grids as the mma.sync tiles of etxb_batch.cuh (column-batched GEMV, expert-grouped gate+up
// and down: etx/ops/gemv.py:40-73, 176-289 and examples/vllm_llm/model.py:194-211 of the reference) and are what the
// batched step uses.  Sizing, measured on B200: one tcgen05.mma (cta_group::1, kind::f16) takes 156 clocks whatever its
// M, N (8 .. 256) or the number of accumulators in flight, so its cost is per instruction: with N = 128 weight rows per
// instruction (4 KB of weights per k16 step) the pipe moves 26 bytes of weights per clock and SM, a little more than
// the 22.5 the HBM delivers, and all of a batch's tokens (up to 32 here) ride along for free -- mma.sync m16n8k16, the
// legacy path, managed about a third of that with 8 tokens per pass.
//
// A job = one tile of 128 weight rows (or two: an expert's gate rows and up rows, accumulated side by side) x all of K x
// up to 32 tokens.  Roles inside the CTA's consumer warps: every thread stages the tokens' vectors into the swizzled
// layout; one thread issues the TMA loads of the weight tile, k-chunk by k-chunk, through a ring of three 16 KB stages;
// one thread issues the MMAs (four k16 steps per 64-wide chunk) and commits each stage back to the loader; when the
// last MMA has completed, four warps read the accumulators (one token per TMEM lane) and run the epilogue.  The weight
// ring of the one-token tiles is not in use during a batched step (their producer warp has nothing to stream), so its
// shared memory holds the tokens here.  Every wait is bounded by the step's deadline; tensor memory is allocated once
// per launch by the kernel and freed on every exit path.
#pragma once
#include <cuda.h>

#include "etxb_gemv.cuh"

namespace etxb {

#define ETXB_TC_ROWS 128               // weight rows per tile (the N of the instruction)
#define ETXB_TC_STAGE 16384            // one k-chunk of a tile: 128 rows x 64 k x 2 bytes
#define ETXB_TC_NSTAGE 3
#define ETXB_TC_XBYTES 143360          // shared memory for the tokens (the idle weight ring), 1024-byte aligned inside it
#define ETXB_TC_MAXTOK 32              // tokens per job (M = 64 up to 8 tokens, 128 above)
#define ETXB_TC_COLS 256               // tensor-memory columns the kernel allocates: two accumulators of 128

struct TcShared {                      // per-CTA state of the tensor-core tiles (static shared memory of the kernel)
  uint64_t full[ETXB_TC_NSTAGE], empty[ETXB_TC_NSTAGE], acc;
  uint32_t n;                          // stages used so far (both role threads count from it)
  uint32_t nacc;                       // completions of `acc` so far
  uint32_t tmem;                       // base address of the allocation
  uint32_t pad;
};

__device__ __forceinline__ void tma_load_2d(void* dst, const void* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// K-major SWIZZLE_128B shared-memory matrix descriptor: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t tc_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
  d |= (uint64_t)1 << 16;                        // leading byte offset: unused for swizzled K-major layouts
  d |= (uint64_t)(1024 >> 4) << 32;              // stride between 8-row groups
  d |= (uint64_t)1 << 46;                        // descriptor version of sm_100
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_alloc(uint32_t* slot) {        // one warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ETXB_TC_COLS) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t base) {       // the same warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(ETXB_TC_COLS) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr) : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// One job: D[tok][j] (+)= sum_k x_tok[k] * W[row[a] + j][k], j < 128, for `nacc` (1 or 2) tiles that share the tokens;
// then epi(tok, j, v0, v1) for every tok < ntok and j < 128 (v1 = 0 with one tile).  xsrc(n): the K bf16 values of token n.
// map: the tensor map of the weight tensor (rows x K, box 64 x 128).  All consumer threads call; ends with a barrier.
template <typename XSrc, typename Epi>
__device__ __forceinline__ void tc_job(const Smem& sm, TcShared& tc, const void* map, int nacc, int row0, int row1, int K, int ntok, int where,
                                       XSrc xsrc, Epi epi) {
  const int tid = tidx(), warp = tid >> 5, lane = tid & 31;
  unsigned char* xs = (unsigned char*)(((uintptr_t)sm.ring + 1023) & ~(uintptr_t)1023);
  unsigned char* ws = (unsigned char*)(((uintptr_t)sm.xs + 1023) & ~(uintptr_t)1023);
  const int M = ntok <= 8 ? 64 : 128, groups = (ntok + 7) >> 3, nchunk = K >> 6;
  const int wc = min(nchunk, (ETXB_TC_XBYTES - (M / 8 - groups) * 1024) / (groups * 1024));      // k-chunks of the tokens that fit at once
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ETXB_TC_ROWS >> 3) << 17) | ((uint32_t)(M >> 4) << 24);   // fp32 D, bf16 A / B, K-major
  const uint32_t n0 = tc.n, a0 = tc.nacc;                          // (the previous job ended with a barrier)
  uint32_t used = 0, windows = 0;
  bool alive = *(volatile int*)sm.stop == 0;
  for (int w0 = 0; w0 < nchunk; w0 += wc, ++windows) {
    const int nc = min(wc, nchunk - w0);
    // the tokens' slice [64 w0, 64 (w0 + nc)) -> swizzled rows: token n is row n % 8 of group n / 8 of its k-chunk
    for (int i = tid; i < ntok * nc * 8; i += ETXB_CONSUMERS) {
      const int n = i / (nc * 8), v = i - n * (nc * 8), c = v >> 3, j = v & 7, r = n & 7;
      const uint4 val = ld_act16((const __nv_bfloat16*)xsrc(n) + (size_t)(w0 * 64 + v * 8));
      *(uint4*)(xs + (size_t)(c * groups + (n >> 3)) * 1024 + r * 128 + ((j ^ r) << 4)) = val;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core's reads
    csync();
    if (warp == 1 && lane == 0 && alive) {                         // loader
      bool ok = true;
      uint32_t n = n0 + used;
      for (int a = 0; a < nacc && ok; ++a)
        for (int c = 0; c < nc && ok; ++c, ++n) {
          const uint32_t st = n % ETXB_TC_NSTAGE, par = (n / ETXB_TC_NSTAGE) & 1;
          ok = mbar_wait(tc.empty + st, par ^ 1, sm, where);
          if (!ok) break;
          mbar_expect_tx(tc.full + st, ETXB_TC_STAGE);
          tma_load_2d(ws + (size_t)st * ETXB_TC_STAGE, map, (w0 + c) * 64, a == 0 ? row0 : row1, tc.full + st);
        }
    } else if (warp == 2 && lane == 0 && alive) {                  // MMA issuer
      bool ok = true;
      uint32_t n = n0 + used;
      for (int a = 0; a < nacc && ok; ++a)
        for (int c = 0; c < nc && ok; ++c, ++n) {
          const uint32_t st = n % ETXB_TC_NSTAGE, par = (n / ETXB_TC_NSTAGE) & 1;
          ok = mbar_wait(tc.full + st, par, sm, where);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t aaddr = smem_u32(xs + (size_t)c * groups * 1024), baddr = smem_u32(ws + (size_t)st * ETXB_TC_STAGE);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            tc_mma(tc.tmem + (uint32_t)a * ETXB_TC_ROWS, tc_desc(aaddr + 32 * k), tc_desc(baddr + 32 * k), idesc, (w0 + c + k) > 0 ? 1u : 0u);
          tc_commit(tc.empty + st);                                // the stage is free once these MMAs have read it
        }
      tc_commit(&tc.acc);                                          // this window's MMAs are complete (tokens may be restaged, accumulators read)
    }
    __syncwarp();                                                  // the role threads' warp-mates wait here, not in a spin beside them
    used += (uint32_t)(nacc * nc);
    if (alive) alive = mbar_wait(&tc.acc, (a0 + windows) & 1, sm, where);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  }
  // epilogue: warps 0, 4, 8, 12 own TMEM lanes 0..31 (one token per lane), a quarter of the 128 columns each
  alive = __all_sync(0xffffffffu, alive);
  if ((warp & 3) == 0 && alive) {
    const int q = warp >> 2;
#pragma unroll 1
    for (int c8 = 0; c8 < 4; ++c8) {
      const int col = 32 * q + 8 * c8;
      float v0[8], v1[8];
      tc_ld8(tc.tmem + (uint32_t)col, v0);
      if (nacc > 1) tc_ld8(tc.tmem + (uint32_t)(ETXB_TC_ROWS + col), v1);
      if (lane < ntok)
#pragma unroll
        for (int j = 0; j < 8; ++j) epi(lane, col + j, v0[j], nacc > 1 ? v1[j] : 0.f);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  csync();
  if (tid == 0) { tc.n = n0 + used; tc.nacc = a0 + windows; }
  csync();
}

// ---------------------------------------------------------------------------------------------- batched dense GEMV
// out[b * sout + r] = bf16(W[r,:] . x[b] (+ bias[r])) for the nb columns b, rows [blk * rpt, ...).  The GEMV block of
// gemv_nb; `ln` = the tensor map of W (rows M, box 64 x 128), put there by the host library when the plan is bound.
__device__ __forceinline__ void tile_gemv_tc(const unsigned char* a, int blk, const Smem& sm, TcShared& tc, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int r0 = blk * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 >= r1) return;
  const __nv_bfloat16* bias = (d.mode & ETXB_MODE_BIAS) ? (const __nv_bfloat16*)d.wts : nullptr;
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  for (int c0 = r0; c0 < r1; c0 += ETXB_TC_ROWS)
    for (int b0 = 0; b0 < d.nb; b0 += ETXB_TC_MAXTOK) {
      const int nt = min(ETXB_TC_MAXTOK, d.nb - b0), nr = min(ETXB_TC_ROWS, r1 - c0);
      tc_job(sm, tc, d.ln, 1, c0, 0, d.K, nt, where,
             [&](int n) { return (const __nv_bfloat16*)d.x + (size_t)(b0 + n) * d.sx; },
             [&](int tok, int j, float v, float) {
               if (j < nr) out[(size_t)(b0 + tok) * d.sout + c0 + j] = __float2bfloat16_rn(bias ? __fadd_rn(v, __bfloat162float(bias[c0 + j])) : v);
             });
    }
}

// ---------------------------------------------------------------------------------------------- expert-grouped gate+up / down
// The blocks of moe_up_g / moe_down_g (task = expert blk / tpe, row chunk blk % tpe; rows = token lists, resid_in = their
// lengths, nb = entries per expert, R = top-k); `ln` = the tensor map of the expert tensor seen as one [E * rows][K] matrix.
__device__ __forceinline__ void tile_moe_up_tc(const unsigned char* a, int blk, const Smem& sm, TcShared& tc, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int e = blk / d.tpe, r0 = (blk - e * d.tpe) * d.rpt, r1 = min(d.M, r0 + d.rpt);
  const int cnt = min(__ldcg((const int32_t*)d.resid_in + e), d.nb);
  if (cnt <= 0 || r0 >= r1) return;
  const int32_t* list = (const int32_t*)d.rows + (size_t)e * d.nb;
  int32_t* ent = (int32_t*)(sm.scr + 96);                          // [32] entries of the pass
  const int erow = (int)((long long)e * d.estride / d.K);          // first row of expert e in the [E * 2M][K] view
  for (int c0 = r0; c0 < r1; c0 += ETXB_TC_ROWS)
    for (int p0 = 0; p0 < cnt; p0 += ETXB_TC_MAXTOK) {
      const int nt = min(ETXB_TC_MAXTOK, cnt - p0), nr = min(ETXB_TC_ROWS, r1 - c0);
      if (tidx() < nt) ent[tidx()] = __ldcg(list + p0 + tidx());
      csync();
      tc_job(sm, tc, d.ln, 2, erow + c0, erow + d.M + c0, d.K, nt, where,
             [&](int n) { return (const __nv_bfloat16*)d.x + (size_t)(ent[n] >> 8) * d.sx; },
             [&](int tok, int j, float g, float u) {
               if (j < nr) {
                 const int en = ent[tok];
                 ((__nv_bfloat16*)d.out)[((size_t)(en >> 8) * d.R + (en & 0xff)) * d.M + c0 + j] = __float2bfloat16_rn(__fmul_rn(bfr(silu_f(bfr(g))), bfr(u)));
               }
             });
    }
}

__device__ __forceinline__ void tile_moe_down_tc(const unsigned char* a, int blk, const Smem& sm, TcShared& tc, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int e = blk / d.tpe, r0 = (blk - e * d.tpe) * d.rpt, r1 = min(d.M, r0 + d.rpt);
  const int cnt = min(__ldcg((const int32_t*)d.resid_in + e), d.nb);
  if (cnt <= 0 || r0 >= r1) return;
  const int32_t* list = (const int32_t*)d.rows + (size_t)e * d.nb;
  int32_t* ent = (int32_t*)(sm.scr + 96);
  float* wt = sm.scr + 128;
  const int erow = (int)((long long)e * d.estride / d.K);
  for (int c0 = r0; c0 < r1; c0 += ETXB_TC_ROWS)
    for (int p0 = 0; p0 < cnt; p0 += ETXB_TC_MAXTOK) {
      const int nt = min(ETXB_TC_MAXTOK, cnt - p0), nr = min(ETXB_TC_ROWS, r1 - c0);
      if (tidx() < nt) {
        const int en = __ldcg(list + p0 + tidx());
        ent[tidx()] = en;
        wt[tidx()] = d.wts ? __ldcg(d.wts + (size_t)(en >> 8) * d.R + (en & 0xff)) : 1.f;
      }
      csync();
      tc_job(sm, tc, d.ln, 1, erow + c0, 0, d.K, nt, where,
             [&](int n) { return (const __nv_bfloat16*)d.x + ((size_t)(ent[n] >> 8) * d.R + (ent[n] & 0xff)) * d.K; },
             [&](int tok, int j, float v, float) {
               if (j < nr) {
                 const int en = ent[tok];
                 const float y = bfr(v);
                 ((__nv_bfloat16*)d.out)[((size_t)(en >> 8) * d.R + (en & 0xff)) * d.M + c0 + j] = __float2bfloat16_rn(d.wts ? bfr(__fmul_rn(y, wt[tok])) : y);
               }
             });
    }
}

}  // namespace etxb
