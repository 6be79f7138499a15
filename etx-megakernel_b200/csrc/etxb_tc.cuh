// Batched decode on the Blackwell tensor cores: tcgen05.mma with the tokens as the M side (A operand, shared memory,
// SWIZZLE_128B K-major), 128 or 256 weight rows as the N side (B operand, loaded by TMA tensor copies --
// cp.async.bulk.tensor.2d with SWIZZLE_128B, one tensor map per weight tensor, boxes of 64 k x 128 rows, one or two per
// instruction) and fp32 accumulators in tensor memory, read back with tcgen05.ld for the epilogue.
//
// These tiles serve the same grids as the mma.sync tiles of etxb_batch.cuh (column-batched GEMV, expert-grouped gate+up
// and down: etx/ops/gemv.py:40-73, 176-289 and examples/vllm_llm/model.py:194-211 of the reference) and are what the
// batched step uses.  Sizing, measured on B200: one tcgen05.mma (cta_group::1, kind::f16) takes 156 clocks whatever its
// M, N (8 .. 256) or the number of accumulators in flight, so its cost is per instruction: with N = 256 weight rows per
// instruction (8 KB of weights per k16 step) the pipe moves 52 bytes of weights per clock and SM, twice what the HBM
// delivers (22.5), and all of a batch's tokens (up to 32 here) ride along for free -- mma.sync m16n8k16, the legacy
// path, managed about a sixth of that with 8 tokens per pass.
//
// A task = a few tiles of up to 256 weight rows (two neighbouring blocks of 128 rows of a matrix, or an expert's 128 gate
// rows and their 128 up rows) x all of K (or a K-slice) x up to 32 tokens.  Roles inside the CTA's consumer warps: every
// thread stages the tokens' vectors into the swizzled layout, once per task; one thread issues the TMA loads of the
// weight tiles, k-chunk by k-chunk, through a ring of 32 KB stages (as many as fit beside the tokens: 2 with 32 tokens
// of 2048 columns, 5 with up to 8); one thread issues the MMAs (four k16 steps per 64-wide chunk) and commits each stage back to the loader; when the last
// MMA of a tile has completed, four warps read its accumulators (one token per TMEM lane) and run the epilogue while
// the next tile's MMAs fill the other accumulator buffer.  The weight ring of the one-token tiles is not in use during
// a batched step (their producer warp has nothing to stream), so its shared memory and the general region form one
// area for tokens and stages here.  Every wait is bounded by the step's deadline; tensor memory is allocated once per
// launch by the kernel and freed on every exit path.
#pragma once
#include <cuda.h>

#include "etxb_gemv.cuh"

namespace etxb {

#define ETXB_TC_ROWS 128               // weight rows per TMA box; an instruction takes one or two boxes (N = 128 or 256)
#define ETXB_TC_BOX 16384              // one box: 128 rows x 64 k x 2 bytes
#define ETXB_TC_STAGE (2 * ETXB_TC_BOX)   // one k-chunk of a tile: up to 256 rows
#define ETXB_TC_MAXSTAGE 6
#define ETXB_TC_TAIL 8192              // end of the area: the routing tables of the expert tiles
#define ETXB_TC_AREA (ETXB_RING_BYTES + ETXB_GEN_BYTES - 1024 - ETXB_TC_TAIL)   // the idle weight ring and the general region, 1024-byte aligned inside
#define ETXB_TC_XBYTES 131072          // at most this much of it holds tokens (32 tokens x 2048 columns); the rest are weight stages
#define ETXB_TC_MAXTOK 32              // tokens per job (M = 64 up to 8 tokens, 128 above)
#define ETXB_TC_COLS 512               // tensor-memory columns the kernel allocates: two accumulator buffers of 256

struct TcShared {                      // per-CTA state of the tensor-core tiles (static shared memory of the kernel)
  uint64_t full[ETXB_TC_MAXSTAGE], empty[ETXB_TC_MAXSTAGE];
  uint64_t acc_full[2], acc_free[2];   // accumulator buffer b: MMAs complete / epilogue done with it
  uint32_t lu[ETXB_TC_MAXSTAGE], mu[ETXB_TC_MAXSTAGE];   // how often the loader / the MMA issuer has used each stage (its barriers' phase)
  uint32_t nfull[2], nfree[2];         // completions of acc_full / acc_free so far
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

// 8 consecutive bf16 results of one token: one 16-byte store when all of them are inside [.., r1), else one by one
__device__ __forceinline__ void tc_store8(__nv_bfloat16* o, int r, int r1, const float (&y)[8]) {
  if (r + 8 <= r1 && (((uintptr_t)(o + r)) & 15) == 0) {
    uint4 pk;
    pk.x = pack_bf(y[0], y[1]); pk.y = pack_bf(y[2], y[3]); pk.z = pack_bf(y[4], y[5]); pk.w = pack_bf(y[6], y[7]);
    *(uint4*)(o + r) = pk;
  } else {
#pragma unroll
    for (int u = 0; u < 8; ++u) if (r + u < r1) o[r + u] = __float2bfloat16_rn(y[u]);
  }
}

// One task: for every tile i < ntiles, D_i[tok][j] = sum_k x_tok[k] * W[boxrow(i, j / 128) + j % 128][k] for j < 128 nbox(i),
// then epi(i, tok, j, v0, v1, two) for every tok < ntok and j = 0, 8, .. 120, with v0[u] = D_i[tok][j + u] and (two: the tile has
// a second box) v1[u] = D_i[tok][128 + j + u].  A tile is one or two TMA boxes of 128 weight rows that one instruction multiplies (N = 128 or 256): two
// neighbouring row blocks of a matrix, or an expert's gate rows and up rows.  The sum runs over the K columns from
// `kofs` on (a K-slice of the matrix: both multiples of 64).  xsrc(n): the bf16 row of token n (column 0);
// map: the tensor map of the weight tensor (rows x all columns, box 64 x 128).  All consumer threads call; ends with a barrier.
//
// The tokens are staged ONCE per task (the tiles of a task share them) whenever all of K fits the token area; the tiles
// then stream back to back through the stage ring, their accumulators alternating between two buffers of tensor
// memory, so that the epilogue of tile i overlaps the MMAs of tile i + 1.  When K does not fit (4096 columns x 32
// tokens) the tokens go in windows of K and a task handles its tiles one by one, accumulating across the windows.
template <typename XSrc, typename NBox, typename BoxRow, typename Epi>
__device__ __forceinline__ void tc_task(const Smem& sm, TcShared& tc, const void* map, int ntiles, int kofs, int K, int ntok, int where,
                                        XSrc xsrc, NBox nbox, BoxRow boxrow, Epi epi) {
  const int tid = tidx(), warp = tid >> 5, lane = tid & 31;
  unsigned char* area = (unsigned char*)(((uintptr_t)sm.ring + 1023) & ~(uintptr_t)1023);
  const int M = ntok <= 8 ? 64 : 128, groups = (ntok + 7) >> 3, nchunk = K >> 6;
  // (an instruction reads M / 8 row groups of its k-chunk: the ones past the tokens' groups are the next chunks' rows or,
  // at the end, the first stage's -- whatever they hold only reaches accumulator rows that nobody reads)
  const int wc = min(nchunk, ETXB_TC_XBYTES / (groups * 1024));    // k-chunks of the tokens that fit at once
  const int nwin = (nchunk + wc - 1) / wc;
  const int xbytes = wc * groups * 1024;
  unsigned char* ws = area + xbytes;
  const int nst = min(ETXB_TC_MAXSTAGE, (ETXB_TC_AREA - xbytes) / ETXB_TC_STAGE);
  const uint32_t idesc0 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(M >> 4) << 24);   // fp32 D, bf16 A / B, K-major; N goes in per tile
  const bool alive0 = *(volatile int*)sm.stop == 0;
  const uint32_t f0[2] = {tc.nfull[0], tc.nfull[1]}, r0[2] = {tc.nfree[0], tc.nfree[1]};     // (the previous task ended with a barrier)
  // one pass = one staging of tokens + the tiles that use it: all tiles x all of K, or (K in windows) one tile x one window
  const int npass = nwin == 1 ? 1 : ntiles * nwin;
  uint32_t tile_seq = 0;                                           // tiles finished before this pass (their buffer = tile_seq & 1)
  for (int pass = 0; pass < npass; ++pass) {
    const int i0 = nwin == 1 ? 0 : pass / nwin, i1 = nwin == 1 ? ntiles : i0 + 1, win = nwin == 1 ? 0 : pass - i0 * nwin;
    const int w0 = win * wc, nc = min(wc, nchunk - w0);
    const bool first_win = win == 0, last_win = win == nwin - 1;
    // the tokens' slice [64 w0, 64 (w0 + nc)) -> swizzled rows: token n is row n % 8 of group n / 8 of its k-chunk
    for (int i = tid; i < ntok * nc * 8; i += ETXB_CONSUMERS) {
      const int n = i / (nc * 8), v = i - n * (nc * 8), c = v >> 3, j = v & 7, r = n & 7;
      const uint4 val = ld_act16((const __nv_bfloat16*)xsrc(n) + (size_t)(kofs + w0 * 64 + v * 8));
      *(uint4*)(area + (size_t)(c * groups + (n >> 3)) * 1024 + r * 128 + ((j ^ r) << 4)) = val;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core's reads
    csync();
    if (sm.tr != nullptr && tid == 0 && pass == 0) sm.tr[4] = globaltimer();
    if (warp == 1 && lane == 0 && alive0) {                        // loader: every tile of the pass, chunk by chunk
      bool ok = true;
      int st = 0;
      for (int i = i0; i < i1 && ok; ++i) {
        const int nb = nbox(i), y0 = boxrow(i, 0), y1 = nb > 1 ? boxrow(i, 1) : 0;
        for (int c = 0; c < nc && ok; ++c) {
          const uint32_t uu = tc.lu[st];
          ok = mbar_wait(tc.empty + st, (uu & 1) ^ 1, sm, where);
          if (!ok) break;
          mbar_expect_tx(tc.full + st, (uint32_t)nb * ETXB_TC_BOX);
          unsigned char* dst = ws + (size_t)st * ETXB_TC_STAGE;
          tma_load_2d(dst, map, kofs + (w0 + c) * 64, y0, tc.full + st);
          if (nb > 1) tma_load_2d(dst + ETXB_TC_BOX, map, kofs + (w0 + c) * 64, y1, tc.full + st);
          tc.lu[st] = uu + 1;
          st = st + 1 == nst ? 0 : st + 1;
        }
      }
    } else if (warp == 2 && lane == 0 && alive0) {                 // MMA issuer
      bool ok = true;
      int st = 0;
      for (int i = i0; i < i1 && ok; ++i) {
        const uint32_t seq = tile_seq + (uint32_t)(i - i0), bsel = seq & 1;
        const uint32_t idesc = idesc0 | ((uint32_t)(nbox(i) * ETXB_TC_ROWS >> 3) << 17);
        if (first_win) {                                           // a fresh accumulator buffer: the epilogue of the tile two back must be done with it
          const uint32_t nth = r0[bsel] + (seq >> 1);              // acc_free[bsel] completions expected before this use
          if (nth > 0) ok = mbar_wait(tc.acc_free + bsel, (nth - 1) & 1, sm, where);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const uint32_t dcol = tc.tmem + bsel * 2 * ETXB_TC_ROWS;
        for (int c = 0; c < nc && ok; ++c) {
          const uint32_t uu = tc.mu[st];
          ok = mbar_wait(tc.full + st, uu & 1, sm, where);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t aaddr = smem_u32(area + (size_t)c * groups * 1024), baddr = smem_u32(ws + (size_t)st * ETXB_TC_STAGE);
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma(dcol, tc_desc(aaddr + 32 * k), tc_desc(baddr + 32 * k), idesc, (w0 + c + k) > 0 ? 1u : 0u);
          tc_commit(tc.empty + st);                                // the stage is free once these MMAs have read it
          tc.mu[st] = uu + 1;
          st = st + 1 == nst ? 0 : st + 1;
        }
        if (ok) tc_commit(tc.acc_full + bsel);                     // the tile's MMAs (of this window) are complete
      }
      if (sm.tr != nullptr && pass == npass - 1) sm.tr[5] = globaltimer();
    }
    __syncwarp();                                                  // the role threads' warp-mates wait here, not in a spin beside them
    // epilogue: warps 0, 4, 8, 12 own TMEM lanes 0..31 (one token per lane), a quarter of each box's 128 columns each.  Only
    // they wait for the accumulators: the issuer runs at most one tile ahead of the slowest of them (it needs their four
    // arrivals to reuse a buffer), so none of them can miss a phase; the other warps go on to the barrier below.
    if ((warp & 3) == 0) {
      for (int i = i0; i < i1; ++i) {
        const uint32_t seq = tile_seq + (uint32_t)(i - i0), bsel = seq & 1;
        // completions of acc_full[bsel] before this one: one per tile on that buffer (per window, when K goes in windows)
        const uint32_t done = f0[bsel] + (nwin == 1 ? (seq >> 1) : (seq >> 1) * (uint32_t)nwin + (uint32_t)win);
        bool alive = alive0;
        if (alive) alive = mbar_wait(tc.acc_full + bsel, done & 1, sm, where);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        alive = __all_sync(0xffffffffu, alive);
        if (!last_win) continue;
        if (alive) {
          const int q = warp >> 2;
          const bool two = nbox(i) > 1;
#pragma unroll 1
          for (int c8 = 0; c8 < 4; ++c8) {
            const int col = 32 * q + 8 * c8;
            float v0[8], v1[8];
            tc_ld8(tc.tmem + bsel * 2 * ETXB_TC_ROWS + (uint32_t)col, v0);
            if (two) tc_ld8(tc.tmem + bsel * 2 * ETXB_TC_ROWS + (uint32_t)(ETXB_TC_ROWS + col), v1);
            if (lane < ntok) epi(i, lane, col, v0, v1, two);
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(tc.acc_free + bsel);            // four arrivals per tile: the buffer may be overwritten
      }
    }
    if (last_win) tile_seq += (uint32_t)(i1 - i0);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    csync();                                                       // the tokens may be restaged
  }
  if (tid == 0) {
    const uint32_t nt = (uint32_t)ntiles;
    for (int b = 0; b < 2; ++b) {
      const uint32_t tiles_b = (nt + (b == 0 ? 1u : 0u)) >> 1;     // tiles that used buffer b
      tc.nfull[b] = f0[b] + tiles_b * (uint32_t)nwin;
      tc.nfree[b] = r0[b] + tiles_b;
    }
  }
  csync();
}

// ---------------------------------------------------------------------------------------------- batched dense GEMV
// out[b * sout + r] = bf16(W[r,:] . x[b] (+ bias[r])) for the nb columns b.  The GEMV block of gemv_nb; `ln` = the tensor
// map of W (rows M, box 64 x 128), put there by the host library when the plan is bound.
//
// tpe = the K-split S of the grid (1: none).  Task blk covers rows [(blk / S) * rpt, ...) and the K-slice blk % S.  A
// matrix of a few thousand rows has too few 128-row tiles for 148 workers (qkv: 40, o_proj: 16, router: 1) and an
// instruction cannot take fewer rows without paying the same time, so the narrow matrices are cut along K instead: every
// slice task stores its fp32 partial sums to `rows` ([S][M][nb] floats) and counts itself in `resid_in` (one int32 per row
// block); the S-th arrival adds the partials in slice order, adds the bias and writes the bf16 result -- the same sum
// whoever comes last.
__device__ __forceinline__ void tile_gemv_tc(const unsigned char* a, int blk, const Smem& sm, TcShared& tc, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const int S = max(1, d.tpe), rb = blk / S, ksl = blk - rb * S, Ks = d.K / S;
  const int r0 = rb * d.rpt, r1 = min(d.M, r0 + d.rpt);
  if (r0 >= r1) return;
  const __nv_bfloat16* bias = (d.mode & ETXB_MODE_BIAS) ? (const __nv_bfloat16*)d.wts : nullptr;
  __nv_bfloat16* out = (__nv_bfloat16*)d.out;
  float* part = S > 1 ? (float*)d.rows + (size_t)ksl * d.nb * d.M : nullptr;   // this slice's [M][nb] partial sums
  const int ntiles = (r1 - r0 + 2 * ETXB_TC_ROWS - 1) / (2 * ETXB_TC_ROWS);
  for (int b0 = 0; b0 < d.nb; b0 += ETXB_TC_MAXTOK) {
    const int nt = min(ETXB_TC_MAXTOK, d.nb - b0);
    tc_task(sm, tc, d.ln, ntiles, ksl * Ks, Ks, nt, where,
            [&](int n) { return (const __nv_bfloat16*)d.x + (size_t)(b0 + n) * d.sx; },
            [&](int i) { return r1 - r0 - i * 2 * ETXB_TC_ROWS > ETXB_TC_ROWS ? 2 : 1; },
            [&](int i, int b) { return r0 + (2 * i + b) * ETXB_TC_ROWS; },
            [&](int i, int tok, int j, const float (&v0)[8], const float (&v1)[8], bool two) {
              const int r = r0 + 2 * i * ETXB_TC_ROWS + j;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                if (h == 1 && !two) break;
                const int rr = r + h * ETXB_TC_ROWS;
                const float (&v)[8] = h ? v1 : v0;
                if (part != nullptr) {                              // [slice][row][column]: the 32 lanes of a store are 32 consecutive floats
#pragma unroll
                  for (int u = 0; u < 8; ++u) if (rr + u < r1) __stcg(part + (size_t)(rr + u) * d.nb + b0 + tok, v[u]);
                } else {
                  float y[8];
#pragma unroll
                  for (int u = 0; u < 8; ++u) y[u] = (bias && rr + u < r1) ? __fadd_rn(v[u], __bfloat162float(bias[rr + u])) : v[u];
                  tc_store8(out + (size_t)(b0 + tok) * d.sout, rr, r1, y);
                }
              }
            });
  }
  if (S == 1) return;
  // (tc_task ended with a barrier: every partial of this task is stored)
  int* last = (int*)(sm.scr + 90);
  if (tidx() == 0) {
    __threadfence();
    const int old = atomicAdd((int*)d.resid_in + rb, 1);
    *last = ((old + 1) % S) == 0;
    __threadfence();
  }
  csync();
  if (*last == 0) return;
  const float* p0 = (const float*)d.rows;
  const size_t sstride = (size_t)d.nb * d.M;
  // Sums with the column index fastest (the partials are [row][column]: coalesced reads), eight loads of four columns in
  // flight per thread (the partials come from L2, a microsecond away); every output is the sum of its slices in slice order.
  // The sums go through shared memory ([row][nb + 1] floats in the area the tile's tokens and stages have left) so that
  // the bf16 results leave with the row index fastest: rows of `out` are contiguous, columns are sout apart.
  const int nr = r1 - r0, nout = d.nb * nr, ld = d.nb + 1;
  float* tile = (float*)(((uintptr_t)sm.ring + 1023) & ~(uintptr_t)1023);
  if ((d.nb & 3) == 0 && (((uintptr_t)p0) & 15) == 0) {
    // four columns per 16-byte load; two such groups x four slices in flight per thread and round
    const int gpr = d.nb >> 2, ngrp = nr * gpr;
    for (int g0 = tidx(); g0 < ngrp; g0 += 2 * ETXB_CONSUMERS) {
      float4 acc[2];
      acc[0] = acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int q0 = 0; q0 < S; q0 += 4) {
        float4 t[2][4];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          const int gi = min(g0 + w * ETXB_CONSUMERS, ngrp - 1);
          const float4* src = (const float4*)(p0 + (size_t)(r0 + gi / gpr) * d.nb) + (gi - (gi / gpr) * gpr);
#pragma unroll
          for (int u = 0; u < 4; ++u) t[w][u] = q0 + u < S ? __ldcg((const float4*)((const float*)src + (size_t)(q0 + u) * sstride)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int w = 0; w < 2; ++w)
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (q0 + u < S) {
              acc[w].x = __fadd_rn(acc[w].x, t[w][u].x); acc[w].y = __fadd_rn(acc[w].y, t[w][u].y);
              acc[w].z = __fadd_rn(acc[w].z, t[w][u].z); acc[w].w = __fadd_rn(acc[w].w, t[w][u].w);
            }
      }
#pragma unroll
      for (int w = 0; w < 2; ++w) {
        const int gi = g0 + w * ETXB_CONSUMERS;
        if (gi >= ngrp) break;
        float* dst = tile + (gi / gpr) * ld + 4 * (gi - (gi / gpr) * gpr);
        dst[0] = acc[w].x; dst[1] = acc[w].y; dst[2] = acc[w].z; dst[3] = acc[w].w;
      }
    }
  } else {
    for (int i = tidx(); i < nout; i += ETXB_CONSUMERS) {
      const int rl = i / d.nb, tok = i - rl * d.nb;
      float v = 0.f;
      for (int q = 0; q < S; ++q) v = __fadd_rn(v, __ldcg(p0 + (size_t)q * sstride + (size_t)(r0 + rl) * d.nb + tok));
      tile[rl * ld + tok] = v;
    }
  }
  csync();
  for (int i = tidx(); i < nout; i += ETXB_CONSUMERS) {
    const int tok = i / nr, rl = i - tok * nr, r = r0 + rl;
    const float v = tile[rl * ld + tok];
    out[(size_t)tok * d.sout + r] = __float2bfloat16_rn(bias ? __fadd_rn(v, __bfloat162float(bias[r])) : v);
  }
  csync();
}

// ---------------------------------------------------------------------------------------------- expert-grouped gate+up / down
// The expert phases of a batched step, scheduled by SHARE: the grid has one task per worker, and task blk of S takes
// tiles [blk * total / S, (blk + 1) * total / S) of the step's active experts (total = active experts x tiles per expert,
// experts in ascending id, an expert's tiles in row order) -- every worker streams the same number of weight rows (+-1
// tile) however the routing falls, where a grid of (expert, row chunk) tasks leaves the workers of unselected experts idle
// and gives others three chunks.  Every task derives the routing tables itself from the step's top-k ids (nb x R int32,
// one L2 read): per-expert counts, the active list, and per expert the (column << 8 | slot) pairs that selected it in
// ascending (column, slot) order.
//
// The GEMV block, read this way: W / estride / M / K / E as in the one-token MoE tiles (gate+up: M gate rows then M up
// rows per expert; down: M rows), ids = the routing ids [nb][R], nb columns, R = top-k, nblocks = S;
// gate+up: x[b * sx ..] the columns' normed vectors, out = act [nb][R][M], resid_out = optional int32 counter that
// share 0 increases by the number of active experts; down: x = act [nb][R][K], wts [nb][R] routing weights, out = y [nb][R][M].
// `ln` = the tensor map of the expert tensor seen as one [E * rows][K] matrix.
struct TcRoute {
  int32_t* sids;     // [nb * R] expert ids of the step
  int32_t* scnt;     // [E] entries per expert
  int32_t* ent;      // [<= nb] entries of the current expert
  float* wt;         // [<= nb] their routing weights (down)
  uint16_t* alist;   // [nact] active experts, ascending
  int32_t* nact;
};
__device__ __forceinline__ TcRoute tc_route_tables(const Smem& sm) {
  unsigned char* tail = (unsigned char*)(((uintptr_t)sm.ring + 1023) & ~(uintptr_t)1023) + ETXB_TC_AREA;
  TcRoute r;
  r.sids = (int32_t*)tail; r.scnt = r.sids + 1024; r.ent = r.scnt + 256; r.wt = (float*)(r.ent + 64); r.alist = (uint16_t*)(r.wt + 64);
  r.nact = (int32_t*)(r.alist + 256);
  return r;
}
// counts and the active list (all consumer threads; ends with a barrier)
__device__ __forceinline__ void tc_route_build(const etxb_gemv_args& d, const TcRoute& rt) {
  const int tid = tidx(), n = d.nb * d.R;
  for (int i = tid; i < n; i += ETXB_CONSUMERS) { const int e = __ldcg(d.ids + i); rt.sids[i] = (unsigned)e < (unsigned)d.E ? e : 0; }
  for (int e = tid; e < d.E; e += ETXB_CONSUMERS) rt.scnt[e] = 0;
  csync();
  for (int i = tid; i < n; i += ETXB_CONSUMERS) atomicAdd(rt.scnt + rt.sids[i], 1);
  csync();
  if (tid < 32) {
    int na = 0;
    for (int e0 = 0; e0 < d.E; e0 += 32) {
      const bool on = e0 + tid < d.E && rt.scnt[e0 + tid] > 0;
      const uint32_t m = __ballot_sync(0xffffffffu, on);
      if (on) rt.alist[na + __popc(m & ((1u << tid) - 1u))] = (uint16_t)(e0 + tid);
      na += __popc(m);
    }
    if (tid == 0) *rt.nact = na;
  }
  csync();
}
// the entries of expert e, in (column, slot) order (warp 0; the caller syncs)
__device__ __forceinline__ void tc_route_entries(const etxb_gemv_args& d, const TcRoute& rt, int e, const float* wts) {
  const int tid = tidx(), n = d.nb * d.R;
  if (tid >= 32) return;
  int cnt = 0;
  for (int i0 = 0; i0 < n; i0 += 32) {
    const int i = i0 + tid;
    const bool hit = i < n && rt.sids[i] == e;
    const uint32_t m = __ballot_sync(0xffffffffu, hit);
    const int at = cnt + __popc(m & ((1u << tid) - 1u));
    if (hit && at < 64) {
      rt.ent[at] = ((i / d.R) << 8) | (i % d.R);
      if (wts != nullptr) rt.wt[at] = __ldcg(wts + i);
    }
    cnt += __popc(m);
  }
}

template <bool UP>
__device__ __forceinline__ void tile_moe_tc(const unsigned char* a, int blk, const Smem& sm, TcShared& tc, int where) {
  const etxb_gemv_args& d = *(const etxb_gemv_args*)a;
  if (blk >= (int)d.nblocks) return;
  const TcRoute rt = tc_route_tables(sm);
  tc_route_build(d, rt);
  const int nact = *rt.nact;
  constexpr int TROWS = UP ? ETXB_TC_ROWS : 2 * ETXB_TC_ROWS;       // rows of M one tile covers (gate+up: 128 gate rows and their 128 up rows)
  const int T = (d.M + TROWS - 1) / TROWS;
  const long long total = (long long)nact * T;
  int t = (int)(total * blk / (long long)d.nblocks);
  const int hi = (int)(total * (blk + 1) / (long long)d.nblocks);
  if (UP && blk == 0 && tidx() == 0 && d.resid_out != nullptr) atomicAdd((int32_t*)d.resid_out, nact);
  while (t < hi) {
    const int ai = t / T, t0 = t - ai * T, t1 = min(T, t0 + (hi - t));
    const int e = rt.alist[ai];
    const int cnt = min(min(rt.scnt[e], d.nb), 64);
    tc_route_entries(d, rt, e, UP ? nullptr : d.wts);
    csync();
    const int erow = (int)((long long)e * d.estride / d.K);         // first row of expert e in the [E * rows][K] view
    const int r0 = t0 * TROWS, r1 = min(d.M, t1 * TROWS);
    for (int p0 = 0; p0 < cnt; p0 += ETXB_TC_MAXTOK) {
      const int nt = min(ETXB_TC_MAXTOK, cnt - p0);
      const int32_t* ent = rt.ent + p0;
      if constexpr (UP) {
        tc_task(sm, tc, d.ln, t1 - t0, 0, d.K, nt, where,
                [&](int n) { return (const __nv_bfloat16*)d.x + (size_t)(ent[n] >> 8) * d.sx; },
                [&](int) { return 2; },                                                          // 128 gate rows and their 128 up rows: one instruction
                [&](int i, int b) { return erow + (b ? d.M : 0) + r0 + i * ETXB_TC_ROWS; },        // up rows follow the M gate rows
                [&](int i, int tok, int j, const float (&g)[8], const float (&up)[8], bool) {
                  const int r = r0 + i * ETXB_TC_ROWS + j, en = ent[tok];
                  float y[8];
#pragma unroll
                  for (int u = 0; u < 8; ++u) y[u] = __fmul_rn(bfr(silu_f(bfr(g[u]))), bfr(up[u]));
                  tc_store8((__nv_bfloat16*)d.out + ((size_t)(en >> 8) * d.R + (en & 0xff)) * d.M, r, r1, y);
                });
      } else {
        const float* wt = rt.wt + p0;
        tc_task(sm, tc, d.ln, t1 - t0, 0, d.K, nt, where,
                [&](int n) { return (const __nv_bfloat16*)d.x + ((size_t)(ent[n] >> 8) * d.R + (ent[n] & 0xff)) * d.K; },
                [&](int i) { return r1 - r0 - i * 2 * ETXB_TC_ROWS > ETXB_TC_ROWS ? 2 : 1; },
                [&](int i, int b) { return erow + r0 + (2 * i + b) * ETXB_TC_ROWS; },
                [&](int i, int tok, int j, const float (&v0)[8], const float (&v1)[8], bool two) {
                  const int r = r0 + 2 * i * ETXB_TC_ROWS + j, en = ent[tok];
                  __nv_bfloat16* o = (__nv_bfloat16*)d.out + ((size_t)(en >> 8) * d.R + (en & 0xff)) * d.M;
                  float y[8];
#pragma unroll
                  for (int u = 0; u < 8; ++u) { const float q = bfr(v0[u]); y[u] = d.wts ? bfr(__fmul_rn(q, wt[tok])) : q; }
                  tc_store8(o, r, r1, y);
                  if (two) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) { const float q = bfr(v1[u]); y[u] = d.wts ? bfr(__fmul_rn(q, wt[tok])) : q; }
                    tc_store8(o, r + ETXB_TC_ROWS, r1, y);
                  }
                });
      }
    }
    t += t1 - t0;
  }
}
__device__ __forceinline__ void tile_moe_up_tc(const unsigned char* a, int blk, const Smem& sm, TcShared& tc, int where) { tile_moe_tc<true>(a, blk, sm, tc, where); }
__device__ __forceinline__ void tile_moe_down_tc(const unsigned char* a, int blk, const Smem& sm, TcShared& tc, int where) { tile_moe_tc<false>(a, blk, sm, tc, where); }

}  // namespace etxb
