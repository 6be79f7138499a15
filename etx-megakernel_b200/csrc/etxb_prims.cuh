// Device primitives of the B200 megakernel: event counters with acquire/release at GPU scope, bounded waits,
// bf16 helpers with explicit round-to-nearest-even, warp/block reductions in a fixed (deterministic) order, and the
// sum-of-squares in numpy's pairwise order so that RMSNorm agrees bit for bit with the CPU numerical path.
//
// Replaces etx/runtime/include/etx/primitives.h:18-30 (wait/arrive), primitives_nvptx.h:5-22 (ld.acquire /
// st.relaxed helpers) and tile_util.h:14-26, 123-155 (wave/block reductions) of the reference.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>
#include "etxb_abi.h"

namespace etxb {

// Thread index through a volatile asm.  The tiles run inside the persistent task loop; with the plain special register
// every lane-dependent address of every unrolled tile is loop-invariant there, gets hoisted out of the task loop and
// the hoisted values alone overflow the register file (8 KB of spills).  A volatile read pins them inside the task.
__device__ __forceinline__ int tidx() {
  int t;
  asm volatile("mov.u32 %0, %%tid.x;" : "=r"(t));
  return t;
}

// Barrier of the consumer warps only (named barrier 1): the producer warp never joins it.
__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(ETXB_CONSUMERS) : "memory"); }

// ---------------------------------------------------------------------------------------------- mbarrier + bulk async copy
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// 16-byte asynchronous copy global -> shared (bypasses L1); !live: the 16 bytes are zero-filled and nothing is read
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool live) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(live ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait0() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
// global -> shared bulk copy (TMA engine, untiled): 16-byte aligned addresses, size a multiple of 16; completes on `bar`
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// The same with an L2 eviction policy.  Weights are read once per step: streamed "evict first", the gigabytes that pass
// through L2 every step leave the small things everybody re-reads (activations, KV cache, tables, argument blocks) in it.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy) : "memory");
}

// ---------------------------------------------------------------------------------------------- memory ordering
__device__ __forceinline__ int32_t ld_acquire(const int32_t* p) {
  int32_t v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int32_t ld_relaxed(const int32_t* p) {
  int32_t v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add(int32_t* p, int32_t v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long globaltimer() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Wait until counter >= target (wrap-safe).  Bounded: gives up when the host sets the abort bit or when the
// deadline passes, records where, and returns false; the kernel then drains and returns (no trap, no endless spin).
__device__ __forceinline__ bool wait_event(const int32_t* events, int32_t* ctrl, int word, int32_t target, int task_id,
                                           unsigned long long deadline) {
  const int32_t* e = events + (size_t)word * ETXB_EV_STRIDE;
  uint32_t n = 0;
  for (;;) {
    const int32_t v = ld_acquire(e);
    if ((int32_t)(v - target) >= 0) return true;
    if ((++n & 63u) == 0) {
      const int32_t c = ld_relaxed(ctrl);
      if (c != 0) return false;                                   // someone else gave up, or the host aborted
      if ((n & 1023u) == 0 && globaltimer() > deadline) {
        if (atomicOr(ctrl, ETXB_CTRL_TIMEOUT) == 0) {           // first to give up records the place
          ctrl[1] = task_id; ctrl[2] = word; ctrl[3] = v; ctrl[4] = target;
        }
        return false;
      }
      __nanosleep(64);
    }
  }
}

__device__ __forceinline__ bool wait_event(const etxb_params& p, int word, int32_t target, int task_id, unsigned long long deadline) {
  return wait_event(p.events, p.ctrl, word, target, task_id, deadline);
}

// ---------------------------------------------------------------------------------------------- bf16
__device__ __forceinline__ float bfr(float x) {                    // RNE to bf16, kept as float (ref_numpy.py:26-32)
  return __bfloat162float(__float2bfloat16_rn(x));
}
__device__ __forceinline__ float bf_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf(float lo, float hi) {  // both already bf16-exact or to be rounded RNE
  const uint32_t a = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(lo));
  const uint32_t b = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(hi));
  return a | (b << 16);
}
__device__ __forceinline__ float ld_bf(const void* base, size_t i) {           // activation written by another CTA
  const unsigned short u = __ldcg((const unsigned short*)base + i);
  return __uint_as_float((uint32_t)u << 16);
}
__device__ __forceinline__ void st_bf(void* base, size_t i, float v) {
  ((__nv_bfloat16*)base)[i] = __float2bfloat16_rn(v);
}
// 16-byte streaming load of weights: read-only path, do not keep in L1
__device__ __forceinline__ uint4 ld_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::128B.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// 16-byte load of activations another CTA produced this step: L2 only (L1 is not coherent across SMs)
__device__ __forceinline__ uint4 ld_act16(const void* p) { return __ldcg((const uint4*)p); }

// Flagged words of a sharded model's exchanged rows: a bf16 value in the low half, a 16-bit flag derived from the step
// in the high half.  A 4-byte store is atomic on every path (NVLink included), so value and flag arrive together and the
// reader needs no fence and no counter: it re-reads until the flag is this step's.  The flag is never 0 (a zeroed buffer
// is never valid) and differs from the previous step's (every buffer is rewritten once per step).
__device__ __forceinline__ uint32_t row_flag(uint32_t epoch) { return ((epoch & 0x7fffu) | 0x8000u) << 16; }
// (a strong store at system scope: the readers poll with volatile loads, possibly from another GPU)
__device__ __forceinline__ void st_flagged(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile16(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// ---------------------------------------------------------------------------------------------- reductions
__device__ __forceinline__ float warp_sum(float v) {               // xor butterfly 16..1: same value in every lane
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// block sum in a fixed order: lanes by butterfly, warps left to right.  red: >= 32 floats.  All threads call.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  csync();
  if ((tidx() & 31) == 0) red[tidx() >> 5] = v;
  csync();
  float s = 0.f;
#pragma unroll
  for (int w = 0; w < ETXB_NWARPS; ++w) s += red[w];
  return s;
}

// Sum of squares of x[0..n) in the order numpy's float32 pairwise summation uses (np.mean(x ** 2) in the CPU path,
// ref_numpy.py:71-73): blocks of 128 with 8 strided accumulators each, combined ((r0+r1)+(r2+r3))+((r4+r5)+(r6+r7)),
// blocks combined by a balanced binary tree.  Exact for n = 128 * 2^j, 128 <= n <= 16 * blockDim; other n fall back
// to block_sum (same value up to fp32 rounding).  x in shared memory; red >= 32 floats; all threads call.
__device__ __forceinline__ float sumsq_numpy_order(const float* x, int n, float* red) {
  const bool pow2 = n >= 128 && (n & (n - 1)) == 0 && n <= 16 * ETXB_CONSUMERS;
  if (!pow2) {
    float s = 0.f;
    for (int i = tidx(); i < n; i += ETXB_CONSUMERS) s = __fmaf_rn(x[i], x[i], s);
    return block_sum(s, red);
  }
  const int nacc = n >> 4;                                         // 8 accumulators per 128-element block
  const int t = tidx();
  float r = 0.f;
  if (t < nacc) {
    const float* b = x + (t >> 3) * 128 + (t & 7);
    r = __fmul_rn(b[0], b[0]);
#pragma unroll
    for (int i = 1; i < 16; ++i) r = __fadd_rn(r, __fmul_rn(b[8 * i], b[8 * i]));
  }
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, o));   // accumulators, then 4 blocks
  csync();
  if ((t & 31) == 0) red[t >> 5] = r;
  csync();
  const int nw = (nacc + 31) >> 5;                                 // power of two (or 1)
  float v = (t & 31) < nw ? red[t & 31] : 0.f;
  for (int o = 1; o < nw; o <<= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
  return __shfl_sync(0xffffffffu, v, 0);
}

// The same for one head of 128 values held in shared memory, computed by one warp (all 32 lanes call).
__device__ __forceinline__ float sumsq128_numpy_order_warp(const float* x) {
  const int lane = tidx() & 31;
  float r = 0.f;
  if (lane < 8) {
    r = __fmul_rn(x[lane], x[lane]);
#pragma unroll
    for (int i = 1; i < 16; ++i) r = __fadd_rn(r, __fmul_rn(x[8 * i + lane], x[8 * i + lane]));
  }
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) r = __fadd_rn(r, __shfl_xor_sync(0xffffffffu, r, o));
  return __shfl_sync(0xffffffffu, r, 0);
}

// numpy's sum of n <= 16 float32 values (n < 8: left to right; else 8 accumulators + tree + tail), one thread.
__device__ __forceinline__ float sum_small_numpy_order(const float* a, int n) {
  if (n < 8) {
    float r = 0.f;
    for (int i = 0; i < n; ++i) r = __fadd_rn(r, a[i]);
    return r;
  }
  float r[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) r[j] = a[j];
  const int full = n - (n & 7);
  for (int i = 8; i < full; i += 8)
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = __fadd_rn(r[j], a[i + j]);
  float res = __fadd_rn(__fadd_rn(__fadd_rn(r[0], r[1]), __fadd_rn(r[2], r[3])),
                        __fadd_rn(__fadd_rn(r[4], r[5]), __fadd_rn(r[6], r[7])));
  for (int i = full; i < n; ++i) res = __fadd_rn(res, a[i]);
  return res;
}

__device__ __forceinline__ float silu_f(float g) { return __fdiv_rn(g, 1.0f + expf(-g)); }   // ref_numpy.py:91-92

}  // namespace etxb
