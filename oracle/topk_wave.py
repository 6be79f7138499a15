"""CPU model of the router's softmax top-k as one wave computes it.  TEST INFRASTRUCTURE ONLY.

Restates `ref_topk` of the reference's bit-level model etx/ops/topk_key32.py:122-147 (which follows the device
tile etx/ops/topk.py:35-156 and dsl_topk_lds, etx/ops/gemv.py:712-749):

  * W lanes, ceil(E / W) logits per lane, lane `l` holds experts l, l + W, ...;
  * m = fmaxf over all logits (NaN ignored), p = expf(l - m), s = xor-butterfly sum of the per-lane sums
    (offsets W/2 .. 1), p *= 1 / s;
  * K rounds of an xor-butterfly argmax over p, the lower expert index winning ties; a row with no candidate
    writes id 0x7fffffff (NaN rows);
  * renorm: weight / (weights summed in round order).

The reference models a 64-lane AMD wave with 2 logits per lane; `lanes` generalises the lane count so the same
model describes a 32-lane warp with 4 logits per lane.  The selection (ids) does not depend on `lanes`; the
butterfly summation order, and so the last bits of the weights, does.  numpy's float32 exp is not the device
expf, so weights are compared with a small tolerance and ids exactly.
"""
from __future__ import annotations

import numpy as np

f32 = np.float32
NO_ID = 0x7FFFFFFF


def bf16_bits(x) -> np.ndarray:
    """float32 -> bf16 bit patterns, RNE, NaN kept NaN (etx/ops/topk_key32.py:27-32)."""
    a = np.asarray(x, np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    return np.where(np.isnan(a), ((u >> 16) | 0x40).astype(np.uint16), r)


def bf16_to_f32(b) -> np.ndarray:
    return (np.asarray(b, np.uint32) << 16).astype(np.uint32).view(np.float32)


def _butterfly_sum(v, lanes):
    v = np.asarray(v, f32).copy()
    idx = np.arange(lanes)
    off = lanes // 2
    while off:
        v = (v + v[idx ^ off]).astype(f32)
        off >>= 1
    return f32(v[0])


def wave_topk(bits, K: int, renorm: bool, lanes: int = 64):
    """ids (list of int), weights (list of float32) for one row of bf16 logit bit patterns."""
    E = len(bits)
    per = -(-E // lanes)
    if not 1 <= E or not 1 <= K <= E:
        raise ValueError("need 1 <= K <= E")
    lane = np.arange(lanes)
    vals = bf16_to_f32(bits)
    l = np.full((per, lanes), -np.inf, f32)
    ok = np.zeros((per, lanes), bool)
    for k in range(per):
        e = lane + k * lanes
        ok[k] = e < E
        l[k, ok[k]] = vals[e[ok[k]]]
    m = f32(np.fmax.reduce(np.fmax.reduce(l, axis=0)))
    with np.errstate(all="ignore"):
        p = np.where(ok, np.exp((l - m).astype(f32)).astype(f32), f32(0))
        lane_sum = np.zeros(lanes, f32)
        for k in range(per):                      # s = 0 + p[0] + p[1] ... per lane, then the butterfly
            lane_sum = (lane_sum + p[k]).astype(f32)
        inv = f32(f32(1) / _butterfly_sum(lane_sum, lanes))
        p = np.where(ok, (p * inv).astype(f32), f32(0))
    taken = ~ok
    ids, wts = [], []
    for _ in range(K):
        bv = np.full(lanes, f32(-1)); bi = np.full(lanes, NO_ID, np.int64)
        for k in range(per):
            take = (~taken[k]) & (p[k] > bv)
            bv = np.where(take, p[k], bv); bi = np.where(take, lane + k * lanes, bi)
        off = lanes // 2
        while off:
            ov, oi = bv[lane ^ off], bi[lane ^ off]
            take = (ov > bv) | ((ov == bv) & (oi < bi))
            bv = np.where(take, ov, bv); bi = np.where(take, oi, bi)
            off >>= 1
        b = int(bi[0])
        for k in range(per):
            taken[k] |= (lane + k * lanes) == b
        ids.append(b); wts.append(f32(bv[0]))
    if renorm:
        tot = f32(0)
        for w in wts:
            tot = f32(tot + w)
        with np.errstate(all="ignore"):
            wts = [f32(w / tot) for w in wts]
    return ids, wts
