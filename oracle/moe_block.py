"""Synthetic MoE-block acceptance fixture (fp32 vectorised path against a scalar float64 restatement).
TEST INFRASTRUCTURE ONLY.

Restates the reference's CPU gate for the MoE block, etx/bench/numerical.py:13-118:
  * `fixture`            seeded N(0, 0.15) float32 tensors: x, unit norm weight, router, gate/up/down per expert
  * `block_fp32`         RMSNorm -> router -> softmax -> top-k (ties to the smallest id) -> optional renorm ->
                         SwiGLU experts -> weighted sum + residual, all float32 numpy
  * `block_scalar64`     the same block with python floats and math.fsum, its own routing
  * `check_output`       finite, completely written, shapes agree, allclose(atol = rtol = 2e-5); the tolerance
                         must be finite so the gate cannot be switched off
The known answers (tests/golden/moe_block_*.npz) were produced by running the reference module itself.
"""
from __future__ import annotations

import math

import numpy as np


def check_output(actual, expected, written, *, atol=2e-5, rtol=2e-5) -> list[str]:
    if not (math.isfinite(atol) and math.isfinite(rtol) and atol >= 0 and rtol >= 0):
        raise ValueError("tolerances must be finite and nonnegative")
    actual, expected, written = np.asarray(actual), np.asarray(expected), np.asarray(written)
    if actual.shape != expected.shape or written.shape != expected.shape or expected.size == 0:
        return ["output/reference/write-mask shape mismatch or empty output"]
    problems = []
    if written.dtype != np.bool_ or not written.all():
        problems.append("output not completely written")
    if not np.isfinite(expected).all():
        problems.append("invalid nonfinite reference")
    if not np.isfinite(actual).all():
        problems.append("nonfinite output")
    if not problems and not np.allclose(actual, expected, atol=atol, rtol=rtol):
        problems.append("numerical mismatch")
    return problems


def fixture(*, experts=8, top_k=2, hidden=8, intermediate=12, seed=17, renormalize=True) -> dict:
    if not 1 <= top_k <= experts or hidden <= 0 or intermediate <= 0:
        raise ValueError("invalid MoE dimensions or top-k")
    rng = np.random.default_rng(seed)
    draw = lambda shape: rng.normal(0, 0.15, shape).astype(np.float32)          # noqa: E731
    x = draw(hidden)
    return {"x": x, "norm": np.ones(hidden, np.float32), "router": draw((experts, hidden)),
            "gate": draw((experts, intermediate, hidden)), "up": draw((experts, intermediate, hidden)),
            "down": draw((experts, hidden, intermediate)), "top_k": top_k, "renormalize": renormalize, "eps": 1e-5}


def block_fp32(data):
    x = data["x"]
    xn = x * (1 / np.sqrt(np.mean(x * x) + data["eps"])) * data["norm"]
    logits = data["router"] @ xn
    p = np.exp(logits - logits.max())
    p /= p.sum()
    chosen = np.lexsort((np.arange(len(p)), -p))[: data["top_k"]]
    w = p[chosen]
    if data["renormalize"]:
        w = w / w.sum()
    g = data["gate"][chosen] @ xn
    u = data["up"][chosen] @ xn
    mid = g / (1 + np.exp(-g)) * u
    contrib = (data["down"][chosen] @ mid[..., None])[..., 0] * w[:, None]
    out = (x + contrib.sum(axis=0)).astype(np.float32)
    return out, np.ones(x.shape, bool), chosen.tolist()


def block_scalar64(data):
    x = [float(v) for v in data["x"]]
    n = len(x)
    rms = math.sqrt(math.fsum(v * v for v in x) / n + data["eps"])
    xn = [v * float(data["norm"][i]) / rms for i, v in enumerate(x)]
    dot = lambda row, vec: math.fsum(float(a) * b for a, b in zip(row, vec))    # noqa: E731
    logits = [dot(row, xn) for row in data["router"]]
    top = max(logits)
    ex = [math.exp(v - top) for v in logits]
    tot = math.fsum(ex)
    p = [v / tot for v in ex]
    chosen = sorted(range(len(p)), key=lambda i: (-p[i], i))[: data["top_k"]]
    denom = math.fsum(p[i] for i in chosen) if data["renormalize"] else 1.0
    parts = [[] for _ in x]
    for e in chosen:
        mid = []
        for grow, urow in zip(data["gate"][e], data["up"][e]):
            g, u = dot(grow, xn), dot(urow, xn)
            mid.append(g / (1 + math.exp(-g)) * u)
        for i, row in enumerate(data["down"][e]):
            parts[i].append(p[e] / denom * dot(row, mid))
    return np.asarray([v + math.fsum(r) for v, r in zip(x, parts)]), chosen
