"""CPU restatement of the absorbed-MLA + DeepSeek-MoE decoder layer (DeepSeek-V2-Lite family).  TEST INFRASTRUCTURE ONLY:
tests and fixture generation may import it; no product path does (no MLA tile is built yet -- this is the oracle the
tiles will be checked against).

It follows the NumPy reference archived in the reference tree,
examples/dsv2lite/results/2026-10-14-k1/b_alld4r0l1kvs_stamps/fleet_src/host/reference_decode.py (third-party
fleet-mi300x snapshot): bf16 rounding points `bf16_round` :36-48 and `rms_norm` :51-66, YaRN rotary tables :84-121,
the interleave-then-rotate rope :129-138, `attention_absorbed` :207-253, `mlp_unit` :256-262, `moe` :265-285,
`decoder_layer` :292-302.  Pinned by tests/golden/mla_layer.npz, which tests/golden/make_golden.py generates by
running that file itself; the operations below are issued in the same order and with the same operand shapes, so the
comparison is bit-exact.

Absorbed form: the cache holds one row c (kv_lora) | k_pe (qk_rope) per position, shared by all heads; W_UK is folded
into the query and W_UV into the output:  q_c[h] = q_nope[h] W_UK[h];  s[h,t] = scale (q_c[h].c[t] + q_pe[h].k_pe[t]);
o_c[h] = sum_t softmax(s)[h,t] c[t];  o[h] = W_UV[h] o_c[h].
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import numpy as np

from .ref_decode import bfr


@dataclass
class MlaDims:
    hidden: int
    heads: int
    kv_lora: int
    qk_nope: int
    qk_rope: int
    v_head: int
    moe_inter: int
    n_routed: int
    top_k: int
    n_shared: int = 2
    dense_inter: int = 0             # > 0: this layer is a dense SwiGLU MLP of that width (layer 0 of DeepSeek-V2-Lite)
    eps: float = 1e-6
    theta: float = 1e4
    rope_factor: float = 40.0
    rope_original_max: int = 4096
    beta_fast: float = 32.0
    beta_slow: float = 1.0
    mscale: float = 0.707
    mscale_all_dim: float = 0.707
    routed_scaling: float = 1.0
    norm_topk: bool = False

    @property
    def q_head(self) -> int:
        return self.qk_nope + self.qk_rope

    @property
    def scale(self) -> float:
        s = self.q_head ** -0.5
        if self.mscale_all_dim:
            m = _yarn_mscale(self.rope_factor, self.mscale_all_dim)
            s = s * m * m
        return s


DSV2_LITE = dict(hidden=2048, heads=16, kv_lora=512, qk_nope=128, qk_rope=64, v_head=128, moe_inter=1408, n_routed=64, top_k=6,
                 n_shared=2, routed_scaling=1.0, norm_topk=False)


# ------------------------------------------------------------------------------------------------ rotary (YaRN)
def _yarn_mscale(scale: float, m: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0


def yarn_tables(d: MlaDims, n_pos: int):
    """(cos, sin) [n_pos, qk_rope]: per-frequency blend of the interpolated and the original inverse frequencies."""
    dim, base = d.qk_rope, d.theta
    expo = np.arange(0, dim, 2, dtype=np.float32) / dim
    f_orig = 1.0 / (base ** expo)
    f_interp = 1.0 / (d.rope_factor * base ** expo)

    def corr(rot):
        return (dim * math.log(d.rope_original_max / (rot * 2 * math.pi))) / (2 * math.log(base))
    low, high = max(math.floor(corr(d.beta_fast)), 0), min(math.ceil(corr(d.beta_slow)), dim - 1)
    if low == high:
        high += 0.001
    ramp = np.clip((np.arange(dim // 2, dtype=np.float32) - low) / (high - low), 0, 1)
    keep = 1.0 - ramp
    inv = f_interp * (1 - keep) + f_orig * keep
    ang = np.outer(np.arange(n_pos, dtype=np.float32), inv)
    ang = np.concatenate([ang, ang], axis=-1)
    m = _yarn_mscale(d.rope_factor, d.mscale) / _yarn_mscale(d.rope_factor, d.mscale_all_dim)
    return np.cos(ang) * m, np.sin(ang) * m


def rope_interleaved(x: np.ndarray, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """DeepSeek's rope: de-interleave (even elements first, then odd), then the half rotation."""
    n = x.shape[-1]
    y = x.reshape(*x.shape[:-1], n // 2, 2).swapaxes(-1, -2).reshape(*x.shape[:-1], n)
    rot = np.concatenate([-y[..., n // 2:], y[..., :n // 2]], axis=-1)
    return y * cos + rot * sin


# ------------------------------------------------------------------------------------------------ pieces
def rmsnorm2(x: np.ndarray, w: np.ndarray, eps: float) -> np.ndarray:
    """bf16(bf16(x / sqrt(mean x^2 + eps)) * w): normalised value and product are both bf16 tensors."""
    x = x.astype(np.float32)
    var = np.mean(x * x, axis=-1, keepdims=True)
    return bfr(bfr(x * (1.0 / np.sqrt(var + eps))) * w.astype(np.float32))


def _softmax(v: np.ndarray) -> np.ndarray:
    e = np.exp(v - np.max(v, axis=-1, keepdims=True))
    return e / np.sum(e, axis=-1, keepdims=True)


def _silu(v: np.ndarray) -> np.ndarray:
    return v / (1.0 + np.exp(-v, dtype=np.float32))


def swiglu(gate: np.ndarray, up: np.ndarray, down: np.ndarray, xn: np.ndarray) -> np.ndarray:
    """bf16(down . bf16(bf16(silu(bf16(gate.x))) * bf16(up.x)))"""
    return bfr(down @ bfr(bfr(_silu(bfr(gate @ xn))) * bfr(up @ xn)))


@dataclass
class MlaLayer:
    """Weights of one layer (float32 holding bf16 values), HF module names."""
    input_layernorm: np.ndarray
    q_proj: np.ndarray                 # [heads * q_head, hidden]
    kv_a_proj_with_mqa: np.ndarray     # [kv_lora + qk_rope, hidden]
    kv_a_layernorm: np.ndarray         # [kv_lora]
    kv_b_proj: np.ndarray              # [heads * (qk_nope + v_head), kv_lora]: per head W_UK rows then W_UV rows
    o_proj: np.ndarray                 # [hidden, heads * v_head]
    post_attention_layernorm: np.ndarray
    mlp: dict = field(default_factory=dict)   # dense: gate, up, down;  MoE: router, egate, eup, edown, sgate, sup, sdown


def synthetic_layer(d: MlaDims, seed: int, std: float = 0.02) -> MlaLayer:
    """Seeded bf16 N(0, std) weights, norm weights 1 + N(0, 0.1), drawn in the field order of MlaLayer then the mlp keys."""
    rng = np.random.default_rng(seed)

    def w(*shape):
        return bfr(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))

    def g(n):
        return bfr(1 + 0.1 * rng.standard_normal(n, dtype=np.float32))
    L = MlaLayer(g(d.hidden), w(d.heads * d.q_head, d.hidden), w(d.kv_lora + d.qk_rope, d.hidden), g(d.kv_lora),
                 w(d.heads * (d.qk_nope + d.v_head), d.kv_lora), w(d.hidden, d.heads * d.v_head), g(d.hidden))
    if d.dense_inter:
        L.mlp = {"gate": w(d.dense_inter, d.hidden), "up": w(d.dense_inter, d.hidden), "down": w(d.hidden, d.dense_inter)}
    else:
        si = d.moe_inter * d.n_shared
        L.mlp = {"router": w(d.n_routed, d.hidden), "egate": w(d.n_routed, d.moe_inter, d.hidden), "eup": w(d.n_routed, d.moe_inter, d.hidden),
                 "edown": w(d.n_routed, d.hidden, d.moe_inter), "sgate": w(si, d.hidden), "sup": w(si, d.hidden), "sdown": w(d.hidden, si)}
    return L


def attention(d: MlaDims, L: MlaLayer, x: np.ndarray, cache: np.ndarray, pos: int, cos: np.ndarray, sin: np.ndarray) -> np.ndarray:
    """One decode step of absorbed MLA; writes row `pos` of cache [n_pos, kv_lora + qk_rope]; returns o_proj's output [hidden]."""
    H, Dk, Dr, Dv, C = d.heads, d.qk_nope, d.qk_rope, d.v_head, d.kv_lora
    xn = rmsnorm2(x, L.input_layernorm, d.eps)
    q = bfr(L.q_proj @ xn).reshape(H, d.q_head)
    kv = bfr(L.kv_a_proj_with_mqa @ xn)
    c_new = rmsnorm2(kv[:C], L.kv_a_layernorm, d.eps)
    kpe_new = bfr(rope_interleaved(kv[C:][None, :], cos[pos][None, :], sin[pos][None, :])[0])
    q_pe = bfr(rope_interleaved(q[:, Dk:], cos[pos][None, :], sin[pos][None, :]))
    cache[pos, :C] = c_new
    cache[pos, C:] = kpe_new
    c, kpe = cache[:pos + 1, :C], cache[:pos + 1, C:]
    out = np.empty(H * Dv, dtype=np.float32)
    for h in range(H):
        b0 = h * (Dk + Dv)
        q_c = q[h, :Dk] @ L.kv_b_proj[b0:b0 + Dk]                                  # W_UK folded into the query: [kv_lora]
        p = _softmax((c @ q_c + kpe @ q_pe[h]) * d.scale)
        out[h * Dv:(h + 1) * Dv] = L.kv_b_proj[b0 + Dk:b0 + Dk + Dv] @ (p @ c)     # W_UV folded into the output
    return bfr(L.o_proj @ bfr(out))


def moe(d: MlaDims, L: MlaLayer, xn: np.ndarray, trace: dict | None = None) -> np.ndarray:
    """fp32 router softmax, top-k unsorted and unnormalised (x routed_scaling) unless norm_topk, routed experts accumulated
    in fp32 in selection order with bf16 per-expert products, plus the shared experts."""
    m = L.mlp
    scores = _softmax(m["router"] @ xn)
    idx = np.argpartition(-scores, d.top_k - 1)[:d.top_k]
    wts = scores[idx]
    wts = wts / (wts.sum() + 1e-20) if (d.top_k > 1 and d.norm_topk) else wts * d.routed_scaling
    y = np.zeros_like(xn)
    for k, e in enumerate(idx):
        y += bfr(wts[k] * swiglu(m["egate"][e], m["eup"][e], m["edown"][e], xn))
    if trace is not None:
        trace["ids"], trace["wts"] = np.asarray(idx, np.int64), np.asarray(wts, np.float32)
    return bfr(bfr(y) + swiglu(m["sgate"], m["sup"], m["sdown"], xn))


def layer(d: MlaDims, L: MlaLayer, x: np.ndarray, cache: np.ndarray, pos: int, cos: np.ndarray, sin: np.ndarray, trace: dict | None = None):
    """x -> bf16(x + attention) -> bf16(. + mlp(norm(.))): one decoder layer; residual adds are bf16 adds."""
    x = bfr(x + attention(d, L, x, cache, pos, cos, sin))
    xn = rmsnorm2(x, L.post_attention_layernorm, d.eps)
    f = swiglu(L.mlp["gate"], L.mlp["up"], L.mlp["down"], xn) if d.dense_inter else moe(d, L, xn, trace)
    return bfr(x + f)


def layer_bytes(d: MlaDims, ctx: int) -> int:
    """Unique HBM bytes of one decode step of one layer at context `ctx` (bf16 weights read once, latent cache read once)."""
    attn = 2 * (d.heads * d.q_head * d.hidden + (d.kv_lora + d.qk_rope) * d.hidden + d.heads * (d.qk_nope + d.v_head) * d.kv_lora
                + d.hidden * d.heads * d.v_head) + 2 * (d.kv_lora + d.qk_rope) * ctx
    if d.dense_inter:
        return attn + 2 * 3 * d.dense_inter * d.hidden
    return attn + 2 * d.n_routed * d.hidden + 2 * 3 * d.moe_inter * d.hidden * (d.top_k + d.n_shared)
