"""CPU oracle of the decode hot path (numpy).  TEST INFRASTRUCTURE ONLY.

This module restates, operation for operation and rounding point for rounding point, the reference's
own CPU numerical path `examples/llm/ref_numpy.py` (cklxx/etx-megakernel):

  bfr            ref_numpy.py:26-32     round-to-nearest-even to bf16, kept as float32
  rmsnorm        ref_numpy.py:71-73     HF RMSNorm in bf16: bfr(w * bfr(x * r))
  rope_tables    ref_numpy.py:76-81     bf16 cos/sin tables
  apply_rope     ref_numpy.py:84-88     rotate_half, every product rounded, the sum rounded
  silu           ref_numpy.py:91-92
  Ref.step       ref_numpy.py:105-158   one decode step (dense SwiGLU or softmax top-k MoE)

It is pinned against that file run in the build container (tests/golden/make_golden.py imports the
reference, drives it with the same synthetic weights, and stores inputs + outputs as fixtures;
tests/test_oracle_golden.py replays them).  Only tests/, __graft_entry__.smoke() and bench.py's
cpu_baseline / --impl reference legs may import this package; the product path (the CUDA library and
the host package) never does.

The paged KV-cache helpers restate the cache layout of the reference's attention-prep tile
(etx/ops/attnprep.py:3-6, 146-165): key cache [blocks][NKV][HD/X][BS][X], value cache
[blocks][NKV][HD][BS], slot = slot_mapping[0], block = slot / BS, offset = slot % BS.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

f32 = np.float32


# ----------------------------------------------------------------------------- bf16 helpers
def bfr(x):
    """Round to nearest even to bf16, returned as float32 (ref_numpy.py:26-32)."""
    x = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
    u = x.view(np.uint32)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    return r.view(np.float32)


def f32_to_bf16_bits(x) -> np.ndarray:
    """float32 values that are already bf16-exact (or not: RNE) -> uint16 bit patterns."""
    return (bfr(x).view(np.uint32) >> 16).astype(np.uint16)


def bf16_bits_to_f32(a) -> np.ndarray:
    """uint16 bf16 bit patterns -> float32 (ref_numpy.py:35-36)."""
    return (np.asarray(a).astype(np.uint32) << 16).view(np.float32)


# ----------------------------------------------------------------------------- model dims
@dataclass
class Dims:
    """The shape record of examples/llm/model.py:45-78 (same field names)."""
    name: str
    H: int
    NH: int
    NKV: int
    HD: int
    INTER: int
    L: int
    V: int
    eps: float = 1e-6
    theta: float = 1e6
    tie: bool = False
    bias: bool = False
    qk_norm: bool = True
    moe: bool = False
    E: int = 0
    TOPK: int = 0
    MI: int = 0
    norm_topk: bool = False

    @property
    def G(self) -> int:
        return self.NH // self.NKV

    @property
    def NQKV(self) -> int:
        return (self.NH + 2 * self.NKV) * self.HD


def dims_from_config(c: dict, name: str = "model", layers: int | None = None) -> Dims:
    """HF config dict -> Dims, the subset of load_dims (examples/llm/model.py:94-147) the decode path needs."""
    H, NH = c["hidden_size"], c["num_attention_heads"]
    E = next((int(c[k]) for k in ("num_experts", "num_local_experts", "n_routed_experts") if c.get(k)), 0)
    mt = c.get("model_type", "")
    L = c["num_hidden_layers"] if layers is None else min(layers, c["num_hidden_layers"])
    return Dims(name=name, H=H, NH=NH, NKV=c.get("num_key_value_heads", NH), HD=c.get("head_dim", H // NH),
                INTER=c.get("intermediate_size", 0), L=L, V=c["vocab_size"], eps=float(c.get("rms_norm_eps", 1e-6)),
                theta=float((c.get("rope_parameters") or {}).get("rope_theta", c.get("rope_theta", 10000.0))),
                tie=bool(c.get("tie_word_embeddings", False)),
                bias=mt == "qwen2" or bool(c.get("attention_bias", False)), qk_norm=mt.startswith("qwen3"),
                moe=E > 0, E=E, TOPK=int(c.get("num_experts_per_tok", 0)),
                MI=c.get("moe_intermediate_size") or (c.get("intermediate_size", 0) if E else 0),
                norm_topk=bool(c.get("norm_topk_prob", mt == "mixtral")))


QWEN3_30B_A3B = {"hidden_size": 2048, "intermediate_size": 6144, "moe_intermediate_size": 768, "num_experts": 128,
                 "num_experts_per_tok": 8, "norm_topk_prob": True, "num_attention_heads": 32,
                 "num_key_value_heads": 4, "head_dim": 128, "num_hidden_layers": 48, "vocab_size": 151936,
                 "rms_norm_eps": 1e-06, "rope_theta": 1000000.0, "tie_word_embeddings": False,
                 "model_type": "qwen3_moe"}
QWEN3_8B = {"hidden_size": 4096, "intermediate_size": 12288, "num_attention_heads": 32, "num_key_value_heads": 8,
            "head_dim": 128, "num_hidden_layers": 36, "vocab_size": 151936, "rms_norm_eps": 1e-06,
            "rope_theta": 1000000, "tie_word_embeddings": False, "model_type": "qwen3"}


# ----------------------------------------------------------------------------- primitives
def rmsnorm(x, w, eps):
    """HF Qwen2RMSNorm in bf16 (ref_numpy.py:71-73): the normalised value is rounded, then the product."""
    r = np.float32(1.0) / np.sqrt(np.float32(np.mean(x.astype(np.float32) ** 2)) + np.float32(eps))
    return bfr(w * bfr(x * r))


def rope_tables(theta, hd, ctx):
    """bf16 cos/sin tables [ctx][hd/2] (ref_numpy.py:76-81)."""
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, hd, 2, dtype=np.float32) / np.float32(hd)))).astype(np.float32)
    pos = np.arange(ctx, dtype=np.float32)[:, None]
    f = pos * inv[None, :]
    return bfr(np.cos(f)), bfr(np.sin(f))


def apply_rope(v, cos, sin):
    """rotate_half; each product rounded, the sum rounded (ref_numpy.py:84-88)."""
    half = v.shape[-1] // 2
    rot = np.concatenate([-v[half:], v[:half]])
    c = np.concatenate([cos, cos]); s = np.concatenate([sin, sin])
    return bfr(bfr(v * c) + bfr(rot * s))


def silu(g):
    return g / (np.float32(1.0) + np.exp(-g))


def softmax_topk(logits, k, renorm):
    """Router selection of Ref.step (ref_numpy.py:136-141): fp32 softmax, top-k with ties to the lower id,
    optional renormalisation, weights rounded to bf16.  Returns (ids in selection order, bf16 weights)."""
    logits = np.asarray(logits, np.float32)
    pr = np.exp(logits - logits.max()); pr = pr / pr.sum()
    order = np.lexsort((np.arange(len(pr)), -pr))[:k]
    wts = pr[order]
    if renorm:
        wts = wts / wts.sum()
    return order.astype(np.int32), bfr(wts)


# ----------------------------------------------------------------------------- synthetic weights
class SyntheticWeights:
    """Seeded random-init weights under HF tensor names, values bf16-exact float32.

    Draw order (fixed so every user of a seed sees the same bytes): embed, final norm, lm_head, then per layer
    input_layernorm, post_attention_layernorm, q/k/v_proj, q_norm, k_norm, o_proj, then router + experts
    (gate, up, down per expert) or the dense gate/up/down.  Linear and embedding weights ~ N(0, std); norm gammas
    ~ N(0, std) when gamma == "normal" (the single-layer parity configuration) or exactly 1.0 when "ones".
    """

    def __init__(self, d: Dims, seed: int = 0, std: float = 0.02, gamma: str = "ones"):
        self.d, self.t = d, {}
        rng = np.random.default_rng(seed)

        def lin(*shape):
            return bfr(rng.standard_normal(shape, dtype=np.float32) * np.float32(std))

        def gam(n):
            return lin(n) if gamma == "normal" else np.ones(n, np.float32)
        t = self.t
        t["model.embed_tokens.weight"] = lin(d.V, d.H)
        t["model.norm.weight"] = gam(d.H)
        if not d.tie:
            t["lm_head.weight"] = lin(d.V, d.H)
        for L in range(d.L):
            p = f"model.layers.{L}."
            t[p + "input_layernorm.weight"] = gam(d.H)
            t[p + "post_attention_layernorm.weight"] = gam(d.H)
            a = p + "self_attn."
            t[a + "q_proj.weight"] = lin(d.NH * d.HD, d.H)
            t[a + "k_proj.weight"] = lin(d.NKV * d.HD, d.H)
            t[a + "v_proj.weight"] = lin(d.NKV * d.HD, d.H)
            if d.bias:
                t[a + "q_proj.bias"] = lin(d.NH * d.HD)
                t[a + "k_proj.bias"] = lin(d.NKV * d.HD)
                t[a + "v_proj.bias"] = lin(d.NKV * d.HD)
            if d.qk_norm:
                t[a + "q_norm.weight"] = gam(d.HD)
                t[a + "k_norm.weight"] = gam(d.HD)
            t[a + "o_proj.weight"] = lin(d.H, d.NH * d.HD)
            m = p + "mlp."
            if d.moe:
                t[m + "gate.weight"] = lin(d.E, d.H)
                for e in range(d.E):
                    t[f"{m}experts.{e}.gate_proj.weight"] = lin(d.MI, d.H)
                    t[f"{m}experts.{e}.up_proj.weight"] = lin(d.MI, d.H)
                    t[f"{m}experts.{e}.down_proj.weight"] = lin(d.H, d.MI)
            else:
                t[m + "gate_proj.weight"] = lin(d.INTER, d.H)
                t[m + "up_proj.weight"] = lin(d.INTER, d.H)
                t[m + "down_proj.weight"] = lin(d.H, d.INTER)

    def __contains__(self, k):
        return k in self.t

    def get(self, k):
        return self.t[k]


class DictWeights:
    """Weights handed over as a dict of float32 arrays (e.g. copied back from the GPU by bench.py)."""

    def __init__(self, tensors: dict):
        self.t = tensors

    def __contains__(self, k):
        return k in self.t

    def get(self, k):
        return self.t[k]


# ----------------------------------------------------------------------------- the decode step
class Ref:
    """Decode-step oracle: Ref.step of ref_numpy.py:95-158 with an injected weight provider.

    `trace` (optional dict) receives the intermediates of the LAST layer run, for per-tile parity:
    xs1, qkv_raw, q, k, v, attn, o, resid2, xs2, rlog, ids, wts, act, y, x_out (MoE) / gu, hh, dn (dense).
    """

    def __init__(self, d: Dims, W, ctx: int):
        self.d, self.W, self.ctx = d, W, ctx
        self.cos, self.sin = rope_tables(d.theta, d.HD, ctx)
        self.kc = np.zeros((d.L, ctx, d.NKV, d.HD), np.float32)
        self.vc = np.zeros((d.L, ctx, d.NKV, d.HD), np.float32)

    def layer(self, L: int, x, pos: int, trace=None):
        d, W = self.d, self.W
        p = f"model.layers.{L}."
        xs = rmsnorm(x, W.get(p + "input_layernorm.weight"), d.eps)
        a = p + "self_attn."
        q = bfr(W.get(a + "q_proj.weight") @ xs + (W.get(a + "q_proj.bias") if (a + "q_proj.bias") in W else 0))
        k = bfr(W.get(a + "k_proj.weight") @ xs + (W.get(a + "k_proj.bias") if (a + "k_proj.bias") in W else 0))
        v = bfr(W.get(a + "v_proj.weight") @ xs + (W.get(a + "v_proj.bias") if (a + "v_proj.bias") in W else 0))
        if trace is not None:
            trace["xs1"] = xs.copy(); trace["qkv_raw"] = np.concatenate([q, k, v])
        q = q.reshape(d.NH, d.HD); k = k.reshape(d.NKV, d.HD); v = v.reshape(d.NKV, d.HD)
        if d.qk_norm:
            qn, kn = W.get(a + "q_norm.weight"), W.get(a + "k_norm.weight")
            q = np.stack([rmsnorm(h, qn, d.eps) for h in q]); k = np.stack([rmsnorm(h, kn, d.eps) for h in k])
        q = np.stack([apply_rope(h, self.cos[pos], self.sin[pos]) for h in q])
        k = np.stack([apply_rope(h, self.cos[pos], self.sin[pos]) for h in k])
        self.kc[L, pos] = k; self.vc[L, pos] = v
        scale = np.float32(1.0 / np.sqrt(d.HD))
        o = np.zeros((d.NH, d.HD), np.float32)
        for h in range(d.NH):
            kvh = h // d.G
            K = self.kc[L, : pos + 1, kvh]; V = self.vc[L, : pos + 1, kvh]
            s = (K @ q[h]) * scale
            s = s - s.max(); pr = np.exp(s); pr = pr / pr.sum()
            o[h] = bfr(pr @ V)
        op = bfr(W.get(a + "o_proj.weight") @ o.reshape(-1))
        x = bfr(x + op)
        xs = rmsnorm(x, W.get(p + "post_attention_layernorm.weight"), d.eps)
        if trace is not None:
            trace.update(q=q.copy(), k=k.copy(), v=v.copy(), attn=o.copy(), o=op, resid2=x.copy(), xs2=xs.copy())
        m = p + "mlp."
        if d.moe:
            logits = bfr(W.get(m + "gate.weight") @ xs)
            pr = np.exp(logits - logits.max()); pr = pr / pr.sum()
            order = np.lexsort((np.arange(d.E), -pr))[: d.TOPK]        # top-k, ties -> lower id
            wts = pr[order]
            if d.norm_topk:
                wts = wts / wts.sum()
            wts = bfr(wts)
            acc = np.float32(0.0)
            acts, ys = {}, {}
            for e, we in sorted(zip(order.tolist(), wts.tolist())):     # ascending expert id, like index_add_
                g = bfr(W.get(f"{m}experts.{e}.gate_proj.weight") @ xs)
                u = bfr(W.get(f"{m}experts.{e}.up_proj.weight") @ xs)
                hh = bfr(bfr(silu(g)) * u)
                y = bfr(bfr(W.get(f"{m}experts.{e}.down_proj.weight") @ hh) * np.float32(we))
                acc = bfr(acc + y)
                acts[e], ys[e] = hh, y
            x = bfr(x + acc)
            if trace is not None:
                trace.update(rlog=logits, ids=order.astype(np.int32), wts=wts,
                             act=np.stack([acts[e] for e in order.tolist()]),
                             y=np.stack([ys[e] for e in order.tolist()]), x_out=x.copy())
        else:
            g = bfr(W.get(m + "gate_proj.weight") @ xs); u = bfr(W.get(m + "up_proj.weight") @ xs)
            hh = bfr(bfr(silu(g)) * u)
            dn = bfr(W.get(m + "down_proj.weight") @ hh)
            x = bfr(x + dn)
            if trace is not None:
                trace.update(hh=hh, dn=dn, x_out=x.copy())
        return x

    def step(self, tok: int, pos: int, dump=None, trace=None, return_logits: bool = False):
        d, W = self.d, self.W
        x = W.get("model.embed_tokens.weight")[tok].copy()
        for L in range(d.L):
            x = self.layer(L, x, pos, trace)
            if dump is not None:
                dump.append(x.copy())
        xs = rmsnorm(x, W.get("model.norm.weight"), d.eps)
        lm = W.get("lm_head.weight") if "lm_head.weight" in W else W.get("model.embed_tokens.weight")
        logits = bfr(lm @ xs)
        tok = int(np.argmax(logits))                     # first max wins, like torch.argmax
        return (tok, logits) if return_logits else tok


# ----------------------------------------------------------------------------- paged KV cache (layout oracle)
def paged_shapes(nblocks: int, nkv: int, hd: int, bs: int = 16, x: int = 8):
    return (nblocks, nkv, hd // x, bs, x), (nblocks, nkv, hd, bs)


def paged_write(kc, vc, k, v, slot: int):
    """Write one token's k [NKV][HD] and v [NKV][HD] at `slot` (etx/ops/attnprep.py:146-165 addressing).
    kc: [blocks][NKV][HD/X][BS][X], vc: [blocks][NKV][HD][BS]; any dtype."""
    bs, x = kc.shape[3], kc.shape[4]
    blk, off = slot // bs, slot % bs
    nkv, hd = k.shape
    kc[blk, :, :, off, :] = k.reshape(nkv, hd // x, x)
    vc[blk, :, :, off] = v


def paged_from_contig(K, V, nblocks: int, bs: int = 16, x: int = 8, dtype=np.float32):
    """Contiguous caches [ctx][NKV][HD] -> paged arrays holding the first ctx positions (identity block table)."""
    ctx, nkv, hd = K.shape
    ks, vs = paged_shapes(nblocks, nkv, hd, bs, x)
    kc = np.zeros(ks, dtype); vc = np.zeros(vs, dtype)
    n = (ctx // bs) * bs
    if n:
        kb = K[:n].reshape(n // bs, bs, nkv, hd // x, x)
        kc[: n // bs] = kb.transpose(0, 2, 3, 1, 4)
        vb = V[:n].reshape(n // bs, bs, nkv, hd)
        vc[: n // bs] = vb.transpose(0, 2, 3, 1)
    for t in range(n, ctx):
        paged_write(kc, vc, K[t], V[t], t)
    return kc, vc


def paged_to_contig(kc, vc, ctx: int):
    nb, nkv, hdx, bs, x = kc.shape
    K = kc.transpose(0, 3, 1, 2, 4).reshape(nb * bs, nkv, hdx * x)[:ctx]
    V = vc.transpose(0, 3, 1, 2).reshape(nb * bs, nkv, hdx * x)[:ctx]
    return K, V


# ----------------------------------------------------------------------------- standalone GEMV (sweep oracle)
def gemv(Wm, x):
    """out[m][n] = bfr(W[n,:] . x[m,:]) with fp32 accumulation; x is [M][K] or [K]."""
    x = np.asarray(x, np.float32)
    return bfr(x @ Wm.T) if x.ndim == 2 else bfr(Wm @ x)


# ----------------------------------------------------------------------------- byte ledger (algorithmic bytes)
def step_bytes(d: Dims, context: int, batch: int = 1, active_experts: float | None = None) -> dict:
    """Bytes one decode step must move (bf16 = 2 B), the ledger the reference prints with
    `python -m examples.vllm_llm.byte_ledger` (docs/qwen/BANDWIDTH-2026-10-07.md:24): per layer norms + qkv + o +
    router + routed experts + KV read/write, plus lm_head and one embedding row."""
    per = {}
    per["norms"] = 2 * (2 * d.H + (2 * d.HD if d.qk_norm else 0))
    per["qkv"] = 2 * d.NQKV * d.H
    per["o"] = 2 * d.H * d.NH * d.HD
    if d.moe:
        per["router"] = 2 * d.E * d.H
        n_e = d.TOPK if batch == 1 and active_experts is None else active_experts
        per["experts"] = int(n_e * 3 * d.MI * d.H * 2)
    else:
        per["mlp"] = 3 * d.INTER * d.H * 2
    per["kv"] = batch * (2 * d.NKV * d.HD * 2 * context + 2 * d.NKV * d.HD * 2)
    layer = sum(per.values())
    total = layer * d.L + 2 * d.V * d.H + 2 * d.H * batch
    return {"per_layer": per, "layer": layer, "lm_head": 2 * d.V * d.H, "total": total}
