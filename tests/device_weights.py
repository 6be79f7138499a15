"""HF-named float32 views of packed bf16 weights that live on the GPU, fetched tensor by tensor on demand.

The oracle (oracle/ref_decode.py: Ref) asks its weight provider for one tensor at a time (`get(name)`, `name in W`).
For a full-size random-init model (61 GB for Qwen3-30B-A3B) the weights exist only on the device; this provider copies
what a step touches -- per layer the dense matrices (cached on the host after their first use) and the experts the
router selected (8 of 128, not cached) -- so the oracle follows the 36- and 48-layer models in a second or two per
token.  Test infrastructure, like the oracle itself.
"""
from __future__ import annotations

import re

import numpy as np
import torch

_LAYER = re.compile(r"model\.layers\.(\d+)\.(.+)")
_EXPERT = re.compile(r"mlp\.experts\.(\d+)\.(gate|up|down)_proj\.weight")


class _Rows:
    """`embed[tok]` without bringing the whole embedding to the host."""

    def __init__(self, t):
        self.t = t

    def __getitem__(self, i):
        return self.t[int(i)].float().cpu().numpy()

    def __matmul__(self, x):                         # tied lm_head: the embedding used as a matrix
        if not hasattr(self, "full"):
            self.full = self.t.float().cpu().numpy()
        return self.full @ x


class DeviceWeights:
    """Small tensors and (up to `cache_bytes` of) dense matrices are kept on the host after their first use; anything
    larger comes through one pinned staging buffer and is valid until the next large `get` -- the oracle multiplies a
    matrix as soon as it has fetched it, so one buffer is enough and the host never holds the model."""

    STAGE_BYTES = 256 << 20

    def __init__(self, d, packed: dict, cache_bytes: int = 6 << 30):
        """d: models.qwen.Dims of the packed model; packed: name -> bf16 device tensor (models.qwen.weight_shapes)."""
        self.d, self.w, self.cache = d, packed, {}
        self.room = cache_bytes
        self.stage = torch.empty(self.STAGE_BYTES // 4, dtype=torch.float32)
        if torch.cuda.is_available():
            self.stage = self.stage.pin_memory()

    def _f(self, t, cacheable: bool = True) -> np.ndarray:
        n = t.numel()
        if n * 4 <= (1 << 20) or n * 4 > self.STAGE_BYTES:             # small (kept by the caller's cache) or too large to stage
            return t.float().cpu().numpy()
        if cacheable and n * 4 <= self.room:                                          # a dense matrix that still fits the host cache
            self.room -= n * 4
            return t.float().cpu().numpy()
        view = self.stage[:n].view(t.shape)
        view.copy_(t.float() if t.is_cuda else t)                       # widened on the device, then one copy into pinned memory
        self._staged = True
        return view.numpy()

    def __contains__(self, k):
        if k == "lm_head.weight":
            return "lm_head" in self.w
        if k.endswith("proj.bias"):
            return self.d.bias
        return True

    def get(self, k):
        if k in self.cache:
            return self.cache[k]
        d, w = self.d, self.w
        keep = True
        self._staged = False
        if k == "model.embed_tokens.weight":
            v = _Rows(w["embed"])
        elif k == "model.norm.weight":
            v = self._f(w["final_norm"])
        elif k == "lm_head.weight":
            v = self._f(w["lm_head"])
        else:
            m = _LAYER.fullmatch(k)
            if not m:
                raise KeyError(k)
            L, rest = int(m.group(1)), m.group(2)
            p = f"{L}."
            nq, nk = d.NH * d.HD, d.NKV * d.HD
            e = _EXPERT.fullmatch(rest)
            if e:
                ei, kind = int(e.group(1)), e.group(2)
                keep = False
                v = self._f(w[p + "w2"][ei] if kind == "down" else w[p + "w13"][ei, :d.MI] if kind == "gate" else w[p + "w13"][ei, d.MI:], cacheable=False)
            elif rest == "input_layernorm.weight":
                v = self._f(w[p + "ln1"])
            elif rest == "post_attention_layernorm.weight":
                v = self._f(w[p + "ln2"])
            elif rest == "self_attn.q_proj.weight":
                v = self._f(w[p + "wqkv"][:nq])
            elif rest == "self_attn.k_proj.weight":
                v = self._f(w[p + "wqkv"][nq:nq + nk])
            elif rest == "self_attn.v_proj.weight":
                v = self._f(w[p + "wqkv"][nq + nk:])
            elif rest == "self_attn.q_proj.bias":
                v = self._f(w[p + "bqkv"][:nq])
            elif rest == "self_attn.k_proj.bias":
                v = self._f(w[p + "bqkv"][nq:nq + nk])
            elif rest == "self_attn.v_proj.bias":
                v = self._f(w[p + "bqkv"][nq + nk:])
            elif rest == "self_attn.q_norm.weight":
                v = self._f(w[p + "qn"])
            elif rest == "self_attn.k_norm.weight":
                v = self._f(w[p + "kn"])
            elif rest == "self_attn.o_proj.weight":
                v = self._f(w[p + "wo"])
            elif rest == "mlp.gate.weight":
                v = self._f(w[p + "wr"])
            elif rest == "mlp.gate_proj.weight":
                v = self._f(w[p + "wgu"][:d.INTER])
            elif rest == "mlp.up_proj.weight":
                v = self._f(w[p + "wgu"][d.INTER:])
            elif rest == "mlp.down_proj.weight":
                v = self._f(w[p + "wd"])
            else:
                raise KeyError(k)
        if keep and not self._staged:
            self.cache[k] = v
        return v


# ---------------------------------------------------------------------------------------------- DeepSeek-V2 family
class LazyExperts:
    """m["egate"][e]-style access to one expert's rows of a packed device tensor, fetched when the oracle asks for them."""

    def __init__(self, t, rows=None):
        self.t, self.rows = t, rows

    def __getitem__(self, e):
        a = self.t[int(e)]
        return (a[self.rows] if self.rows is not None else a).float().cpu().numpy()


def mla_oracle_dims(R, d, dense: bool):
    return R.MlaDims(hidden=d.H, heads=d.NH, kv_lora=d.C, qk_nope=d.DN, qk_rope=d.DR, v_head=d.DV, moe_inter=d.MI, n_routed=d.E, top_k=d.TOPK, n_shared=d.NS,
                     dense_inter=d.DENSE_INTER if dense else 0, eps=d.eps, theta=d.theta, rope_factor=d.rope_factor, rope_original_max=d.rope_original_max,
                     beta_fast=d.beta_fast, beta_slow=d.beta_slow, mscale=d.mscale, mscale_all_dim=d.mscale_all_dim, norm_topk=d.norm_topk)


def mla_oracle_layer(R, d, weights: dict, L: int):
    """oracle.ref_mla.MlaLayer of layer L over the device's packed weights (models.dsv2.weight_shapes): the shared experts are
    experts E .. E + NS - 1 of the packed tensors, the routed experts are fetched one by one when the oracle selects them."""
    g = lambda n: weights[f"{L}.{n}"].float().cpu().numpy()                 # noqa: E731
    wqa = g("wqa")
    lw = R.MlaLayer(g("ln1"), wqa[:d.NH * d.QH], wqa[d.NH * d.QH:], g("kvln"), g("wkvb"), g("wo"), g("ln2"))
    if d.dense(L):
        wgu = g("wgu")
        lw.mlp = {"gate": wgu[:d.DENSE_INTER], "up": wgu[d.DENSE_INTER:], "down": g("wd")}
    else:
        w13, w2 = weights[f"{L}.w13"], weights[f"{L}.w2"]
        sh = [w13[d.E + i].float().cpu().numpy() for i in range(d.NS)]
        lw.mlp = {"router": g("wr"), "egate": LazyExperts(w13, slice(0, d.MI)), "eup": LazyExperts(w13, slice(d.MI, 2 * d.MI)), "edown": LazyExperts(w2),
                  "sgate": np.concatenate([s[:d.MI] for s in sh]), "sup": np.concatenate([s[d.MI:] for s in sh]),
                  "sdown": np.concatenate([w2[d.E + i].float().cpu().numpy() for i in range(d.NS)], axis=1)}
    return lw
