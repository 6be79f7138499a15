"""DeepSeek-V2 family (multi-head latent attention + DeepSeek-MoE) decode step as an ETX program on B200.

What this takes over from the reference: the DeepSeek-V2-Lite task graph of examples/dsv2lite/graph.py:98-209 (qkv_fused,
q_absorb, attention, merge_uv, o_proj, norm_router, expert_gate_up, expert_down, the dense layer, lm_head, argmax), whose
tile bodies there are a third-party library; the arithmetic follows that model's archived NumPy reference
(examples/dsv2lite/results/2026-10-14-k1/b_alld4r0l1kvs_stamps/fleet_src/host/reference_decode.py:207-302).

Phases per layer (one event after each), all inside the one persistent launch of a decode step:
  qkv_a   q_proj and kv_a_proj as ONE streamed GEMV with the input-norm fold (rows: NH q heads of DN + DR, then the
          C + DR row of the latent projection)
  attn    absorbed latent attention, one task per (head, 128 positions): latent norm + rope + cache row, q W_UK, scores
          over the latent cache, softmax statistics, weighted latent; the last partition's task merges and applies W_UV
          (csrc/etxb_mla.cuh)
  o_proj  streamed GEMV
  MoE layers:   router (post-attention norm fold) -> gate+up -> down.  The shared experts are stored as experts
          E .. E + NS - 1 of the same tensors and take the last NS slots of every token with weight 1 (top-k fold mode
          bits 24..27), so routed and shared experts stream through the same two grids and the down tile's
          ascending-id bf16 sum is the expert combine
  dense layers: gate+up (norm fold) -> down
then lm_head with the final-norm fold and the greedy argmax.

Differences from the NumPy reference that stay inside the parity tolerance (2e-2 of scale per layer, greedy tokens equal
outside near ties): router logits are rounded to bf16 before the softmax; the experts' outputs are added in bf16 in
ascending expert id (reference: fp32 in selection order, rounded once; the shared experts as one MLP of width NS * MI
added last); routed_scaling must be 1 (DeepSeek-V2-Lite's value).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

from ..frontends import cuda_link
from ..importer import argblock
from ..ir import Graph, Resource
from ..machine import MachineModel, load_machine
from ..ops import gemv as op_gemv
from ..ops import mla as op_mla
from ..passes import PassOptions, compile_graph
from ..runtime import Session
from . import qwen as Q
from .qwen import SRC, ArgPool

_DT = {"bf16": torch.bfloat16, "f32": torch.float32, "i32": torch.int32, "i64": torch.int64}


@dataclass
class MlaDims:
    name: str
    H: int
    NH: int
    C: int                 # kv_lora_rank: width of the latent
    DN: int                # qk_nope_head_dim
    DR: int                # qk_rope_head_dim
    DV: int                # v_head_dim
    MI: int                # moe_intermediate_size
    E: int                 # routed experts
    TOPK: int
    NS: int                # shared experts (each of width MI)
    DENSE_LAYERS: int      # the first layers are dense MLPs of width DENSE_INTER
    DENSE_INTER: int
    L: int
    V: int
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
    def QH(self) -> int:
        return self.DN + self.DR

    @property
    def ROW(self) -> int:
        return self.C + self.DR

    @property
    def NQKV(self) -> int:
        return self.NH * self.QH + self.ROW

    @property
    def SLOTS(self) -> int:
        return self.TOPK + self.NS

    @property
    def scale(self) -> float:
        s = self.QH ** -0.5
        if self.mscale_all_dim:
            m = _yarn_mscale(self.rope_factor, self.mscale_all_dim)
            s = s * m * m
        return float(np.float32(s))

    def dense(self, layer: int) -> bool:
        return layer < self.DENSE_LAYERS


CONFIGS = {"deepseek-v2-lite": dict(hidden_size=2048, num_attention_heads=16, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                                    moe_intermediate_size=1408, n_routed_experts=64, num_experts_per_tok=6, n_shared_experts=2, first_k_dense_replace=1,
                                    intermediate_size=10944, num_hidden_layers=27, vocab_size=102400, rms_norm_eps=1e-6, rope_theta=10000.0,
                                    rope_scaling=dict(factor=40.0, original_max_position_embeddings=4096, beta_fast=32, beta_slow=1, mscale=0.707,
                                                      mscale_all_dim=0.707), routed_scaling_factor=1.0, norm_topk_prob=False)}


def load_dims(config="deepseek-v2-lite", layers: int | None = None, name: str | None = None) -> MlaDims:
    """config: a bundled name or a HF config dict of the DeepSeek-V2 family."""
    c, nm = (CONFIGS[config], config) if isinstance(config, str) else (config, name or "model")
    rs = c.get("rope_scaling") or {}
    nl = c["num_hidden_layers"] if layers is None else min(layers, c["num_hidden_layers"])
    if float(c.get("routed_scaling_factor", 1.0)) != 1.0:
        raise ValueError("routed_scaling_factor != 1 is not supported by this builder")
    if c.get("q_lora_rank"):
        raise ValueError("a low-rank q projection (q_lora_rank) is not supported by this builder")
    return MlaDims(name=name or nm, H=c["hidden_size"], NH=c["num_attention_heads"], C=c["kv_lora_rank"], DN=c["qk_nope_head_dim"], DR=c["qk_rope_head_dim"],
                   DV=c["v_head_dim"], MI=c["moe_intermediate_size"], E=c["n_routed_experts"], TOPK=c["num_experts_per_tok"], NS=c.get("n_shared_experts", 0),
                   DENSE_LAYERS=min(c.get("first_k_dense_replace", 0), nl), DENSE_INTER=c.get("intermediate_size", 0), L=nl, V=c["vocab_size"],
                   eps=float(c.get("rms_norm_eps", 1e-6)), theta=float(c.get("rope_theta", 1e4)), rope_factor=float(rs.get("factor", 1.0)),
                   rope_original_max=int(rs.get("original_max_position_embeddings", 4096)), beta_fast=float(rs.get("beta_fast", 32)),
                   beta_slow=float(rs.get("beta_slow", 1)), mscale=float(rs.get("mscale", 0.0)), mscale_all_dim=float(rs.get("mscale_all_dim", 0.0)),
                   norm_topk=bool(c.get("norm_topk_prob", False)))


def _yarn_mscale(scale: float, m: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0


def yarn_table(d: MlaDims, maxlen: int) -> np.ndarray:
    """float32 [maxlen][cos(DR) | sin(DR)]: YaRN rotary table -- per frequency a blend of the original inverse frequency and
    the one interpolated by rope_factor (linear ramp between the dimensions that complete beta_fast and beta_slow turns
    within the original context), angles duplicated over the two halves, scaled by mscale / mscale_all_dim."""
    dim, base = d.DR, d.theta
    expo = np.arange(0, dim, 2, dtype=np.float32) / dim
    f_orig = 1.0 / (base ** expo)
    f_interp = 1.0 / (d.rope_factor * base ** expo)

    def turns_dim(rot):
        return (dim * math.log(d.rope_original_max / (rot * 2 * math.pi))) / (2 * math.log(base))
    lo, hi = max(math.floor(turns_dim(d.beta_fast)), 0), min(math.ceil(turns_dim(d.beta_slow)), dim - 1)
    if lo == hi:
        hi += 0.001
    ramp = np.clip((np.arange(dim // 2, dtype=np.float32) - lo) / (hi - lo), 0, 1)
    mask = 1.0 - ramp                                                  # 1: keep the original frequency, 0: fully interpolated
    inv = f_interp * (1 - mask) + f_orig * mask
    ang = np.outer(np.arange(maxlen, dtype=np.float32), inv)
    ang = np.concatenate([ang, ang], axis=-1)
    m = _yarn_mscale(d.rope_factor, d.mscale) / _yarn_mscale(d.rope_factor, d.mscale_all_dim)
    return np.concatenate([np.cos(ang) * m, np.sin(ang) * m], axis=1).astype(np.float32)


# ------------------------------------------------------------------------------------------------ weights and buffers
def weight_shapes(d: MlaDims, maxlen: int) -> dict:
    """name -> (shape, dtype) of every packed weight; per-layer names are prefixed "<layer>."."""
    s = {"embed": ((d.V, d.H), "bf16"), "final_norm": ((d.H,), "bf16"), "lm_head": ((d.V, d.H), "bf16"), "cos_sin": ((maxlen, 2 * d.DR), "f32")}
    for L in range(d.L):
        p = f"{L}."
        s[p + "ln1"], s[p + "ln2"], s[p + "kvln"] = ((d.H,), "bf16"), ((d.H,), "bf16"), ((d.C,), "bf16")
        s[p + "wqa"] = ((d.NQKV, d.H), "bf16")                      # q_proj rows, then kv_a_proj_with_mqa rows
        s[p + "wkvb"] = ((d.NH * (d.DN + d.DV), d.C), "bf16")         # kv_b_proj: per head W_UK rows then W_UV rows
        s[p + "wo"] = ((d.H, d.NH * d.DV), "bf16")
        if d.dense(L):
            s[p + "wgu"], s[p + "wd"] = ((2 * d.DENSE_INTER, d.H), "bf16"), ((d.H, d.DENSE_INTER), "bf16")
        else:
            s[p + "wr"] = ((d.E, d.H), "bf16")
            s[p + "w13"], s[p + "w2"] = ((d.E + d.NS, 2 * d.MI, d.H), "bf16"), ((d.E + d.NS, d.H, d.MI), "bf16")
    return s


def pack_layer(d: MlaDims, L: int, lw) -> dict:
    """HF module tensors of layer L (float arrays holding bf16 values; attributes input_layernorm, q_proj, kv_a_proj_with_mqa,
    kv_a_layernorm, kv_b_proj, o_proj, post_attention_layernorm and the dict mlp with gate / up / down or router, egate,
    eup, edown, sgate, sup, sdown) -> the packed float arrays of weight_shapes."""
    p = f"{L}."
    out = {p + "ln1": lw.input_layernorm, p + "ln2": lw.post_attention_layernorm, p + "kvln": lw.kv_a_layernorm,
           p + "wqa": np.concatenate([lw.q_proj, lw.kv_a_proj_with_mqa], axis=0), p + "wkvb": lw.kv_b_proj, p + "wo": lw.o_proj}
    m = lw.mlp
    if d.dense(L):
        out[p + "wgu"], out[p + "wd"] = np.concatenate([m["gate"], m["up"]], axis=0), m["down"]
    else:
        MI = d.MI
        gate = [m["egate"][e] for e in range(d.E)] + [m["sgate"][i * MI:(i + 1) * MI] for i in range(d.NS)]
        up = [m["eup"][e] for e in range(d.E)] + [m["sup"][i * MI:(i + 1) * MI] for i in range(d.NS)]
        down = [m["edown"][e] for e in range(d.E)] + [m["sdown"][:, i * MI:(i + 1) * MI] for i in range(d.NS)]
        out[p + "wr"] = m["router"]
        out[p + "w13"] = np.stack([np.concatenate([g, u], axis=0) for g, u in zip(gate, up)])
        out[p + "w2"] = np.stack([np.ascontiguousarray(x) for x in down])
    return out


def to_device(d: MlaDims, packed: dict, maxlen: int, device) -> dict:
    """float arrays (bf16 values) -> device tensors of the dtypes weight_shapes names; adds the rotary table."""
    out = {}
    for k, (shape, dt) in weight_shapes(d, maxlen).items():
        a = yarn_table(d, maxlen) if k == "cos_sin" else np.asarray(packed[k], np.float32)
        if tuple(a.shape) != tuple(shape):
            raise ValueError(f"weight {k}: expected shape {shape}, got {a.shape}")
        out[k] = torch.from_numpy(np.ascontiguousarray(a)).to(device).to(_DT[dt]).contiguous()
    return out


def random_weights(d: MlaDims, maxlen: int, device, seed: int = 0, std: float = 0.02) -> dict:
    """Seeded random-init weights generated on the device: linear / embedding weights ~ N(0, std) in bf16, norm weights 1."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    out = {}
    for name, (shape, dt) in weight_shapes(d, maxlen).items():
        if name == "cos_sin":
            out[name] = torch.from_numpy(yarn_table(d, maxlen)).to(device)
            continue
        t = torch.empty(shape, dtype=_DT[dt], device=device)
        if name.rsplit(".", 1)[-1] in ("ln1", "ln2", "kvln", "final_norm"):
            t.fill_(1.0)
        else:
            t.normal_(0.0, std, generator=gen)
        out[name] = t
    return out


def buffer_shapes(d: MlaDims, maxlen: int, steps: int) -> dict:
    mi = max(d.MI, 1)
    s = {"resid": ((d.H,), "bf16"), "resid2": ((d.H,), "bf16"), "hn": ((d.H,), "bf16"), "qkv": ((d.NQKV,), "bf16"),
         "attn_out": ((d.NH * d.DV,), "bf16"), "o": ((d.H,), "bf16"), "o_norm": ((d.H,), "bf16"), "logits": ((d.V,), "bf16"),
         "positions": ((1,), "i64"), "seq_lens": ((1,), "i32"), "slot_mapping": ((1,), "i64"),
         "token_in": ((steps + 2,), "i32"), "token_out": ((steps + 1,), "i32"), "token_time": ((2 * (steps + 1),), "i64"),
         "ckv": ((d.L, maxlen, d.ROW), "bf16"), "moe_out": ((d.H,), "bf16"), "mla_tmp": ((op_mla.tmp_pairs(d.NH, d.C, maxlen), 2), "f32"),
         "rlog": ((max(d.E, 1),), "bf16"), "tw": ((max(d.SLOTS, 1),), "f32"), "ti": ((max(d.SLOTS, 1),), "i32"),
         "mc2": ((max(d.SLOTS * mi, d.DENSE_INTER, 1),), "bf16")}
    return s


def step_bytes(d: MlaDims, ctx: int) -> dict:
    """Unique HBM bytes of one decode step at context `ctx` (bf16 weights read once, latent cache read once)."""
    attn = 2 * (d.NQKV * d.H + d.NH * (d.DN + d.DV) * d.C + d.H * d.NH * d.DV) + 2 * d.ROW * ctx
    dense = attn + 2 * 3 * d.DENSE_INTER * d.H
    moe = attn + 2 * d.E * d.H + 2 * 3 * d.MI * d.H * d.SLOTS
    total = d.DENSE_LAYERS * dense + (d.L - d.DENSE_LAYERS) * moe + 2 * d.V * d.H + 2 * d.H
    return {"dense_layer": dense, "moe_layer": moe, "lm_head": 2 * d.V * d.H, "total": total}


# ------------------------------------------------------------------------------------------------ the graph
def build_graph(d: MlaDims, ptr, maxlen: int = 1072, machine: MachineModel | str = "b200"):
    """The decode step of `d` as a Graph plus its argument pool.  ptr(name) -> device address of a buffer (buffer_shapes) or
    packed weight (weight_shapes).  Returns (graph, pool: ArgPool, info)."""
    m = load_machine(machine) if isinstance(machine, str) else machine
    op_mla.check_shape(d.NH, d.C, d.DN, d.DR, d.DV, maxlen)
    ent = {}
    for mod in (op_gemv, op_mla):
        ent.update(mod.import_entries())
    W = m.workers()
    # task splits: the MoE layers through the sizing of a model with SLOTS expert slots per token, the dense ones as a dense model
    moe_sz = Q.size_for(Q.Dims(name=d.name, H=d.H, NH=d.NH, NKV=d.NH, HD=128, INTER=0, L=1, V=d.V, moe=True, E=d.E, TOPK=d.SLOTS, MI=d.MI), m, maxlen) \
        if d.L > d.DENSE_LAYERS else None
    dense_sz = Q.size_for(Q.Dims(name=d.name, H=d.H, NH=d.NH, NKV=d.NH, HD=128, INTER=d.DENSE_INTER, L=1, V=d.V), m, maxlen) if d.DENSE_LAYERS else None
    g = Graph(f"mla_{d.name}")
    g.codegen.update(fold_topk=True, nb=1, requests=1)
    g.tensor("impargs", ("POOL",), role="weight", bytes_per_elem=1)
    g.tensor("vl", (1,), role="weight", bytes_per_elem=8)
    pool = ArgPool()
    res = Resource(threads=op_gemv.THREADS, vgpr=128, lds_bytes=0)

    def add(name, export, role, layer, blob, tasks, in_ev, out_ev, M=0, K=0, after=None, slots=1):
        off = pool.add(blob)
        pool.rows.append((name, export, role, layer, off, tasks, M, K))
        g.etensor(out_ev, (1,), wait_count=tasks)
        g.call_device(name, (tasks,), cuda_link(SRC, "etx_tile_" + export, stream_after=after), resource=res, args=["impargs"], consts=(off,),
                      in_edges={in_ev: "i->(0)"}, out_edges={out_ev: "i->(0)"},
                      duration_us=round(m.tile_duration_us(role, 2.0 * slots * M * K / max(1, tasks)), 2))
        return out_ev

    def gb(export, tasks, **f):
        return argblock.pack_named(ent[export], (tasks, 1, 1), **f)

    g.etensor("E_pro", (1,), wait_count=1)
    g.call_device("prologue", (1,), cuda_link(SRC, "vl_prologue"), resource=res, args=["vl"], consts=(0,), out_edges={"E_pro": "i->i"}, duration_us=3.8)
    prev = "E_pro"
    cache_layer_bytes = maxlen * d.ROW * 2
    nparts = op_mla.partitions(maxlen)
    for L in range(d.L):
        Wl = lambda n, L=L: ptr(f"{L}.{n}")                                  # noqa: E731
        first = L == 0
        t, rpt = m.gemv_tasks(d.NQKV)
        blob = gb("dsl_gemv_fold", t, W=Wl("wqa"), x=ptr("hn"), out=ptr("qkv"), M=d.NQKV, K=d.H, rpt=rpt, tpe=1, rows=0 if first else ptr("moe_out"),
                  resid_in=ptr("resid") if first else ptr("resid2"), resid_out=0 if first else ptr("resid"), ln=Wl("ln1"), R=0 if first else 1, eps=d.eps,
                  mode=op_gemv.MODE_NORM, nb=1)
        prev = add(f"qkv_{L}", "dsl_gemv_fold", "qkv", L, blob, t, prev, f"E_qkv_{L}", d.NQKV, d.H, after="")
        blob = argblock.pack_named(ent["mla_attn"], (d.NH * (nparts + op_mla.FINISHERS), 1, 1), qkv=ptr("qkv"), kvln=Wl("kvln"), cos_sin=ptr("cos_sin"), wkvb=Wl("wkvb"),
                                   cache=ptr("ckv") + L * cache_layer_bytes, positions=ptr("positions"), out=ptr("attn_out"), NH=d.NH, C=d.C, DN=d.DN, DR=d.DR,
                                   DV=d.DV, maxlen=maxlen, scale=d.scale, eps=d.eps, tmp=ptr("mla_tmp"), max_parts=nparts, tag=L & 0xff)
        prev = add(f"attn_{L}", "mla_attn", "attn_fused", L, blob, d.NH * (nparts + op_mla.FINISHERS), prev, f"E_attn_{L}")
        t, rpt = m.gemv_tasks(d.H)
        blob = gb("dsl_gemv", t, W=Wl("wo"), x=ptr("attn_out"), out=ptr("o"), M=d.H, K=d.NH * d.DV, rpt=rpt, tpe=1, eps=d.eps, nb=1)
        prev = add(f"o_proj_{L}", "dsl_gemv", "o_proj", L, blob, t, prev, f"E_o_{L}", d.H, d.NH * d.DV, after="")
        if d.dense(L):
            spt, tpe, rpt = dense_sz.up
            blob = gb("dsl_moe_up", tpe, W=Wl("wgu"), x=ptr("o_norm"), out=ptr("mc2"), estride=0, M=d.DENSE_INTER, K=d.H, rpt=rpt, tpe=tpe, rows=ptr("o"),
                      resid_in=ptr("resid"), resid_out=ptr("resid2"), ln=Wl("ln2"), R=1, eps=d.eps, mode=op_gemv.MODE_NORM, nb=1)
            prev = add(f"gate_up_{L}", "dsl_moe_up", "gate_up", L, blob, tpe, prev, f"E_up_{L}", d.DENSE_INTER, d.H, after="", slots=2)
            tpe, rpt = dense_sz.down
            blob = gb("dsl_moe_down", tpe, W=Wl("wd"), x=ptr("mc2"), out=ptr("moe_out"), estride=0, M=d.H, K=d.DENSE_INTER, rpt=rpt, tpe=tpe, eps=d.eps, nb=1)
            prev = add(f"down_{L}", "dsl_moe_down", "down", L, blob, tpe, prev, f"E_dn_{L}", d.H, d.DENSE_INTER, after="")
            continue
        t, rpt = moe_sz.router
        blob = gb("dsl_gemv_fold", t, W=Wl("wr"), x=ptr("o_norm"), out=ptr("rlog"), M=d.E, K=d.H, rpt=rpt, tpe=1, rows=ptr("o"), resid_in=ptr("resid"),
                  resid_out=ptr("resid2"), ln=Wl("ln2"), R=1, eps=d.eps, mode=op_gemv.MODE_NORM, nb=1)
        prev = add(f"router_{L}", "dsl_gemv_fold", "router", L, blob, t, prev, f"E_rt_{L}", d.E, d.H, after="")
        topk_mode = (op_gemv.MODE_TOPK_RENORM if d.norm_topk else op_gemv.MODE_TOPK) | op_gemv.mode_shared(d.NS)
        spt, tpe, rpt = moe_sz.up
        groups = d.SLOTS // spt
        blob = gb("dsl_moe_up_fold", groups * tpe, W=Wl("w13"), x=ptr("o_norm"), out=ptr("mc2"), ids=ptr("ti"), wts=ptr("tw"), estride=2 * d.MI * d.H, M=d.MI,
                  K=d.H, rpt=rpt, tpe=tpe, R=d.SLOTS, eps=d.eps, mode=topk_mode | op_gemv.mode_spt(spt), E=d.E, logits=ptr("rlog"), nb=1)
        prev = add(f"moe_up_{L}", "dsl_moe_up_fold", "moe_up", L, blob, groups * tpe, prev, f"E_up_{L}", d.MI, d.H, slots=2 * d.SLOTS)
        tpe, rpt = moe_sz.down
        blob = gb("dsl_moe_down_fold", tpe, W=Wl("w2"), x=ptr("mc2"), out=ptr("moe_out"), ids=ptr("ti"), wts=ptr("tw"), estride=d.H * d.MI, M=d.H, K=d.MI,
                  rpt=rpt, tpe=tpe, R=d.SLOTS, eps=d.eps, mode=topk_mode | op_gemv.MODE_ROUTE_READY | op_gemv.mode_spt(d.SLOTS) | op_gemv.MODE_SUM_SLOTS,
                  E=d.E, logits=ptr("rlog"), nb=1)
        prev = add(f"moe_down_{L}", "dsl_moe_down_fold", "moe_down", L, blob, tpe, prev, f"E_dn_{L}", d.H, d.MI, after=f"E_rt_{L}", slots=d.SLOTS)
    t, rpt = m.gemv_tasks(d.V, waves=1)
    blob = gb("dsl_gemv_fold", t, W=ptr("lm_head"), x=ptr("hn"), out=ptr("logits"), M=d.V, K=d.H, rpt=rpt, tpe=1, rows=ptr("moe_out"), resid_in=ptr("resid2"),
              resid_out=ptr("resid"), ln=ptr("final_norm"), R=1, eps=d.eps, mode=op_gemv.MODE_NORM, nb=1)
    prev = add("lm_head", "dsl_gemv_fold", "lm_head", -1, blob, t, prev, "E_lm", d.V, d.H, after="")
    g.etensor("E_argmax", (1,), wait_count=1)
    g.call_device("argmax", (1,), cuda_link(SRC, "vl_argmax"), resource=res, args=["vl"], consts=(0,), in_edges={prev: "i->(0)"},
                  out_edges={"E_argmax": "i->i"}, duration_us=8.5)
    return g, pool, {"workers": W, "moe": moe_sz, "dense": dense_sz}


class MlaProgram:
    """A DeepSeek-V2-family decode session on one GPU: weights, buffers, latent caches, plan, session, token loop."""

    def __init__(self, dims: MlaDims, weights: dict, device: int = 0, maxlen: int = 1072, steps: int | None = None, machine="b200"):
        self.d, self.maxlen = dims, maxlen
        self.dev = torch.device("cuda", device)
        self.machine = load_machine(machine) if isinstance(machine, str) else machine
        self.steps = steps or maxlen
        self.w = weights
        for k, (shape, dt) in weight_shapes(dims, maxlen).items():
            if k not in weights or tuple(weights[k].shape) != tuple(shape) or weights[k].dtype != _DT[dt]:
                raise ValueError(f"weight {k}: expected {shape} {dt}, got {tuple(weights[k].shape) if k in weights else None}")
        self.buf = {n: torch.zeros(shape, dtype=_DT[dt], device=self.dev) for n, (shape, dt) in buffer_shapes(dims, maxlen, self.steps).items()}
        self.vl = torch.zeros(1, dtype=torch.int64, device=self.dev)

        def ptr(name):
            t = self.buf.get(name)
            if t is None:
                t = self.w[name]
            return t.data_ptr()
        self.graph, self.pool, self.info = build_graph(dims, ptr, maxlen, self.machine)
        pool = self.pool.bytes()
        self.plan = compile_graph(self.graph, self.machine, {"POOL": len(pool)}, options=PassOptions())
        self.session = Session(self.plan, {"vl": self.vl}, pool, device)
        b = self.buf
        self.session.set_step(tok=0, pos=0, write_next=0, H=dims.H, V=dims.V, nrep=1, embed=self.w["embed"], resid=b["resid"], positions=b["positions"],
                              seq_lens=b["seq_lens"], slot_mapping=b["slot_mapping"], logits=b["logits"], token_in=b["token_in"], token_out=b["token_out"],
                              token_time=b["token_time"])

    def read(self, name: str) -> np.ndarray:
        t = self.buf[name]
        return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()

    def step(self, t: int, pos: int, write_next: bool, wait: bool = True):
        self.session.set_step(tok=t, pos=pos, write_next=int(write_next))
        if wait:
            self.session.run(60.0)
        else:
            self.session.launch()

    def generate(self, prompt, n_gen: int, start_pos: int = 0, sync_every: int = 64):
        """Feed `prompt` token by token, then n_gen greedy tokens (the next token never leaves the device)."""
        prompt = [int(x) for x in prompt]
        n = len(prompt) + n_gen - 1
        if n + 2 > self.buf["token_in"].numel() or start_pos + n > self.maxlen:
            raise ValueError("sequence longer than the session was sized for")
        tin = torch.zeros_like(self.buf["token_in"])
        tin[:len(prompt)] = torch.tensor(prompt, dtype=torch.int32)
        self.buf["token_in"].copy_(tin)
        torch.cuda.synchronize(self.dev)
        for t in range(n):
            self.step(t, start_pos + t, write_next=t + 1 >= len(prompt), wait=(t % sync_every == sync_every - 1) or t == n - 1)
        return self.buf["token_out"][len(prompt) - 1:n].cpu().numpy()

    def generate_host(self, prompt, n_gen: int, start_pos: int = 0):
        toks, ms = self.session.decode_host(np.asarray(prompt, np.int32), len(prompt) + n_gen - 1, start_pos)
        return toks[len(prompt) - 1:], ms

    def close(self):
        self.session.close()


__all__ = ["MlaDims", "MlaProgram", "build_graph", "load_dims", "pack_layer", "random_weights", "step_bytes", "to_device", "weight_shapes", "yarn_table"]
