"""Qwen-family decode (dense SwiGLU and softmax top-k MoE) as an ETX program on the B200 megakernel.

What this module takes over from the reference:
  * `Dims` / `load_dims`         examples/llm/model.py:45-147 (same field names; HF config.json -> shape record)
  * the task graph of one step   examples/vllm_llm/model.py:254-705 (`instances`, `build`): phases per layer in launch
                                 order, one argument block per grid instance, one event between consecutive phases
  * packed weight layouts        examples/vllm_llm/prep.py:71-150: wqkv = [q; k; v], w13 = [E][gate rows; up rows][H],
                                 w2 = [E][H][I], cos_sin = bf16 [maxlen][cos(HD/2) | sin(HD/2)]
  * the argument-block fill      examples/vllm_llm/host.hip:340-522
  * module protocol              build() / bindings() / runtime()  (etx/contracts/compiler.py:33-39)

Phases per layer on B200 (one event tensor after each):
  qkv (norm fold, R expert rows summed in bf16 in ascending expert id)  ->  prep (per kv head: q/k norm, rope, cache write)
  -> attn (32 positions x kv head)  -> reduce (per q head)  -> o_proj  -> router (norm fold; task 0 stores residual + normed x)
  -> moe_up (top-k folded in; per-slot events)  -> moe_down  -> [next layer's qkv]           (dense: gate_up -> down)
then lm_head (final norm fold) -> argmax.  Task counts follow the machine model (one wave of tasks per SM for the
dense GEMVs, two for the expert phases), not the MI300X numbers of the reference.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from pathlib import Path

import numpy as np

from ..frontends import cuda_link
from ..importer import argblock
from ..ir import Graph, Resource
from ..machine import MachineModel, load_machine
from ..ops import attn as op_attn
from ..ops import attnprep as op_prep
from ..ops import gemv as op_gemv

BS, X = 16, 8            # paged KV block size and key-cache inner width (vLLM layout the reference uses)
SRC = "etx-megakernel_b200/csrc"

CONFIGS = {
    "qwen3-30b-a3b": {"hidden_size": 2048, "intermediate_size": 6144, "moe_intermediate_size": 768, "num_experts": 128,
                      "num_experts_per_tok": 8, "norm_topk_prob": True, "num_attention_heads": 32, "num_key_value_heads": 4,
                      "head_dim": 128, "num_hidden_layers": 48, "vocab_size": 151936, "rms_norm_eps": 1e-06, "rope_theta": 1000000.0,
                      "tie_word_embeddings": False, "model_type": "qwen3_moe"},
    "qwen3-8b": {"hidden_size": 4096, "intermediate_size": 12288, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
                 "num_hidden_layers": 36, "vocab_size": 151936, "rms_norm_eps": 1e-06, "rope_theta": 1000000, "tie_word_embeddings": False,
                 "model_type": "qwen3"},
}


@dataclass
class Dims:
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
    VL: int = 0            # rows of the lm_head this rank holds when a sharded model splits it by vocabulary (0: all V)

    @property
    def lm_rows(self) -> int:
        return self.VL or self.V

    @property
    def G(self) -> int:
        return self.NH // self.NKV

    @property
    def NQKV(self) -> int:
        return (self.NH + 2 * self.NKV) * self.HD


def load_dims(config=None, layers: int | None = None, name: str | None = None) -> Dims:
    """config: a bundled name ("qwen3-30b-a3b", "qwen3-8b"), a path to a HF config.json, or the dict itself."""
    if config is None:
        config = "qwen3-8b"
    if isinstance(config, dict):
        c, nm = config, name or "model"
    elif config in CONFIGS:
        c, nm = CONFIGS[config], config
    else:
        p = Path(config)
        c, nm = json.loads(p.read_text()), (p.parent.name if p.name == "config.json" else p.stem)
    rs = (c.get("rope_scaling") or c.get("rope_parameters") or {})
    kind = rs.get("rope_type") or rs.get("type") or "default"
    if kind != "default":
        raise ValueError(f"{nm}: unsupported rope type {kind}")
    mt = c.get("model_type", "")
    E = next((int(c[k]) for k in ("num_experts", "num_local_experts", "n_routed_experts") if c.get(k)), 0)
    topk = int(c.get("num_experts_per_tok", 0))
    if not E and any("expert" in k for k in c):
        raise ValueError(f"{nm}: config mentions experts but no expert count is set; refusing to plan it as dense")
    if E and not 1 <= topk <= min(E, 16):
        raise ValueError(f"{nm}: num_experts_per_tok={topk} must be between 1 and {min(E, 16)}")
    if E and (c.get("mlp_only_layers") or c.get("decoder_sparse_step", 1) != 1 or c.get("first_k_dense_replace", 0)
              or c.get("n_shared_experts", 0) or c.get("shared_expert_intermediate_size", 0)):
        raise ValueError("mixed dense / MoE layer layouts (or shared experts) are not supported by this builder")
    H, NH = c["hidden_size"], c["num_attention_heads"]
    nl = c["num_hidden_layers"] if layers is None else min(layers, c["num_hidden_layers"])
    return Dims(name=name or nm, H=H, NH=NH, NKV=c.get("num_key_value_heads", NH), HD=c.get("head_dim", H // NH),
                INTER=c.get("intermediate_size", 0), L=nl, V=c["vocab_size"], eps=float(c.get("rms_norm_eps", 1e-6)),
                theta=float((c.get("rope_parameters") or {}).get("rope_theta", c.get("rope_theta", 10000.0))),
                tie=bool(c.get("tie_word_embeddings", False)), bias=mt == "qwen2" or bool(c.get("attention_bias", False)),
                qk_norm=mt.startswith("qwen3"), moe=E > 0, E=E, TOPK=topk,
                MI=c.get("moe_intermediate_size") or (c.get("intermediate_size", 0) if E else 0),
                norm_topk=bool(c.get("norm_topk_prob", mt == "mixtral")))


def rope_table(theta: float, hd: int, maxlen: int) -> np.ndarray:
    """bf16 bit patterns [maxlen][cos(hd/2) | sin(hd/2)]: float32 angles pos * theta^(-2i/hd), cos / sin rounded to
    nearest even (HF rotary embedding evaluated in float32, stored in bf16)."""
    inv = (1.0 / (np.float32(theta) ** (np.arange(0, hd, 2, dtype=np.float32) / np.float32(hd)))).astype(np.float32)
    f = np.arange(maxlen, dtype=np.float32)[:, None] * inv[None, :]
    t = np.concatenate([np.cos(f), np.sin(f)], axis=1).astype(np.float32)
    u = np.ascontiguousarray(t).view(np.uint32)
    return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


# ------------------------------------------------------------------------------------------------ sharding
def kv_replication(d: Dims, ranks: int) -> int:
    """How many ranks hold a copy of each kv head when `d` is sharded `ranks` ways: 1 while the kv heads split evenly,
    ranks / NKV when there are more ranks than kv heads (Qwen3-30B-A3B on 8 ranks: 4 kv heads, each on 2 ranks, which
    hold different halves of its 8 q heads).  Raises where the heads do not split."""
    if d.NH % ranks:
        raise ValueError(f"{d.name}: {d.NH} q heads do not split {ranks} ways")
    if d.NKV % ranks == 0:
        return 1
    qpr = d.NH // ranks                                                  # q heads per rank: all of them must share one kv head
    if ranks % d.NKV or d.G % qpr:
        raise ValueError(f"{d.name}: {d.NKV} kv heads neither split nor replicate over {ranks} ranks ({qpr} q heads per rank, {d.G} per kv head)")
    return ranks // d.NKV


def shard_dims(d: Dims, ranks: int, shard_vocab: bool = True) -> Dims:
    """The model one of `ranks` tensor-parallel ranks runs: its share of the q heads, its kv heads (a share of them, or --
    more ranks than kv heads -- the one kv head its q heads attend to, replicated: kv_replication), its share of the MLP
    (or of every expert's) intermediate rows and -- shard_vocab, when the vocabulary splits into multiples of 8 -- of the
    lm_head's rows; hidden size, embedding, experts and router stay whole."""
    from dataclasses import replace
    if ranks == 1:
        return d
    mi = d.MI if d.moe else d.INTER
    rep = kv_replication(d, ranks)
    if mi % ranks or (mi // ranks) % 8:
        raise ValueError(f"{d.name}: {mi} intermediate rows do not split {ranks} ways into multiples of 8")
    return replace(d, name=f"{d.name}/tp{ranks}", NH=d.NH // ranks, NKV=d.NKV // ranks if rep == 1 else 1, MI=d.MI // ranks if d.moe else d.MI,
                   INTER=d.INTER if d.moe else d.INTER // ranks, VL=d.V // ranks if shard_vocab and d.V % (8 * ranks) == 0 else 0)


def exchange_bytes(d: Dims, ranks: int) -> int:
    """Size of a rank's exchange region: per layer one [ranks][H] block of flagged 4-byte words for o_proj and one for down."""
    return 2 * d.L * ranks * d.H * 4 + ARGMAX_BLOCK


ARGMAX_BLOCK = 256         # tail of a region: [ranks] 16-byte slots of the sharded argmax (exchange_argmax_offset)


def argmax_offset(d: Dims, ranks: int) -> int:
    return 2 * d.L * ranks * d.H * 4


def shard_weights(w: dict, d: Dims, ranks: int, rank: int, shard_vocab: bool = True) -> dict:
    """Packed weights of the whole model `d` (weight_shapes) -> those of rank `rank` of shard_dims(d, ranks): q / k / v rows
    and gate / up rows by columns of the output (column-parallel), o_proj and down by columns of the input
    (row-parallel), everything else replicated.  Works on numpy arrays and torch tensors alike."""
    if ranks == 1:
        return dict(w)
    cat = (lambda xs, axis: np.concatenate(xs, axis)) if isinstance(w["embed"], np.ndarray) else \
        (lambda xs, axis: __import__("torch").cat(xs, axis))
    cont = (lambda a: np.ascontiguousarray(a)) if isinstance(w["embed"], np.ndarray) else (lambda a: a.contiguous())
    nq, nk = d.NH * d.HD, d.NKV * d.HD
    rep = kv_replication(d, ranks)
    ql = nq // ranks
    # this rank's k / v rows: its share of the kv heads, or the one (replicated) kv head its q heads belong to
    kl, k0 = (nk // ranks, rank * (nk // ranks)) if rep == 1 else (d.HD, (rank // rep) * d.HD)
    mi = d.MI if d.moe else d.INTER
    ml = mi // ranks
    vl = shard_dims(d, ranks, shard_vocab).VL
    out = {}
    for name, a in w.items():
        kind = name.rsplit(".", 1)[-1]
        if kind in ("wqkv", "bqkv"):
            a = cat([a[rank * ql:(rank + 1) * ql], a[nq + k0:nq + k0 + kl], a[nq + nk + k0:nq + nk + k0 + kl]], 0)
        elif kind == "wo":
            a = cont(a[:, rank * ql:(rank + 1) * ql])
        elif kind == "w13":
            a = cat([a[:, rank * ml:(rank + 1) * ml], a[:, mi + rank * ml:mi + (rank + 1) * ml]], 1)
        elif kind == "wgu":
            a = cat([a[rank * ml:(rank + 1) * ml], a[mi + rank * ml:mi + (rank + 1) * ml]], 0)
        elif kind in ("w2", "wd"):
            a = cont(a[..., rank * ml:(rank + 1) * ml])
        elif name == "lm_head" and vl:
            a = a[rank * vl:(rank + 1) * vl]
        out[name] = a
    return out


# ------------------------------------------------------------------------------------------------ sizing
@dataclass
class Sizing:
    workers: int
    qkv: tuple          # (tasks, rows per task)
    o: tuple
    router: tuple
    up: tuple           # (expert slots per task, row chunks per slot group, rows per chunk)
    down: tuple         # (tasks, rows per task): every task covers all slots and sums them
    lm: tuple
    parts: int          # attention partitions (of 32 positions) covering maxlen
    attn: tuple = (0, 0, 0)   # grouped attention tile: (q heads per task, positions per task, partitions); (0, 0, 0): general tile


def size_for(d: Dims, m: MachineModel, maxlen: int) -> Sizing:
    W = m.workers()
    slots = d.TOPK if d.moe else 1
    mi = d.MI if d.moe else d.INTER

    def up_split():
        """(slots per task, chunks per slot group, rows per chunk): the divisor of the slot count that loads the SMs most
        evenly with ONE task per SM (a task then streams 2 * spt * rpt rows without a restart)."""
        best = None
        for spt in [s for s in range(1, slots + 1) if slots % s == 0]:
            groups = slots // spt
            tpe = max(1, W // groups)
            rpt = -(-mi // tpe)
            tpe = -(-mi // rpt)
            if 2 * spt * rpt > op_gemv.MAX_RESULTS or groups * tpe > W:
                continue
            eff = (slots * mi) / (W * spt * rpt)
            if best is None or eff > best[0] + 1e-9 or (abs(eff - best[0]) < 1e-9 and spt > best[1]):
                best = (eff, spt, tpe, rpt)
        if best is None:
            raise ValueError("no expert task split fits the tile limits")
        return best[1:]
    dt, drpt = m.gemv_tasks(d.H)
    return Sizing(workers=W, qkv=m.gemv_tasks(d.NQKV), o=m.gemv_tasks(d.H), router=m.gemv_tasks(d.E) if d.moe else (0, 0),
                  up=up_split(), down=(dt, drpt), lm=m.gemv_tasks(d.lm_rows, waves=1), parts=-(-maxlen // m.attention_part()),
                  attn=m.attention_groups(d.NH, d.NKV, d.HD, BS, maxlen))


# ------------------------------------------------------------------------------------------------ buffers
def buffer_shapes(d: Dims, maxlen: int, steps: int, parts: int) -> dict:
    """name -> (shape, dtype) of every activation / runtime buffer of one request (examples/vllm_llm/host.hip:274-317)."""
    nblk = -(-maxlen // BS)
    s = {"resid": ((d.H,), "bf16"), "resid2": ((d.H,), "bf16"), "hn": ((d.H,), "bf16"), "qkv": ((d.NQKV,), "bf16"),
         "attn_out": ((d.NH * d.HD,), "bf16"), "o": ((d.H,), "bf16"), "o_norm": ((d.H,), "bf16"),
         "logits": ((d.V,), "bf16"), "positions": ((1,), "i64"), "seq_lens": ((1,), "i32"), "slot_mapping": ((1,), "i64"),
         "block_tables": ((nblk,), "i32"), "token_in": ((steps + 2,), "i32"), "token_out": ((steps + 1,), "i32"),
         "token_time": ((2 * (steps + 1),), "i64"),
         "exp_sums": ((d.NH, parts), "f32"), "max_logits": ((d.NH, parts), "f32"), "tmp_out": ((d.NH, parts, max(d.HD, op_attn.GQ_PARTIAL_FLOATS)), "f32"),
         "kc": ((d.L, nblk, d.NKV, d.HD // X, BS, X), "bf16"), "vc": ((d.L, nblk, d.NKV, d.HD, BS), "bf16"),
         "attn_counters": ((d.L, d.NH), "i32"), "moe_out": ((d.H,), "bf16")}
    if d.moe:
        s.update({"rlog": ((d.E,), "bf16"), "tw": ((d.TOPK,), "f32"), "ti": ((d.TOPK,), "i32"), "tei": ((d.TOPK,), "i32"),
                  "mc2": ((d.TOPK, d.MI), "bf16"), "mc3": ((d.TOPK, d.H), "bf16")})
    else:
        s.update({"mc2": ((1, d.INTER), "bf16"), "mc3": ((1, d.H), "bf16")})
    return s


def weight_shapes(d: Dims, maxlen: int) -> dict:
    """name -> shape of every packed weight tensor (bf16); per-layer names are prefixed "<layer>."."""
    s = {"embed": (d.V, d.H), "final_norm": (d.H,), "cos_sin": (maxlen, d.HD)}
    if not d.tie:
        s["lm_head"] = (d.lm_rows, d.H)
    for L in range(d.L):
        p = f"{L}."
        s[p + "ln1"], s[p + "ln2"] = (d.H,), (d.H,)
        s[p + "wqkv"], s[p + "wo"] = (d.NQKV, d.H), (d.H, d.NH * d.HD)
        if d.bias:
            s[p + "bqkv"] = (d.NQKV,)
        if d.qk_norm:
            s[p + "qn"], s[p + "kn"] = (d.HD,), (d.HD,)
        if d.moe:
            s[p + "wr"], s[p + "w13"], s[p + "w2"] = (d.E, d.H), (d.E, 2 * d.MI, d.H), (d.E, d.H, d.MI)
        else:
            s[p + "wgu"], s[p + "wd"] = (2 * d.INTER, d.H), (d.H, d.INTER)
    return s


def pack_hf(d: Dims, get, maxlen: int) -> dict:
    """HF-named float32 (bf16-exact) numpy tensors -> packed uint16 arrays in the layouts above.  `get(name)` returns a
    tensor or raises KeyError."""
    def b(a):
        u = np.ascontiguousarray(np.asarray(a, np.float32)).view(np.uint32)
        return (u >> 16).astype(np.uint16)
    out = {"embed": b(get("model.embed_tokens.weight")), "final_norm": b(get("model.norm.weight")),
           "cos_sin": rope_table(d.theta, d.HD, maxlen)}
    if not d.tie:
        out["lm_head"] = b(get("lm_head.weight"))
    for L in range(d.L):
        p, q = f"model.layers.{L}.", f"{L}."
        a = p + "self_attn."
        out[q + "ln1"], out[q + "ln2"] = b(get(p + "input_layernorm.weight")), b(get(p + "post_attention_layernorm.weight"))
        out[q + "wqkv"] = b(np.concatenate([get(a + "q_proj.weight"), get(a + "k_proj.weight"), get(a + "v_proj.weight")]))
        if d.bias:
            out[q + "bqkv"] = b(np.concatenate([get(a + "q_proj.bias"), get(a + "k_proj.bias"), get(a + "v_proj.bias")]))
        if d.qk_norm:
            out[q + "qn"], out[q + "kn"] = b(get(a + "q_norm.weight")), b(get(a + "k_norm.weight"))
        out[q + "wo"] = b(get(a + "o_proj.weight"))
        m = p + "mlp."
        if d.moe:
            out[q + "wr"] = b(get(m + "gate.weight"))
            out[q + "w13"] = np.stack([np.concatenate([b(get(f"{m}experts.{e}.gate_proj.weight")), b(get(f"{m}experts.{e}.up_proj.weight"))])
                                       for e in range(d.E)])
            out[q + "w2"] = np.stack([b(get(f"{m}experts.{e}.down_proj.weight")) for e in range(d.E)])
        else:
            out[q + "wgu"] = np.concatenate([b(get(m + "gate_proj.weight")), b(get(m + "up_proj.weight"))])
            out[q + "wd"] = b(get(m + "down_proj.weight"))
    return out


def unpack_layer_hf(d: Dims, packed_get, L: int, out_layer: int | None = None) -> dict:
    """Inverse of pack_hf for one layer: packed uint16 arrays -> HF-named float32 tensors (for a CPU cross-check of
    weights that were generated on the device)."""
    def f(u):
        return (np.asarray(u).astype(np.uint32) << 16).view(np.float32)
    o = L if out_layer is None else out_layer
    p, q = f"model.layers.{o}.", f"{L}."
    a, m = p + "self_attn.", p + "mlp."
    nq, nk = d.NH * d.HD, d.NKV * d.HD
    wqkv = f(packed_get(q + "wqkv"))
    t = {p + "input_layernorm.weight": f(packed_get(q + "ln1")), p + "post_attention_layernorm.weight": f(packed_get(q + "ln2")),
         a + "q_proj.weight": wqkv[:nq], a + "k_proj.weight": wqkv[nq:nq + nk], a + "v_proj.weight": wqkv[nq + nk:],
         a + "o_proj.weight": f(packed_get(q + "wo"))}
    if d.bias:
        bq = f(packed_get(q + "bqkv"))
        t.update({a + "q_proj.bias": bq[:nq], a + "k_proj.bias": bq[nq:nq + nk], a + "v_proj.bias": bq[nq + nk:]})
    if d.qk_norm:
        t[a + "q_norm.weight"], t[a + "k_norm.weight"] = f(packed_get(q + "qn")), f(packed_get(q + "kn"))
    if d.moe:
        t[m + "gate.weight"] = f(packed_get(q + "wr"))
        w13, w2 = f(packed_get(q + "w13")), f(packed_get(q + "w2"))
        for e in range(d.E):
            t[f"{m}experts.{e}.gate_proj.weight"], t[f"{m}experts.{e}.up_proj.weight"] = w13[e, :d.MI], w13[e, d.MI:]
            t[f"{m}experts.{e}.down_proj.weight"] = w2[e]
    else:
        wgu = f(packed_get(q + "wgu"))
        t[m + "gate_proj.weight"], t[m + "up_proj.weight"], t[m + "down_proj.weight"] = wgu[:d.INTER], wgu[d.INTER:], f(packed_get(q + "wd"))
    return t


# ------------------------------------------------------------------------------------------------ the graph
class ArgPool:
    """Argument blocks of every grid instance, 16-byte aligned, in graph order (plan_offsets, model.py:403-425)."""

    def __init__(self):
        self.buf = bytearray()
        self.rows = []          # (grid name, export, role, layer, offset, tasks, M, K)

    def add(self, data: bytes) -> int:
        self.buf += b"\0" * (-len(self.buf) % 16)
        off = len(self.buf)
        self.buf += data
        return off

    def bytes(self) -> bytes:
        return bytes(self.buf + b"\0" * (-len(self.buf) % 16))


def build_graph(d: Dims, ptr, maxlen: int = 1072, machine: MachineModel | str = "b200", *, fold_topk: bool = True,
                fused_attn: bool | str = True, ranks: int = 1, rank: int = 0, flagged: bool = False):
    """The decode step of `d` as a Graph plus its argument pool.

    flagged (one rank): hand the row-parallel grids' outputs (o_proj, down) to the norm folds that follow as flagged words
    in an exchange region of one row per block -- the single-GPU form of the sharded hand-off below: the fold polls the
    data itself instead of waiting for the producing grid's event and then loading.

    ranks > 1: the step of ONE rank of a model sharded `ranks` ways (`d` = shard_dims(full, ranks): its share of the
    heads and of the MLP / expert rows).  ptr("xrows") then names the rank's exchange region: 2 * L blocks of
    [ranks][H] flagged words (exchange_bytes); the row-parallel grids (o_proj, down) are marked `exchange` and publish
    the rows they wrote into row `rank` of their block on every rank, the norm folds that follow read all `ranks`
    rows from their own rank's copy and add them in rank order.

    ptr(name) -> device address (int) of a buffer (buffer_shapes) or packed weight (weight_shapes); "kc" / "vc" are the
    whole [L, ...] caches (layer slices are addressed by offset here).  Returns (graph, pool: ArgPool, sizing)."""
    m = load_machine(machine) if isinstance(machine, str) else machine
    sz = size_for(d, m, maxlen)
    ent = {}
    for mod in (op_gemv, op_prep, op_attn):
        ent.update(mod.import_entries())
    from ..ops import topk as op_topk
    ent.update(op_topk.import_entries())
    g = Graph(f"vl_{d.name}")
    g.codegen.update(fold_topk=fold_topk, nb=1, requests=1)
    g.tensor("impargs", ("POOL",), role="weight", bytes_per_elem=1)
    g.tensor("vl", (1,), role="weight", bytes_per_elem=8)
    pool = ArgPool()
    res = Resource(threads=op_gemv.THREADS, vgpr=128, lds_bytes=0)
    nblk = -(-maxlen // BS)
    kv_layer_bytes = nblk * d.NKV * d.HD * BS * 2
    slots = d.TOPK if d.moe else 1
    mi = d.MI if d.moe else d.INTER
    scale = float(np.float32(1.0 / np.sqrt(d.HD)))
    hf_mode = op_gemv.MODE_BF16_WTS

    if not (1 <= ranks <= 8 and 0 <= rank < ranks):
        raise ValueError("1 <= ranks <= 8 and 0 <= rank < ranks")
    exch = ranks > 1 or flagged
    xmode = op_gemv.MODE_FLAGGED if exch else 0

    def xblock(layer, kind):
        """The block of flagged rows o_proj (kind 0) / down (kind 1) of `layer` publish into; 0 when not sharded."""
        return ptr("xrows") + (2 * layer + kind) * ranks * d.H * 4 if exch else 0

    def tile(symbol, stream_after=None, exchange=False):
        return cuda_link(SRC, symbol, stream_after=stream_after, exchange=exchange)

    def add(name, export, role, layer, blob, tasks, grid, in_ev, in_map, out_ev, out_map, out_shape, out_count, M=0, K=0, after=None, exchange=False):
        off = pool.add(blob)
        pool.rows.append((name, export, role, layer, off, tasks, M, K))
        g.etensor(out_ev, out_shape, wait_count=out_count)
        slots = (d.TOPK if role in ("moe_up", "moe_down") else 1) * (2 if role in ("moe_up", "gate_up") else 1)
        g.call_device(name, grid, tile("etx_tile_" + export, after, exchange and exch), resource=res, args=["impargs"], consts=(off,),
                      in_edges={in_ev: in_map}, out_edges={out_ev: out_map},
                      duration_us=round(m.tile_duration_us(role, 2.0 * slots * M * K / max(1, tasks)), 2))
        return out_ev

    def gemv_block(export, tasks, **f):
        return argblock.pack_named(ent[export], (tasks, 1, 1), **f)

    g.etensor("E_pro", (1,), wait_count=1)
    g.call_device("prologue", (1,), tile("vl_prologue"), resource=res, args=["vl"], consts=(0,), out_edges={"E_pro": "i->i"}, duration_us=3.8)
    prev = "E_pro"
    before_x = prev
    for L in range(d.L):
        W = lambda n, L=L: ptr(f"{L}.{n}")                                  # noqa: E731
        # ---- qkv with the input-norm fold
        t, rpt = sz.qkv
        first = L == 0
        blob = gemv_block("dsl_gemv_fold", t, W=W("wqkv"), x=ptr("hn"), out=ptr("qkv"), M=d.NQKV, K=d.H, rpt=rpt, tpe=1,
                          rows=0 if first else (xblock(L - 1, 1) or ptr("moe_out")), resid_in=ptr("resid") if first else ptr("resid2"),
                          resid_out=0 if first else ptr("resid"), ln=W("ln1"), R=0 if first else ranks, eps=d.eps,
                          ids=0, wts=W("bqkv") if d.bias else 0,
                          mode=op_gemv.MODE_NORM | (op_gemv.MODE_BIAS if d.bias else 0) | (0 if first else xmode), nb=1)
        # (sharded: the fold polls the step flags of the rows the ranks publish, which says more than the exchanged grid's
        # event -- that only counts this rank's tasks -- so it waits for the event BEFORE that grid and starts polling at once)
        prev = add(f"qkv_{L}", "dsl_gemv_fold", "qkv", L, blob, t, (t,), (before_x if exch and not first else prev), "i->(0)", f"E_qkv_{L}", "i->(0)", (1,), t, d.NQKV, d.H, after="")
        if fused_attn:
            # ---- the attention phase as one grid: prep + split-KV partitions + merge by the last task to finish
            gq, plen, gparts = (0, 0, 0) if fused_attn == "general" else sz.attn
            nparts, ntask = (gparts, gparts * (d.NH // gq)) if gq else (sz.parts, sz.parts * d.NKV)
            op_attn.check_fused(d.NH, d.NKV, d.HD, BS, X, nparts, gq, plen)
            blob = argblock.pack_named(ent["attn_fused"], (ntask, 1, 1), qkv=ptr("qkv"), qw=W("qn") if d.qk_norm else 0,
                                       kw=W("kn") if d.qk_norm else 0, cos_sin=ptr("cos_sin"), kc=ptr("kc") + L * kv_layer_bytes,
                                       vc=ptr("vc") + L * kv_layer_bytes, block_tables=ptr("block_tables"), seq_lens=ptr("seq_lens"),
                                       positions=ptr("positions"), slot_mapping=ptr("slot_mapping"), exp_sums=ptr("exp_sums"),
                                       max_logits=ptr("max_logits"), tmp_out=ptr("tmp_out"), out=ptr("attn_out"),
                                       counters=ptr("attn_counters") + 4 * L * d.NH, scale=scale, eps=d.eps, NH=d.NH, NKV=d.NKV, HD=d.HD,
                                       BS=BS, X=X, max_parts=nparts, gq=gq, part_len=op_attn.tagged_part_len(L) if gq else plen)
            prev = add(f"attn_{L}", "attn_fused", "attn_fused", L, blob, ntask, (ntask,), prev, "i->(0)",
                       f"E_red_{L}", "i->(0)", (1,), ntask)
        else:
            # ---- attention prep per kv head
            blob = argblock.pack_named(ent["dsl_attnprep"], (d.NKV, 1, 1), qkv=ptr("qkv"), qw=W("qn") if d.qk_norm else 0,
                                       kw=W("kn") if d.qk_norm else 0, cos_sin=ptr("cos_sin"), positions=ptr("positions"),
                                       kc=ptr("kc") + L * kv_layer_bytes, vc=ptr("vc") + L * kv_layer_bytes, slot_mapping=ptr("slot_mapping"),
                                       NH=d.NH, NKV=d.NKV, HD=d.HD, eps=d.eps, BS=BS, X=X)
            prev = add(f"prep_{L}", "dsl_attnprep", "prep", L, blob, d.NKV, (d.NKV,), prev, "i->(0)", f"E_prep_{L}", "i->i", (d.NKV,), 1)
            # ---- attention partitions and their merge
            ablob = argblock.pack_named(ent["attn_decode"], (sz.parts * d.NKV, 1, 1), q=ptr("qkv"), kc=ptr("kc") + L * kv_layer_bytes,
                                        vc=ptr("vc") + L * kv_layer_bytes, block_tables=ptr("block_tables"), seq_lens=ptr("seq_lens"),
                                        exp_sums=ptr("exp_sums"), max_logits=ptr("max_logits"), tmp_out=ptr("tmp_out"), out=ptr("attn_out"),
                                        scale=scale, NH=d.NH, NKV=d.NKV, HD=d.HD, BS=BS, X=X, max_parts=sz.parts, max_blocks=nblk)
            prev = add(f"attn_{L}", "attn_decode", "attn", L, ablob, sz.parts * d.NKV, (sz.parts * d.NKV,), prev, f"i->(i%{d.NKV})",
                       f"E_attn_{L}", f"i->(i%{d.NKV})", (d.NKV,), sz.parts)
            rblob = ablob[:op_attn.GRID_OFF] + np.asarray([d.NH, 1, 1, d.NH], "<u4").tobytes()
            prev = add(f"reduce_{L}", "attn_reduce", "reduce", L, rblob, d.NH, (d.NH,), prev, f"i->(i/{d.G})", f"E_red_{L}", "i->(0)", (1,), d.NH)

        # ---- o_proj
        t, rpt = sz.o
        blob = gemv_block("dsl_gemv", t, W=W("wo"), x=ptr("attn_out"), out=ptr("o"), M=d.H, K=d.NH * d.HD, rpt=rpt, tpe=1, eps=d.eps, nb=1,
                          rows=xblock(L, 0), mode=xmode)
        before_x = prev
        prev = add(f"o_proj_{L}", "dsl_gemv", "o_proj", L, blob, t, (t,), prev, "i->(0)", f"E_o_{L}", "i->(0)", (1,), t, d.H, d.NH * d.HD, after="", exchange=True)
        fold_in = before_x if exch else prev
        if d.moe:
            # ---- router with the post-attention norm fold: task 0 stores resid2 and the normed vector
            t, rpt = sz.router
            blob = gemv_block("dsl_gemv_fold", t, W=W("wr"), x=ptr("o_norm"), out=ptr("rlog"), M=d.E, K=d.H, rpt=rpt, tpe=1, rows=xblock(L, 0) or ptr("o"),
                              resid_in=ptr("resid"), resid_out=ptr("resid2"), ln=W("ln2"), R=ranks, eps=d.eps, mode=op_gemv.MODE_NORM | xmode, nb=1)
            prev = add(f"router_{L}", "dsl_gemv_fold", "router", L, blob, t, (t,), fold_in, "i->(0)", f"E_rt_{L}", "i->(0)", (1,), t, d.E, d.H, after="")
            topk_mode = (op_gemv.MODE_TOPK_RENORM if d.norm_topk else op_gemv.MODE_TOPK) | hf_mode
            if not fold_topk:
                from ..ops import topk as op_topk2
                blob = argblock.pack_named(op_topk2.import_entries()["dsl_topk"], (1, 1, 1), logits=ptr("rlog"), wts=ptr("tw"), ids=ptr("ti"),
                                           tei=ptr("tei"), E=d.E, K=d.TOPK, mode=(1 if d.norm_topk else 0) | hf_mode, nbsv=0)
                prev = add(f"topk_{L}", "dsl_topk", "topk", L, blob, 1, (1,), prev, "i->(0)", f"E_topk_{L}", "i->(0)", (1,), 1)
            # ---- experts: one gate+up task per SM (spt slots x one row chunk), then one down task per SM that covers every
            #      slot of its output rows and adds them in bf16 in ascending expert id (the expert combine)
            spt, tpe, rpt = sz.up
            groups = slots // spt
            up_export = "dsl_moe_up_fold" if fold_topk else "dsl_moe_up"
            blob = gemv_block(up_export, groups * tpe, W=W("w13"), x=ptr("o_norm"), out=ptr("mc2"),
                              ids=ptr("ti"), wts=ptr("tw"), estride=2 * d.MI * d.H, M=d.MI, K=d.H, rpt=rpt, tpe=tpe, R=d.TOPK, eps=d.eps,
                              mode=(topk_mode if fold_topk else 0) | op_gemv.mode_spt(spt), E=d.E, logits=ptr("rlog"), nb=1)
            prev = add(f"moe_up_{L}", up_export, "moe_up", L, blob, groups * tpe, (groups * tpe,),
                       prev, "i->(0)", f"E_up_{L}", "i->(0)", (1,), groups * tpe, d.MI, d.H)
            tpe, rpt = sz.down
            dn_export = "dsl_moe_down_fold" if fold_topk else "dsl_moe_down"
            blob = gemv_block(dn_export, tpe, W=W("w2"), x=ptr("mc2"), out=ptr("moe_out"), ids=ptr("ti"), wts=ptr("tw"), rows=xblock(L, 1),
                              estride=d.H * d.MI, M=d.H, K=d.MI, rpt=rpt, tpe=tpe, R=d.TOPK, eps=d.eps,
                              mode=(topk_mode | op_gemv.MODE_ROUTE_READY if fold_topk else 0) | op_gemv.mode_spt(slots) | op_gemv.MODE_SUM_SLOTS | xmode, E=d.E, logits=ptr("rlog"), nb=1)
            # expert weights depend on the routing only: with the top-k folded in, the stream may start once the router is done
            before_x = prev
            prev = add(f"moe_down_{L}", dn_export, "moe_down", L, blob, tpe, (tpe,), prev, "i->(0)",
                       f"E_dn_{L}", "i->(0)", (1,), tpe, d.H, d.MI, after=f"E_rt_{L}" if fold_topk else None, exchange=True)
        else:
            # ---- dense SwiGLU: gate+up with the post-attention norm fold, then down
            spt, tpe, rpt = sz.up
            blob = gemv_block("dsl_moe_up", tpe, W=W("wgu"), x=ptr("o_norm"), out=ptr("mc2"), estride=0, M=d.INTER, K=d.H, rpt=rpt, tpe=tpe,
                              rows=xblock(L, 0) or ptr("o"), resid_in=ptr("resid"), resid_out=ptr("resid2"), ln=W("ln2"), R=ranks, eps=d.eps,
                              mode=op_gemv.MODE_NORM | xmode, nb=1)
            prev = add(f"gate_up_{L}", "dsl_moe_up", "gate_up", L, blob, tpe, (tpe,), fold_in, "i->(0)", f"E_up_{L}", "i->(0)", (1,), tpe, d.INTER, d.H, after="")
            tpe, rpt = sz.down
            blob = gemv_block("dsl_moe_down", tpe, W=W("wd"), x=ptr("mc2"), out=ptr("moe_out"), estride=0, M=d.H, K=d.INTER, rpt=rpt, tpe=tpe,
                              eps=d.eps, nb=1, rows=xblock(L, 1), mode=xmode)
            before_x = prev
            prev = add(f"down_{L}", "dsl_moe_down", "down", L, blob, tpe, (tpe,), prev, "i->(0)", f"E_dn_{L}", "i->(0)", (1,), tpe, d.H, d.INTER, after="", exchange=True)
    # ---- lm_head with the final-norm fold, then greedy sampling
    t, rpt = sz.lm
    # (a sharded lm_head: this rank's d.VL rows -- of the whole embedding when the weights are tied -- and its logits only)
    blob = gemv_block("dsl_gemv_fold", t, W=ptr("embed") + (rank * d.VL * d.H * 2 if d.VL else 0) if d.tie else ptr("lm_head"), x=ptr("hn"),
                      out=ptr("logits"), M=d.lm_rows, K=d.H, rpt=rpt,
                      tpe=1, rows=xblock(d.L - 1, 1) or ptr("moe_out"), resid_in=ptr("resid2"), resid_out=ptr("resid"), ln=ptr("final_norm"), R=ranks, eps=d.eps,
                      ids=0, mode=op_gemv.MODE_NORM | xmode, nb=1)
    prev = add("lm_head", "dsl_gemv_fold", "lm_head", -1, blob, t, (t,), (before_x if exch else prev), "i->(0)", "E_lm", "i->(0)", (1,), t, d.lm_rows, d.H, after="")
    g.etensor("E_argmax", (1,), wait_count=1)
    g.call_device("argmax", (1,), tile("vl_argmax"), resource=res, args=["vl"], consts=(0,), in_edges={prev: "i->(0)"},
                  out_edges={"E_argmax": "i->i"}, duration_us=8.5)
    return g, pool, sz


def plan_rows_text(d: Dims, pool: ArgPool, sz: Sizing, maxlen: int) -> str:
    """The plan listing the reference writes as vl_plan.txt (model.py:688-704): one row per grid instance."""
    lines = [f"# vl plan {d.name}: instance export layer role offset tasks M K; total {len(pool.bytes())} bytes",
             f"total {len(pool.bytes())} parts {sz.parts} maxlen {maxlen} requests 1"]
    lines += [f"{n} {ex} {layer} {role} {off} {tasks} {M} {K}" for n, (_, ex, role, layer, off, tasks, M, K) in enumerate(pool.rows)]
    return "\n".join(lines) + "\n"


# ---- module protocol of an ETX program (etx/contracts/compiler.py:33-39) for the default model, pointers unset
def build() -> Graph:
    import os
    d = load_dims(os.environ.get("ETX_LLM_CONFIG", "qwen3-30b-a3b"), layers=int(os.environ.get("ETX_LLM_LAYERS", "0")) or None)
    return build_graph(d, lambda name: 0, int(os.environ.get("ETX_VL_MAXLEN", "1072")))[0]


def bindings(**overrides) -> dict:
    return {"POOL": 0, **overrides}


def runtime(bindings, rng=None):
    return {}
