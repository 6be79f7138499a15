"""Operator specifications of the bf16 decode path on B200.

Mirrors the reference's operator table (etx/importer/spec.py:213-233 `Operator`, 236-253 `ARGUMENTS`, 257-369
`OPERATORS`, 372-406 `grid_for` / `validate_values`).  There the table describes vLLM kernels imported as tiles; here it
describes the built-in sm_100a tiles, one entry per export, with the same fields: grid rule, supported shapes,
constants, reads / writes, layouts, checks on the packed values, and the per-role argument recipe a host follows to
fill the block (expressions over the model dims and the session's buffer names).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from ..ops import attn as _attn
from ..ops import attnprep as _prep
from ..ops import gemv as _gemv
from ..ops import topk as _topk


@dataclass(frozen=True)
class Operator:
    name: str
    template: str
    grid_rule: tuple
    supported_shapes: str
    constants: dict
    reads: tuple
    writes: tuple
    aliases: tuple = ()
    layouts: str = "contiguous row-major tensors"
    dtypes: str = "bf16 tensors, fp32 reductions, int32 indices, int64 positions"
    checks: tuple = ()               # (parameter index, name, expression over p<i>, gx, gy, gz)
    arguments: dict = field(default_factory=dict)
    block_rule: tuple = (("544", "544"), ("1", "1"), ("1", "1"))

    def grid(self, **context):
        return tuple(int(eval(v, {"__builtins__": {}}, context)) for v in self.grid_rule)


# role -> [(type, expression)] in parameter order; names are the model dims (H, NH, NKV, HD, NQKV, E, TOPK, MI, V,
# eps) and the session's buffers (examples/vllm_llm/host.hip:274-317 naming: resid, resid2, hn, qkv, attn_out, o,
# o_norm, rlog, tw, ti, tei, mc2, mc3, logits; W("<layer>.<name>") = packed weight).
def _gemv_recipe(**kw):
    base = dict(W="nullptr", x="nullptr", out="nullptr", ids="nullptr", wts="nullptr", estride="0", M="0", K="0", rpt="rpt", tpe="1",
                rows="nullptr", resid_in="nullptr", resid_out="nullptr", ln="nullptr", R="0", eps="eps", mode="0", E="0",
                logits="nullptr", nb="1", sx="0", sout="0", srows="0", srin="0", srout="0")
    base.update(kw)
    ty = {"ptr addrspace(1)": "ptr", "i64": "i64", "i32": "i32", "float": "f32"}
    return [(ty[t], base[n]) for n, t, _, _ in _gemv.PARAMS]


ARGUMENTS = {
    "qkv": _gemv_recipe(W='W(pl + "wqkv")', x="hn", out="qkv", M="NQKV", K="H", rows="mc3 (layer > 0)", resid_in="resid2 | resid",
                        resid_out="resid", ln='W(pl + "ln1")', R="TOPK | 1 | 0", ids="ti", mode="1"),
    "o_proj": _gemv_recipe(W='W(pl + "wo")', x="attn_out", out="o", M="H", K="NH * HD"),
    "router": _gemv_recipe(W='W(pl + "wr")', x="o_norm", out="rlog", M="E", K="H", rows="o", resid_in="resid", resid_out="resid2",
                           ln='W(pl + "ln2")', R="1", mode="1"),
    "moe_up": _gemv_recipe(W='W(pl + "w13")', x="o_norm", out="mc2", ids="ti", wts="tw", estride="2 * MI * H", M="MI", K="H", tpe="tpe",
                           R="TOPK", mode="3 | 0x100", E="E", logits="rlog"),
    "moe_down": _gemv_recipe(W='W(pl + "w2")', x="mc2", out="mc3", ids="ti", wts="tw", estride="H * MI", M="H", K="MI", tpe="tpe"),
    "gate_up": _gemv_recipe(W='W(pl + "wgu")', x="o_norm", out="act", estride="0", M="INTER", K="H", tpe="tpe"),
    "down": _gemv_recipe(W='W(pl + "wd")', x="act", out="dn", M="H", K="INTER", tpe="tpe"),
    "lm_head": _gemv_recipe(W='W("lm_head")', x="hn", out="logits", M="V", K="H", rows="mc3 | dn", resid_in="resid2", resid_out="resid",
                            ln='W("final_norm")', R="TOPK | 1", ids="ti", mode="1"),
    "topk": [("ptr", "rlog"), ("ptr", "tw"), ("ptr", "ti"), ("ptr", "tei"), ("i32", "E"), ("i32", "TOPK"), ("i32", "norm_topk | 0x100"), ("i32", "0")],
    "prep": [("ptr", "qkv"), ("ptr", 'W(pl + "qn")'), ("ptr", 'W(pl + "kn")'), ("ptr", 'W("cos_sin")'), ("ptr", "positions"),
             ("ptr", "kc[layer]"), ("ptr", "vc[layer]"), ("ptr", "slot_mapping"), ("i32", "NH"), ("i32", "NKV"), ("i32", "HD"),
             ("f32", "eps"), ("i32", "BS"), ("i32", "X")],
    "attn": [("ptr", "qkv"), ("ptr", "kc[layer]"), ("ptr", "vc[layer]"), ("ptr", "block_tables"), ("ptr", "seq_lens"), ("ptr", "exp_sums"),
             ("ptr", "max_logits"), ("ptr", "tmp_out"), ("ptr", "attn_out"), ("f32", "scale"), ("i32", "NH"), ("i32", "NKV"), ("i32", "HD"),
             ("i32", "BS"), ("i32", "X"), ("i32", "parts"), ("i32", "MAXBLK")],
}
ARGUMENTS["reduce"] = ARGUMENTS["attn"]
ARGUMENTS["attn_fused"] = [("ptr", "qkv"), ("ptr", 'W(pl + "qn")'), ("ptr", 'W(pl + "kn")'), ("ptr", 'W("cos_sin")'), ("ptr", "kc[layer]"),
                           ("ptr", "vc[layer]"), ("ptr", "block_tables"), ("ptr", "seq_lens"), ("ptr", "positions"), ("ptr", "slot_mapping"),
                           ("ptr", "exp_sums"), ("ptr", "max_logits"), ("ptr", "tmp_out"), ("ptr", "attn_out"), ("ptr", "attn_counters + layer * NKV"),
                           ("f32", "scale"), ("f32", "eps"), ("i32", "NH"), ("i32", "NKV"), ("i32", "HD"), ("i32", "BS"), ("i32", "X"), ("i32", "parts")]

_I = {n: i for i, (n, *_rest) in enumerate(_gemv.PARAMS)}
_GEMV_CHECKS = ((_I["K"], "K % 8", "p%d - p%d %% 8" % (_I["K"], _I["K"])),)


def _gemv_op(name, form, grid, shape, reads, writes, roles):
    return Operator(name, f"etxb::tile_{form}", grid, shape, dict(THREADS=_gemv.THREADS, MAX_K=_gemv.MAX_K, NB=_gemv.NB_ALLOWED),
                    reads, writes, layouts="W row-major [M][K] (MoE: [E][...]), activations contiguous",
                    checks=_GEMV_CHECKS, arguments={r: ARGUMENTS[r] for r in roles})


OPERATORS = {
    "dsl_gemv": _gemv_op("dsl_gemv", "gemv", ("CU", "1", "1"), "K % 8 == 0, K <= 12288; stand-alone nb in (2,4,8) with nb*K <= 40960", ("weights", "input", "bias"),
                         ("output",), ("o_proj",)),
    "dsl_gemv_fold": _gemv_op("dsl_gemv_fold", "gemv", ("CU", "1", "1"), "as dsl_gemv; norm fold over R <= 16 rows", ("weights", "rows", "residual", "norm_weight", "expert_ids"),
                              ("output", "residual_out", "normed"), ("qkv", "router", "lm_head")),
    "dsl_moe_up": _gemv_op("dsl_moe_up", "moe_up", ("TOPK*tpe", "1", "1"), "K <= 12288, rpt <= 1024", ("weights", "input", "expert_ids"), ("activation",), ("gate_up",)),
    "dsl_moe_up_fold": _gemv_op("dsl_moe_up_fold", "moe_up", ("TOPK*tpe", "1", "1"), "as dsl_moe_up; E <= 256, TOPK <= 16", ("weights", "input", "logits"),
                                ("activation", "expert_ids", "routing_weights"), ("moe_up",)),
    "dsl_moe_down": _gemv_op("dsl_moe_down", "moe_down", ("TOPK*tpe", "1", "1"), "K <= 12288", ("weights", "activation", "expert_ids", "routing_weights"), ("expert_output",), ("moe_down", "down")),
    "dsl_moe_down_fold": _gemv_op("dsl_moe_down_fold", "moe_down", ("TOPK*tpe", "1", "1"), "as dsl_moe_down", ("weights", "activation", "logits"), ("expert_output",), ("moe_down",)),
    "dsl_topk": Operator("dsl_topk", "etxb::tile_topk", ("1", "1", "1"), "E <= 256, K <= 16, batch columns <= 16", dict(MAX_E=_topk.MAX_E, MAX_K=_topk.MAX_K),
                         ("logits",), ("routing_weights", "expert_ids", "token_expert_indices"),
                         checks=((4, "E", "min(max(p4, 1), 256)"), (5, "K", "min(max(p5, 1), 16)")), arguments={"topk": ARGUMENTS["topk"]}),
    "dsl_attnprep": Operator("dsl_attnprep", "etxb::tile_attnprep", ("NKV", "1", "1"), "G + 2 <= 16, HD % 32 == 0, HD <= 256, BS in (16, 32), X = 8",
                             dict(X=8), ("qkv", "q_weight", "k_weight", "cos_sin", "positions", "slot_mapping"), ("qkv", "key_cache", "value_cache"),
                             aliases=(("qkv", "output"),), layouts="key cache [block, head, HD/8, BS, 8], value cache [block, head, HD, BS]",
                             checks=((13, "X", "8"),), arguments={"prep": ARGUMENTS["prep"]}),
    "attn_decode": Operator("attn_decode", "etxb::tile_attn", ("parts*NKV", "1", "1"), "G <= 16, HD <= 256, PART = 32", dict(PART=_attn.PART, X=8),
                            ("query", "key_cache", "value_cache", "block_tables", "seq_lens"), ("exp_sums", "max_logits", "tmp_out"),
                            layouts="query row-major, key cache [block, head, HD/8, BS, 8], value cache [block, head, HD, BS]",
                            checks=((14, "X", "8"),), arguments={"attn": ARGUMENTS["attn"]}),
    "attn_fused": Operator("attn_fused", "etxb::tile_attn_fused", ("parts*NKV", "1", "1"), "G + 2 <= 16, G * HD <= 2048, G * parts <= 8192, PART = 32",
                           dict(PART=_attn.PART, X=8), ("qkv", "q_weight", "k_weight", "cos_sin", "key_cache", "value_cache", "block_tables", "seq_lens",
                                                       "positions", "slot_mapping"), ("key_cache", "value_cache", "exp_sums", "max_logits", "tmp_out", "output", "counters"),
                           layouts="key cache [block, head, HD/8, BS, 8], value cache [block, head, HD, BS]",
                           checks=((21, "X", "8"),), arguments={"attn_fused": ARGUMENTS["attn_fused"]}),
    "attn_reduce": Operator("attn_reduce", "etxb::tile_attn_reduce", ("NH", "1", "1"), "max_parts <= 4096", dict(PART=_attn.PART),
                            ("exp_sums", "max_logits", "tmp_out", "seq_lens"), ("output",), arguments={"reduce": ARGUMENTS["reduce"]}),
}


# ---- the tiles of a batched step (several sequences per launch; ops/batch.py)
from ..ops import batch as _batch  # noqa: E402

ARGUMENTS.update({
    "norm_col": _gemv_recipe(x="hn | o_norm", rows="mc3 | o", resid_in="resid2 | resid", resid_out="resid | resid2", ln='W(pl + "ln1" | "ln2")', ids="ti",
                             R="TOPK | 1 | 0", K="H", M="H", rpt="1", nb="B", sx="H", srows="TOPK * H | H", srin="H", srout="H"),
    "gemv_nb": _gemv_recipe(W='W(pl + "wqkv" | "wo" | "wr") | W("lm_head")', x="hn | attn_out | o_norm", out="qkv | o | rlog | logits", M="rows", K="H | NH * HD",
                            nb="B", sx="K", sout="M"),
    "moe_up_g": _gemv_recipe(W='W(pl + "w13")', x="o_norm", out="mc2", estride="2 * MI * H", M="MI", K="H", tpe="tpe", rows="elist", resid_in="ecount", nb="B",
                             R="TOPK", sx="H"),
    "moe_down_g": _gemv_recipe(W='W(pl + "w2")', x="mc2", out="mc3", wts="tw", estride="H * MI", M="H", K="MI", tpe="tpe", rows="elist", resid_in="ecount",
                               nb="B", R="TOPK"),
    "route": [("ptr", "rlog"), ("ptr", "tw"), ("ptr", "ti"), ("ptr", "ecount"), ("ptr", "elist"), ("ptr", "active + layer"), ("i32", "E"), ("i32", "TOPK"),
              ("i32", "norm_topk | 0x100"), ("i32", "B"), ("i32", "B")],
    "cols": [("i32", "B"), ("i32", "nblk * BS")],
})


def _batch_op(name, tile, grid, shape, reads, writes):
    recipe = {"gemv_tc": "gemv_nb", "moe_up_tc": "moe_up_g", "moe_down_tc": "moe_down_g"}.get(name, name)
    return Operator(name, f"etxb::{tile}", grid, shape, dict(NB_MAX=_batch.NB_MAX, XBYTES=_batch.XBYTES, GROUP_ROWS=_batch.GROUP_ROWS), reads, writes,
                    layouts="column b of a batched buffer at base + b * stride (element counts, the reference's sx / sout / srows / srin / srout)",
                    arguments={recipe: ARGUMENTS[recipe]})


OPERATORS.update({
    "norm_col": _batch_op("norm_col", "tile_norm_col", ("B", "1", "1"), "K <= 8192, R <= 64, B <= 64", ("rows", "residual", "norm_weight", "expert_ids"),
                          ("residual_out", "normed")),
    "gemv_nb": _batch_op("gemv_nb", "tile_gemv_nb", ("CU", "1", "1"), "K % 8 == 0, 2 K + 64 <= 40960, B <= 64", ("weights", "input", "bias"), ("output",)),
    "route": _batch_op("route", "tile_route", ("1", "1", "1"), "E <= 256, TOPK <= 16, B <= 64", ("logits",), ("routing_weights", "expert_ids", "expert_lists")),
    "moe_up_g": _batch_op("moe_up_g", "tile_moe_up_g", ("E*tpe", "1", "1"), "as gemv_nb", ("weights", "input", "expert_lists"), ("activation",)),
    "moe_down_g": _batch_op("moe_down_g", "tile_moe_down_g", ("E*tpe", "1", "1"), "as gemv_nb", ("weights", "activation", "expert_lists", "routing_weights"),
                            ("expert_output",)),
    "gemv_tc": _batch_op("gemv_tc", "tile_gemv_tc", ("CU", "1", "1"), "K % 64 == 0, B <= 64 (32 columns per pass)", ("weights", "input", "bias"), ("output",)),
    "moe_up_tc": _batch_op("moe_up_tc", "tile_moe_up_tc", ("E*tpe", "1", "1"), "as gemv_tc", ("weights", "input", "expert_lists"), ("activation",)),
    "moe_down_tc": _batch_op("moe_down_tc", "tile_moe_down_tc", ("E*tpe", "1", "1"), "as gemv_tc", ("weights", "activation", "expert_lists", "routing_weights"),
                             ("expert_output",)),
    "cols": _batch_op("cols", "tile_prologue_nb / tile_argmax", ("B", "1", "1"), "B <= 64", ("token_in", "embedding", "logits"), ("residual", "positions", "token_out")),
})


# ---- absorbed multi-head latent attention (ops/mla.py)
from ..ops import mla as _mla  # noqa: E402

ARGUMENTS["mla_attn"] = [("ptr", "qkv"), ("ptr", 'W(pl + "kvln")'), ("ptr", "cos_sin"), ("ptr", 'W(pl + "wkvb")'), ("ptr", "ckv + layer"), ("ptr", "positions"),
                         ("ptr", "attn_out"), ("i32", "NH"), ("i32", "C"), ("i32", "DN"), ("i32", "DR"), ("i32", "DV"), ("i32", "maxlen"), ("f32", "scale"), ("f32", "eps"), ("ptr", "mla_tmp"),
                         ("i32", "parts"), ("i32", "layer")]
OPERATORS["mla_attn"] = Operator("mla_attn", "etxb::tile_mla_attn", ("(parts+4)*NH", "1", "1"), "C <= 512, DR <= 64, DN + DR <= 256, context <= 8192", dict(MAX_CTX=_mla.MAX_CTX),
                                 ("qkv", "latent_norm_weight", "cos_sin", "kv_b_proj", "latent_cache", "positions"), ("latent_cache", "output"),
                                 layouts="latent cache [position][C + DR] (normed latent | rotated k_pe), kv_b_proj [head][DN rows of W_UK, DV rows of W_UV][C]",
                                 arguments={"mla_attn": ARGUMENTS["mla_attn"]})


def grid_for(export, dims, *, role, cu, parts, tpe=1):
    """The launch grid of `export` for a model (etx/importer/spec.py:372-389)."""
    spec = OPERATORS[export]
    return spec.grid(CU=cu, parts=parts, NKV=dims.NKV, NH=dims.NH, TOPK=max(getattr(dims, "TOPK", 0), 1), tpe=tpe)


def validate_values(export, values, grid):
    """Check arguments before Python packs the block (etx/importer/spec.py:392-406): the spec's scalar checks plus the
    shape limits of the CUDA tiles, so a block the kernel cannot run never reaches the device."""
    name = export.removeprefix("etx_tile_").removeprefix("etx_imp_")
    spec = OPERATORS.get(name)
    if spec is None:
        return
    gx, gy, gz = grid
    env = dict(gx=gx, gy=gy, gz=gz, min=min, max=max) | {f"p{i}": v for i, v in enumerate(values)}
    for index, label, expr in spec.checks:
        expected = eval(expr, {"__builtins__": {}}, env)
        if values[index] != expected:
            raise ValueError(f"{spec.name}: {label} conflicts: expected {expected}, got {values[index]}")
    if name in _gemv.FORMS:
        v = dict(zip((n for n, *_ in _gemv.PARAMS), values))
        _gemv.check_shape(name, M=v["M"], K=v["K"], rpt=v["rpt"], nb=v["nb"], mode=v["mode"])
        need = -(-v["M"] // v["rpt"]) * (1 if _gemv.FORMS[name] == "plain" else 1)
        if _gemv.FORMS[name] == "plain" and gx * gy * gz < need:
            raise ValueError(f"{spec.name}: grid of {gx * gy * gz} tasks leaves rows unwritten (needs {need})")
        if _gemv.FORMS[name] != "plain":
            if v["tpe"] < 1 or v["tpe"] * v["rpt"] < v["M"]:
                raise ValueError(f"{spec.name}: tpe * rpt = {v['tpe'] * v['rpt']} does not cover M = {v['M']}")
            spt = ((v["mode"] >> 16) & 0xff) or 1
            slots = max(v["R"], 1) if (v["mode"] & 0xff) >= 2 or v["ids"] else 1
            if slots % spt or gx * gy * gz != (slots // spt) * v["tpe"]:
                raise ValueError(f"{spec.name}: grid {gx * gy * gz} != (slots {slots} / {spt} per task) * tpe {v['tpe']}")
            if (v["mode"] & _gemv.MODE_SUM_SLOTS) and (name.startswith("dsl_moe_up") or spt != slots):
                raise ValueError(f"{spec.name}: the summed form is for moe_down with every slot in one task")
        if (v["mode"] & 0xff) >= 2:
            _topk.check_shape(v["E"], v["R"])
    elif name == "dsl_topk":
        _topk.check_shape(values[4], values[5])
    elif name == "dsl_attnprep":
        _prep.check_shape(values[8], values[9], values[10], values[12], values[13])
        if gx * gy * gz != values[9]:
            raise ValueError(f"{spec.name}: grid must be one task per kv head")
    elif name == "mla_attn":
        _mla.check_shape(*values[7:13])
        if values[16] != _mla.partitions(values[12]) or gx * gy * gz != values[7] * (values[16] + _mla.FINISHERS):
            raise ValueError(f"{spec.name}: max_parts must cover maxlen in partitions of {_mla.PART} and the grid is (max_parts + {_mla.FINISHERS}) * NH tasks")
    elif name == "attn_fused":
        _attn.check_fused(*values[17:25])
        whole = bool(values[23]) and bool(values[24] & _attn.GQ_WHOLE)
        if whole and not _attn.whole_sequence_fits(values[23], values[22]):
            raise ValueError(f"{spec.name}: whole-sequence form: 64 KB + max_parts * gq * 130 floats must fit the weight ring")
        want = (1 if whole else values[22]) * (values[17] // values[23] if values[23] else values[18])
        if gx * gy * gz != want:
            raise ValueError(f"{spec.name}: grid must be max_parts * NKV tasks (grouped form: max_parts * NH / gq; whole-sequence form: NH / gq)")
    elif name in ("attn_decode", "attn_reduce"):
        _attn.check_shape(values[10], values[11], values[12], values[13], values[14], values[15])
