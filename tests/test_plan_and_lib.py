"""CPU tests of the plan (task enumeration, event counts, static queues, binary blob), of the decode graph builder and
of the C-ABI library's symbol table (no compute call is made: there is no GPU here)."""
import re
import struct
from pathlib import Path

import numpy as np
import pytest

import etx_megakernel_b200 as P
from etx_megakernel_b200.frontends import cuda_link
from etx_megakernel_b200.ir import Graph
from etx_megakernel_b200.models import qwen as Q
from etx_megakernel_b200.passes import PassOptions, compile_graph, verify_plan
from etx_megakernel_b200.passes.plan import MAGIC, TILE_SYMBOLS
from etx_megakernel_b200.runtime import lib

ROOT = Path(__file__).resolve().parents[1]


def _fake_ptr(name):
    return 0x7F0000000000 + (hash(name) % 4096) * 4096


def test_qwen3_moe_graph_phases_and_counts():
    """Launch order and grid sizes of the MoE decode step (the reference pins its own in tests/test_vllm_moe.py:58-66)."""
    d = Q.load_dims("qwen3-30b-a3b", layers=2)
    assert (d.H, d.NH, d.NKV, d.HD, d.NQKV, d.E, d.TOPK, d.MI, d.V, d.qk_norm, d.norm_topk) == (2048, 32, 4, 128, 5120, 128, 8, 768, 151936, True, True)
    g, pool, sz = Q.build_graph(d, _fake_ptr, 1072)
    names = [gr.name for gr in g.grids]
    assert names == ["prologue", "qkv_0", "attn_0", "o_proj_0", "router_0", "moe_up_0", "moe_down_0",
                     "qkv_1", "attn_1", "o_proj_1", "router_1", "moe_up_1", "moe_down_1", "lm_head", "argmax"]
    plan = compile_graph(g, "b200", {"POOL": len(pool.bytes())})
    shape = {n: plan.inst.grid_shapes[n] for n in names}
    assert shape["qkv_0"] == (147,) and shape["attn_0"] == (9 * 16,) and shape["o_proj_0"] == (147,) and shape["router_0"] == (128,)
    assert shape["moe_up_0"] == (148,) and shape["moe_down_0"] == (147,) and shape["lm_head"] == (148,)
    assert all(m == "static" for m in plan.modes.values())
    assert plan.events["E_up_0"].counts == [148] and plan.events["E_red_0"].counts == [144] and sz.attn == (2, 128, 9)
    assert verify_plan(plan) == []
    assert sz.up == (2, 37, 21)                            # two expert slots per task, 37 row chunks of 21 rows: 148 tasks
    # the unfused structure keeps the reference's phases
    g2, pool2, _ = Q.build_graph(d, _fake_ptr, 1072, fused_attn=False, fold_topk=False)
    assert [gr.name for gr in g2.grids][1:8] == ["qkv_0", "prep_0", "attn_0", "reduce_0", "o_proj_0", "router_0", "topk_0"]
    text = Q.plan_rows_text(d, pool, sz, 1072)
    assert text.splitlines()[1].startswith("total ") and " parts 34 maxlen 1072" in text


def test_dense_graph_and_config_refusals():
    d = Q.load_dims("qwen3-8b", layers=1)
    g, pool, _ = Q.build_graph(d, _fake_ptr, 1072)
    assert [gr.name for gr in g.grids] == ["prologue", "qkv_0", "attn_0", "o_proj_0", "gate_up_0", "down_0", "lm_head", "argmax"]
    compile_graph(g, "b200", {"POOL": len(pool.bytes())})
    with pytest.raises(ValueError, match="refusing to plan it as dense"):
        Q.load_dims({"hidden_size": 64, "num_attention_heads": 2, "num_hidden_layers": 1, "vocab_size": 8, "expert_capacity": 3})
    with pytest.raises(ValueError, match="shared experts"):
        Q.load_dims(dict(Q.CONFIGS["qwen3-30b-a3b"], n_shared_experts=2))
    with pytest.raises(ValueError, match="rope type"):
        Q.load_dims(dict(Q.CONFIGS["qwen3-8b"], rope_scaling={"rope_type": "yarn"}))


def test_blob_layout_and_stream_words():
    d = Q.load_dims("qwen3-30b-a3b", layers=1)
    g, pool, _ = Q.build_graph(d, _fake_ptr, 128)
    pb = pool.bytes()
    plan = compile_graph(g, "b200", {"POOL": len(pb)})
    blob = plan.to_blob([("impargs", len(pb)), ("vl", 8)], pb)
    magic, version, workers, ntasks, ntypes, nev, nin, nout, ntens, poolb = struct.unpack_from("<Q9I", blob, 0)
    assert (magic, version, workers, ntasks, ntypes, ntens, poolb) == (MAGIC, 1, 148, len(plan.tasks), len(g.grids), 2, len(pb))
    assert nev == plan.event_words and nout == sum(len(w) for w in plan.task_out_words)
    off = 64 + 2 * 64
    types = np.frombuffer(blob, "<i4", count=ntypes * 12, offset=off).reshape(ntypes, 12)
    by_name = {gr.name: types[plan.type_ids[gr.name]] for gr in g.grids}
    assert by_name["qkv_0"][0] == TILE_SYMBOLS["etx_tile_dsl_gemv_fold"] and by_name["qkv_0"][10] == -1      # static weights: stream ahead
    assert by_name["moe_up_0"][10] == -2                                                                    # waits for its own in-event
    assert by_name["moe_down_0"][10] == plan.events["E_rt_0"].offset                                        # expert weights: after the router
    assert by_name["attn_0"][0] == 12 and by_name["prologue"][5] == 1                                       # args: tensor 1 ("vl")
    with pytest.raises(ValueError, match="argument pool"):
        plan.to_blob([("impargs", 5)], pb)
    with pytest.raises(ValueError, match="does not bind"):
        plan.to_blob([("impargs", len(pb))], pb)


def test_plan_rejects_deadlock_and_oversubscription():
    g = Graph("two")
    g.tensor("impargs", (16,), role="weight", bytes_per_elem=1)
    g.etensor("E0", (1,), wait_count=1)
    g.call_device("a", (1,), cuda_link("", "nop"), args=["impargs"], out_edges={"E0": "i->i"})
    g.call_device("b", (1,), cuda_link("", "nop"), args=["impargs"], in_edges={"E0": "i->i"})
    plan = compile_graph(g, "b200", {})
    plan.static_queues[(0, 0)] = [1, 0]; plan.static_queues[(0, 1)] = []
    assert any("deadlock" in e for e in verify_plan(plan))
    with pytest.raises(ValueError, match="persistent CTAs"):
        compile_graph(g, "b200", {}, options=PassOptions(workers=149))
    with pytest.raises(ValueError, match="static scheduling"):
        compile_graph(g, "b200", {}, options=PassOptions(force_mode="dynamic"))
    g.call_device("c", (1,), cuda_link("", "no_such_tile"), args=["impargs"])
    with pytest.raises(ValueError, match="no built-in tile"):
        compile_graph(g, "b200", {}).to_blob([("impargs", 16)], bytes(16))
    j = compile_graph(g, "b200", {}).to_json()
    assert {"types", "events", "descs", "static_queues", "task_in"} <= set(j)


def test_library_exports_every_declared_symbol():
    """Every function include/etxb200.h declares resolves in the built library (built by __graft_entry__.build())."""
    header = (ROOT / "include" / "etxb200.h").read_text()
    declared = set(re.findall(r"\b(etxb_[a-z_0-9]+)\s*\(", header)) - {"etxb_session"}
    assert declared == set(lib.SYMBOLS)
    import __graft_entry__ as ge
    ge.build()
    handle = lib.load()
    for name in declared:
        assert hasattr(handle, name), name
    assert handle.etxb_version() == 0x00010000


def test_install_as_etx_alias():
    P.install_as_etx()
    from etx.frontends import hip_link                      # noqa: F401  (resolves to this package)
    from etx.importer import argblock, spec                 # noqa: F401
    from etx.ir import Graph as G2
    assert G2 is Graph


def test_weight_pack_round_trip():
    from oracle import ref_decode as O
    from tests.golden.cases import SMALL_MOE
    W = O.SyntheticWeights(SMALL_MOE, seed=1)
    d = Q.Dims(**{f: getattr(SMALL_MOE, f) for f in ("name", "H", "NH", "NKV", "HD", "INTER", "L", "V", "eps", "theta", "tie", "bias",
                                                     "qk_norm", "moe", "E", "TOPK", "MI", "norm_topk")})
    packed = Q.pack_hf(d, W.get, 64)
    assert {k: v.shape for k, v in packed.items()} == {k: tuple(s) for k, s in Q.weight_shapes(d, 64).items()}
    back = Q.unpack_layer_hf(d, packed.__getitem__, 1)
    for k, v in back.items():
        assert np.array_equal(v, W.get(k)), k
    cos, sin = O.rope_tables(d.theta, d.HD, 64)
    tab = (packed["cos_sin"].astype(np.uint32) << 16).view(np.float32)
    assert np.array_equal(tab[:, :d.HD // 2], cos) and np.array_equal(tab[:, d.HD // 2:], sin)


def test_batched_graph_phases_and_argument_blocks():
    """The batched step (several sequences per launch): phase order, one argument block per sequence for the attention grid
    (addressed by the grid's second coordinate), a valid plan; tensor-core engine: one routing task per column, expert grids
    of one share per worker, narrow dense grids cut along K; mma.sync engine: one routing task, E x chunks expert tasks."""
    from etx_megakernel_b200.models import batched as BT
    from etx_megakernel_b200.ops import attn as op_attn
    from etx_megakernel_b200.sim.protocol import simulate
    d = Q.load_dims("qwen3-30b-a3b", layers=2)
    B = 8
    g, pool, info = BT.build_graph(d, _fake_ptr, B, 1072)
    names = [gr.name for gr in g.grids]
    assert names[:11] == ["prologue", "norm1_0", "qkv_0", "attn_0", "o_proj_0", "norm2_0", "router_0", "route_0", "moe_up_0", "moe_down_0", "norm1_1"]
    assert names[-3:] == ["norm_f", "lm_head", "argmax"]
    plan = compile_graph(g, "b200", {"POOL": len(pool.bytes())})
    assert verify_plan(plan) == [] and not simulate(plan).deadlock
    shape = plan.inst.grid_shapes
    assert shape["attn_0"] == (info["attn_tasks"], B) and info["attn"] == (8, 128, 9) and shape["norm1_0"] == (B,) and shape["route_0"] == (B,)
    assert shape["moe_up_0"] == (148,) and shape["moe_down_0"] == (148,)
    assert shape["qkv_0"] == (80,) and shape["o_proj_0"] == (64,) and shape["router_0"] == (8,) and shape["lm_head"] == (132,)
    rows = {r[0]: r for r in pool.rows}
    pb = pool.bytes()
    q0, q1, o0 = (pb[rows[n][4]: rows[n][4] + 160] for n in ("qkv_0", "qkv_1", "o_proj_0"))
    assert struct.unpack_from("<2i", q0, 56) == (256, 4) and struct.unpack_from("<2i", o0, 56) == (256, 8)          # rows per task, K-split
    assert struct.unpack_from("<Q", q0, 72)[0] == struct.unpack_from("<Q", q1, 72)[0] == _fake_ptr("skc")            # layers share a shape's counters
    assert struct.unpack_from("<Q", o0, 72)[0] == _fake_ptr("skc") + 4 * 20 and struct.unpack_from("<Q", o0, 64)[0] == _fake_ptr("skp")
    g3, pool3, info3 = BT.build_graph(d, _fake_ptr, 32, 1072)              # enough sequences: one attention task per (sequence, kv head)
    shape3 = compile_graph(g3, "b200", {"POOL": len(pool3.bytes())}).inst.grid_shapes
    assert info3["attn_whole"] and not info["attn_whole"] and shape3["attn_0"] == (4, 32)
    blk3 = pool3.bytes()[{r[0]: r for r in pool3.rows}["attn_1"][4]:][:op_attn.F_ARG_BYTES]
    assert struct.unpack_from("<i", blk3, 156)[0] == 128 | (1 << 16) | op_attn.GQ_WHOLE
    g2, pool2, info2 = BT.build_graph(d, _fake_ptr, B, 1072, engine="mma")
    shape2 = compile_graph(g2, "b200", {"POOL": len(pool2.bytes())}).inst.grid_shapes
    assert shape2["route_0"] == (1,) and shape2["moe_up_0"] == (128 * 3,) and shape2["moe_down_0"] == (128 * 4,)
    off = rows["attn_1"][4]
    for b in range(B):                                       # block b of the attention grid: sequence b's q rows and partial buffers
        blk = pb[off + b * op_attn.F_ARG_BYTES: off + (b + 1) * op_attn.F_ARG_BYTES]
        assert struct.unpack_from("<Q", blk, 0)[0] == _fake_ptr("qkv") + b * d.NQKV * 2
        assert struct.unpack_from("<Q", blk, 104)[0] == _fake_ptr("attn_out") + b * d.NH * d.HD * 2
        assert struct.unpack_from("<4I", blk, 160) == (info["attn_tasks"], 1, 1, info["attn_tasks"])
    with pytest.raises(ValueError, match="MoE"):
        BT.build_graph(Q.load_dims("qwen3-8b", layers=1), _fake_ptr, 4, 1072)
