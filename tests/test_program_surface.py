"""CPU tests of the program surface: edge maps, graph verification, machine model, argument blocks, operator specs,
plan compilation and the binary plan (the reference pins the same things in tests/test_edgemap.py, test_ir_verify.py,
test_machine.py, test_ops_gemv.py, test_operator_spec.py, test_passes.py and test_vllm_moe.py)."""
import struct

import numpy as np
import pytest

import etx_megakernel_b200 as P  # noqa: F401
from etx_megakernel_b200 import ops
from etx_megakernel_b200.frontends import cuda_link, hip_link
from etx_megakernel_b200.importer import argblock, spec
from etx_megakernel_b200.ir import EdgeMap, Graph, VerifyError, instantiate, verify
from etx_megakernel_b200.machine import list_archs, load_machine
from etx_megakernel_b200.models import qwen as Q
from etx_megakernel_b200.passes import PassOptions, compile_graph, verify_plan
from etx_megakernel_b200.passes.plan import MAGIC


# ------------------------------------------------------------------------------------------------ edge maps
def test_edge_map_forms():
    assert EdgeMap.parse("ij->i").targets((3, 1), (8,)) == [(3,)]
    assert EdgeMap.parse("h->bh").targets((2,), (3, 4)) == [(0, 2), (1, 2), (2, 2)]                 # broadcast letter
    assert EdgeMap.parse("ij->(i/2)j").targets((5, 1), (4, 2)) == [(2, 1)]
    assert EdgeMap.parse("i->(i%NKV)").targets((6,), (4,), bindings={"NKV": 4}) == [(2,)]
    rt = {"indptr": [0, 2, 5], "topk": [[1, 3], [0, 2]]}
    assert EdgeMap.parse("i->range(indptr[i], indptr[i+1])").targets((1,), (8,), rt) == [(2,), (3,), (4,)]
    assert EdgeMap.parse("i->topk[i,:]").targets((1,), (8,), rt) == [(0,), (2,)]
    assert EdgeMap.parse("*").targets((0,), (2, 2)) == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert EdgeMap.parse("i->()").targets((4,), ()) == [()]
    assert EdgeMap.parse("i->topk[i,:]").is_runtime and not EdgeMap.parse("i->i").is_runtime
    for bad in ("i", "i->(j)", "i->((i)", "1->i", "i->i+"):
        with pytest.raises(ValueError):
            EdgeMap.parse(bad)
    with pytest.raises(ValueError):
        EdgeMap.parse("ij->i").targets((0, 0), (2, 2))                                            # rank mismatch
    with pytest.raises(KeyError):
        EdgeMap.parse("i->topk[i,:]").targets((0,), (4,))                                          # runtime tensor missing


def _splitk(n=4, parts=4, wait=None):
    g = Graph("splitk_sum")
    g.tensor("A", ("n*32", 128)); g.tensor("B", ("n*32", parts), role="scratch", bytes_per_elem=4); g.tensor("C", ("n*32",), bytes_per_elem=4)
    g.etensor("E", ("n",), wait_count=parts if wait is None else wait)
    g.call_device("partial_sum", ("n", parts), hip_link("examples/tiles/splitk.hip", "etx_tile_partial_sum"), args=["A", "B"], reads=["A"],
                  writes=["B"], out_edges={"E": "ij->i"})
    g.call_device("final_sum", ("n",), hip_link("examples/tiles/splitk.hip", "etx_tile_final_sum"), args=["B", "C"], reads=["B"], writes=["C"],
                  in_edges={"E": "i->i"})
    return g


def test_verify_checks():
    assert verify(_splitk(), {"n": 4}) == []
    with pytest.raises(VerifyError, match="wait_count=3 but 4 producers"):                        # count conservation
        verify(_splitk(wait=3), {"n": 4})
    g = _splitk()
    g.grids.reverse()                                                                            # consumer before producer
    with pytest.raises(VerifyError, match="later grid"):
        verify(g, {"n": 4})
    g = _splitk()
    g.call_device("again", ("n",), cuda_link("", "nop"), writes=["C"])
    assert any(i.check == "coverage" for i in verify(g, {"n": 4}, strict=False))                  # two writers of C
    g = Graph("rt")
    g.etensor("E", (4,), wait_count=1)
    g.call_device("a", (2,), cuda_link("", "nop"), out_edges={"E": "i->topk[i,:]"})
    assert any(i.check == "runtime-first" for i in verify(g, {}, {"topk": [[0, 1], [2, 3]]}, strict=False))
    with pytest.raises(ValueError, match="pure=True"):
        Graph("p").call_device("x", (1,), cuda_link("", "nop"), reads=["q"], writes=["q"], pure=True)
    with pytest.raises(ValueError, match="consts"):
        Graph("p").call_device("x", (1,), cuda_link("", "nop"), consts=(1, 2, 3, 4, 5))


def test_instantiate_counts_and_symbols():
    g = _splitk()
    assert g.symbols == ["n"]
    inst = instantiate(g, {"n": 3})
    assert inst.n_tasks() == 3 * 4 + 3
    assert all(len(v) == 4 for k, v in inst.producers.items() if k[0] == "E")
    assert inst.task_in[("final_sum", (2,))] == [("E", (2,))]


# ------------------------------------------------------------------------------------------------ machine model
def test_machine_model_b200():
    assert {"b200", "sm_100"} <= set(list_archs())
    m = load_machine("b200")
    assert m.total_cus() == 148 and m.workers() == 148 and m.wave_size == 32 and not m.has_domain_level
    from etx_megakernel_b200.ir import Scope
    assert m.effective_scope(Scope.DOMAIN) == Scope.DEVICE and m.effective_scope(Scope.SYSTEM) == Scope.SYSTEM
    assert m.vis(Scope.DEVICE).poll.startswith("ld.acquire.gpu") and m.supports("tma") and not m.supports("tma_cluster_broadcast")
    assert m.gemv_tasks(5120) == (147, 35) and m.gemv_tasks(128) == (128, 1)
    assert m.hbm_bw_bytes_per_us() == 8.0e6
    with pytest.raises(FileNotFoundError):
        load_machine("gfx942")


# ------------------------------------------------------------------------------------------------ argument blocks
def test_gemv_block_layout_matches_reference():
    """25 parameters, 160 bytes, grid words at 144, the reference's type string (tests/test_ops_gemv.py)."""
    e = ops.gemv.import_entries()["dsl_gemv"]
    assert ops.gemv.type_string() == "pppppliiiippppifiipiiiiii"
    assert (e["arg_bytes"], e["grid_offset"], len(e["params"])) == (160, 144, 25)
    assert [p["offset"] for p in e["params"]][:10] == [0, 8, 16, 24, 32, 40, 48, 52, 56, 60]
    b = argblock.pack_named(e, (147, 1, 1), W=0x1000, x=0x2000, out=0x3000, M=5120, K=2048, rpt=35, eps=1e-6, nb=1)
    assert len(b) == 160 and struct.unpack_from("<QQQ", b, 0) == (0x1000, 0x2000, 0x3000)
    assert struct.unpack_from("<ii", b, 48) == (5120, 2048) and struct.unpack_from("<IIII", b, 144) == (147, 1, 1, 147)
    assert abs(struct.unpack_from("<f", b, 100)[0] - 1e-6) < 1e-12
    t = ops.topk.import_entries()["dsl_topk"]; a = ops.attnprep.import_entries()["dsl_attnprep"]
    assert (t["arg_bytes"], t["grid_offset"]) == (64, 48) and (a["arg_bytes"], a["grid_offset"]) == (112, 96)
    assert set(ops.all_entries()) >= {"dsl_gemv", "dsl_gemv_fold", "dsl_moe_up", "dsl_moe_up_fold", "dsl_moe_down", "dsl_moe_down_fold",
                                      "dsl_topk", "dsl_attnprep", "attn_decode", "attn_reduce", "attn_fused"}


def test_pack_rejects_bad_blocks():
    e = ops.all_entries()
    with pytest.raises(ValueError, match="values for"):
        argblock.pack(e["dsl_topk"], [1, 2, 3], (1, 1, 1))
    with pytest.raises(TypeError):
        argblock.pack_named(e["dsl_topk"], (1, 1, 1), logits=1.5, E=8, K=2)
    with pytest.raises(KeyError):
        argblock.pack_named(e["dsl_topk"], (1, 1, 1), nonsense=1)
    with pytest.raises(ValueError):
        argblock.pack_named(e["dsl_topk"], (1, 1, 1), logits=1, wts=2, ids=3, E=512, K=8)        # E > 256
    with pytest.raises(ValueError):
        argblock.pack_named(e["dsl_attnprep"], (4, 1, 1), qkv=1, NH=32, NKV=4, HD=128, BS=16, X=4)  # X must be 8
    with pytest.raises(ValueError):
        argblock.pack_named(e["dsl_gemv"], (4, 1, 1), W=1, x=2, out=3, M=64, K=16384, rpt=16, nb=1)  # K > 12288
    with pytest.raises(ValueError, match="grid"):                                                # up grid != groups * tpe
        argblock.pack_named(e["dsl_moe_up"], (10, 1, 1), W=1, x=2, out=3, ids=4, M=768, K=2048, rpt=21, tpe=37, R=8, nb=1)
    with pytest.raises(ValueError, match="summed"):
        argblock.pack_named(e["dsl_moe_down"], (74, 1, 1), W=1, x=2, out=3, ids=4, M=2048, K=768, rpt=56, tpe=37, R=8, nb=1,
                            mode=0x400 | (4 << 16))


def test_operator_table():
    assert set(spec.OPERATORS) == set(ops.all_entries())
    d = Q.load_dims("qwen3-30b-a3b")
    assert spec.grid_for("dsl_gemv", d, role="qkv", cu=147, parts=34) == (147, 1, 1)
    assert spec.grid_for("attn_fused", d, role="attn_fused", cu=148, parts=34) == (34 * 4, 1, 1)
    assert spec.grid_for("dsl_attnprep", d, role="prep", cu=148, parts=34) == (4, 1, 1)
    assert spec.grid_for("attn_reduce", d, role="reduce", cu=148, parts=34) == (32, 1, 1)
    for op in spec.OPERATORS.values():
        for recipe in op.arguments.values():
            assert all(t in ("ptr", "i32", "i64", "f32") for t, _ in recipe)
    assert len(spec.ARGUMENTS["qkv"]) == 25 and len(spec.ARGUMENTS["topk"]) == 8 and len(spec.ARGUMENTS["prep"]) == 14
