"""Host side of the DeepSeek-V2 (latent attention + shared-expert MoE) program: dims, rotary table, weight packing, graph."""
import os
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200.models import dsv2 as M  # noqa: E402
from etx_megakernel_b200.passes import compile_graph, verify_plan  # noqa: E402
from etx_megakernel_b200.sim.protocol import simulate  # noqa: E402
from oracle import ref_mla as R  # noqa: E402


def oracle_dims(d: M.MlaDims, dense: bool = False) -> R.MlaDims:
    return R.MlaDims(hidden=d.H, heads=d.NH, kv_lora=d.C, qk_nope=d.DN, qk_rope=d.DR, v_head=d.DV, moe_inter=d.MI, n_routed=d.E, top_k=d.TOPK,
                     n_shared=d.NS, dense_inter=d.DENSE_INTER if dense else 0, eps=d.eps, theta=d.theta, rope_factor=d.rope_factor,
                     rope_original_max=d.rope_original_max, beta_fast=d.beta_fast, beta_slow=d.beta_slow, mscale=d.mscale,
                     mscale_all_dim=d.mscale_all_dim, routed_scaling=d.routed_scaling, norm_topk=d.norm_topk)


def test_dims_scale_and_rotary_table_equal_the_oracles():
    d = M.load_dims("deepseek-v2-lite")
    od = oracle_dims(d)
    assert (d.L, d.NQKV, d.ROW, d.SLOTS, d.DENSE_LAYERS) == (27, 16 * 192 + 576, 576, 8, 1)
    assert d.scale == float(np.float32(od.scale))
    cos, sin = R.yarn_tables(od, 300)
    t = M.yarn_table(d, 300)
    assert t.dtype == np.float32 and np.array_equal(t[:, :64], cos.astype(np.float32)) and np.array_equal(t[:, 64:], sin.astype(np.float32))
    sb = M.step_bytes(d, 1025)
    assert sb["moe_layer"] == R.layer_bytes(od, 1025) and sb["dense_layer"] == R.layer_bytes(oracle_dims(d, dense=True), 1025)
    with pytest.raises(ValueError, match="routed_scaling"):
        M.load_dims(dict(M.CONFIGS["deepseek-v2-lite"], routed_scaling_factor=16.0))


def test_packing_stores_the_shared_experts_after_the_routed_ones():
    d = M.MlaDims(name="t", H=256, NH=2, C=128, DN=64, DR=32, DV=64, MI=128, E=4, TOPK=2, NS=2, DENSE_LAYERS=1, DENSE_INTER=384, L=2, V=512)
    lw = R.synthetic_layer(oracle_dims(d), seed=3)
    p = M.pack_layer(d, 1, lw)
    shapes = M.weight_shapes(d, 64)
    for k, v in p.items():
        assert tuple(v.shape) == shapes[k][0], k
    w13, w2 = p["1.w13"], p["1.w2"]
    assert np.array_equal(w13[1, :128], lw.mlp["egate"][1]) and np.array_equal(w13[1, 128:], lw.mlp["eup"][1])
    assert np.array_equal(w13[4, :128], lw.mlp["sgate"][:128]) and np.array_equal(w13[5, 128:], lw.mlp["sup"][128:])
    assert np.array_equal(w2[5], lw.mlp["sdown"][:, 128:]) and np.array_equal(w2[2], lw.mlp["edown"][2])
    assert np.array_equal(p["1.wqa"][:2 * 96], lw.q_proj) and np.array_equal(p["1.wqa"][2 * 96:], lw.kv_a_proj_with_mqa)
    dl = R.synthetic_layer(oracle_dims(d, dense=True), seed=4)
    p0 = M.pack_layer(d, 0, dl)
    assert np.array_equal(p0["0.wgu"][384:], dl.mlp["up"]) and tuple(p0["0.wd"].shape) == (256, 384)


def test_the_full_size_graph_verifies_and_simulates():
    d = M.load_dims("deepseek-v2-lite", layers=3)
    addr = {}

    def ptr(name):
        return addr.setdefault(name, 0x10000000 + 0x1000000 * len(addr))
    g, pool, info = M.build_graph(d, ptr, 1072)
    names = [gr.name for gr in g.grids]
    assert names[:6] == ["prologue", "qkv_0", "attn_0", "o_proj_0", "gate_up_0", "down_0"]
    assert names[6:12] == ["qkv_1", "attn_1", "o_proj_1", "router_1", "moe_up_1", "moe_down_1"] and names[-2:] == ["lm_head", "argmax"]
    plan = compile_graph(g, "b200", {"POOL": len(pool.bytes())})
    assert verify_plan(plan) == [] and not simulate(plan).deadlock
    shape = plan.inst.grid_shapes
    assert shape["attn_1"] == (16 * (9 + 4),) and shape["moe_up_1"][0] <= 148 and shape["moe_down_1"][0] <= 148
    rows = {r[0]: r for r in pool.rows}
    blk = pool.bytes()[rows["moe_up_1"][4]: rows["moe_up_1"][4] + 160]
    import struct
    mode, E = struct.unpack_from("<i", blk, 104)[0], struct.unpack_from("<i", blk, 108)[0]
    assert (mode & 0xff) == 2 and (mode >> 24) & 0xf == 2 and E == 64 and struct.unpack_from("<i", blk, 96)[0] == 8       # no renorm, 2 shared, 8 slots
    with pytest.raises(ValueError, match="mla_attn"):
        M.build_graph(M.MlaDims(name="x", H=256, NH=2, C=1024, DN=64, DR=32, DV=64, MI=128, E=4, TOPK=2, NS=0, DENSE_LAYERS=0, DENSE_INTER=0, L=1, V=512), ptr, 64)


def test_latent_attention_block_layout_and_checks():
    """The 128-byte block: field offsets, the grid of (partitions + finishing tasks) x heads, and the refusals of the
    packer (shape outside the tile's shared-memory layout, a grid that does not match max_parts)."""
    import struct
    from etx_megakernel_b200 import ops
    from etx_megakernel_b200.importer import argblock
    from etx_megakernel_b200.ops import mla as op_mla
    ent = ops.all_entries()["mla_attn"]
    kw = dict(qkv=0x1000, kvln=0x2000, cos_sin=0x3000, wkvb=0x4000, cache=0x5000, positions=0x6000, out=0x7000, NH=16, C=512, DN=128, DR=64, DV=128,
              maxlen=1072, scale=0.125, eps=1e-6, tmp=0x8000, max_parts=9, tag=5)
    blob = argblock.pack_named(ent, (16 * (9 + op_mla.FINISHERS), 1, 1), **kw)
    assert len(blob) == op_mla.ARG_BYTES == 128
    assert struct.unpack_from("<7Q", blob, 0) == (0x1000, 0x2000, 0x3000, 0x4000, 0x5000, 0x6000, 0x7000)
    assert struct.unpack_from("<6i", blob, 56) == (16, 512, 128, 64, 128, 1072)
    assert struct.unpack_from("<Q2i", blob, 88) == (0x8000, 9, 5)
    assert struct.unpack_from("<4I", blob, 112) == (16 * 13, 1, 1, 16 * 13)
    assert op_mla.partitions(1072) == 9 and op_mla.tmp_pairs(16, 512, 1072) == 16 * 9 * 520
    with pytest.raises(ValueError, match="max_parts"):
        argblock.pack_named(ent, (16 * 9, 1, 1), **kw)                               # the finishing tasks are missing from the grid
    with pytest.raises(ValueError, match="max_parts"):
        argblock.pack_named(ent, (16 * 12, 1, 1), **dict(kw, max_parts=8))           # 8 partitions do not cover 1072 positions
    with pytest.raises(ValueError, match="multiples of 8"):
        argblock.pack_named(ent, (16 * 13, 1, 1), **dict(kw, DR=60))
    with pytest.raises(ValueError, match="context"):
        argblock.pack_named(ent, (16 * 13, 1, 1), **dict(kw, maxlen=9000, max_parts=71))


def test_split_k_keeps_one_wave_and_whole_slices():
    """The K-split of the dense tensor-core grids: tasks stay within one wave of the workers, slices are multiples of 64
    columns and at least 256 wide, a matrix with a wave of row blocks of its own is not split."""
    from etx_megakernel_b200.ops import batch as op_batch
    for M, K in ((5120, 2048), (2048, 4096), (128, 2048), (151936, 2048), (3648, 2048), (64, 2048), (2048, 1408), (102400, 2048)):
        tasks, rpt, S = op_batch.split_k(M, K, 148)
        blocks = -(-M // rpt)
        assert tasks == blocks * S and (tasks <= 148 or S == 1) and rpt % 128 == 0
        assert K % (64 * S) == 0 and (S == 1 or K // S >= 256) and S in (1, 2, 4, 8)
        if blocks * 2 <= 148 and K % 128 == 0 and K // 2 >= 256:
            assert S >= 2
