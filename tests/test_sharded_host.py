"""Host side of the sharded (tensor-parallel) decode step, on CPU: the weight split recombines to the whole model's
result, a rank's graph compiles and verifies as a single-device program with its exchanged grids flagged in the plan
blob, and two gloo ranks pass their region handles around."""
import os
import struct

import numpy as np
import pytest

import etx_megakernel_b200  # noqa: F401
from etx_megakernel_b200.models import qwen as Q
from etx_megakernel_b200.passes import compile_graph
from etx_megakernel_b200.passes.plan import verify_plan
from etx_megakernel_b200.sim.protocol import simulate
from oracle import ref_decode as O
from tests.golden.cases import SMALL_DENSE, SMALL_MOE

FIELDS = ("name", "H", "NH", "NKV", "HD", "INTER", "L", "V", "eps", "theta", "tie", "bias", "qk_norm", "moe", "E", "TOPK", "MI", "norm_topk")


def qdims(od):
    return Q.Dims(**{f: getattr(od, f) for f in FIELDS})


def f32(u):
    return (np.asarray(u).astype(np.uint32) << 16).view(np.float32)


@pytest.mark.parametrize("od", [SMALL_MOE, SMALL_DENSE])
def test_shards_recombine_to_the_whole_model(od):
    d = qdims(od)
    full = Q.pack_hf(d, O.SyntheticWeights(od, seed=3, gamma="ones").get, 64)
    ranks = 2
    sd = Q.shard_dims(d, ranks)
    shards = [Q.shard_weights(full, d, ranks, r) for r in range(ranks)]
    want = Q.weight_shapes(sd, 64)
    for s in shards:
        assert {k: tuple(v.shape) for k, v in s.items()} == {k: tuple(v) for k, v in want.items()}
    rng = np.random.default_rng(0)
    x = rng.standard_normal(d.H).astype(np.float32)
    # column-parallel qkv: the ranks' rows are a permutation of the whole model's rows
    qkv = f32(full["0.wqkv"]) @ x
    nq, nk = d.NH * d.HD, d.NKV * d.HD
    parts = [f32(s["0.wqkv"]) @ x for s in shards]
    ql, kl = nq // ranks, nk // ranks
    assert np.array_equal(np.concatenate([p[:ql] for p in parts]), qkv[:nq])
    assert np.array_equal(np.concatenate([p[ql:ql + kl] for p in parts]), qkv[nq:nq + nk])
    assert np.array_equal(np.concatenate([p[ql + kl:] for p in parts]), qkv[nq + nk:])
    # row-parallel o_proj: the ranks' partial rows add up to the whole row
    a = rng.standard_normal(nq).astype(np.float32)
    o = f32(full["0.wo"]).astype(np.float64) @ a
    o_parts = sum(f32(s["0.wo"]).astype(np.float64) @ a[r * ql:(r + 1) * ql] for r, s in enumerate(shards))
    assert np.allclose(o, o_parts, rtol=1e-12, atol=1e-12)
    # MLP / one expert: gate+up by rows, down by columns
    if d.moe:
        e = 5
        w13, w2 = f32(full["0.w13"])[e].astype(np.float64), f32(full["0.w2"])[e].astype(np.float64)
        s13 = [f32(s["0.w13"])[e].astype(np.float64) for s in shards]
        s2 = [f32(s["0.w2"])[e].astype(np.float64) for s in shards]
        mi = d.MI
    else:
        w13, w2 = f32(full["0.wgu"]).astype(np.float64), f32(full["0.wd"]).astype(np.float64)
        s13 = [f32(s["0.wgu"]).astype(np.float64) for s in shards]
        s2 = [f32(s["0.wd"]).astype(np.float64) for s in shards]
        mi = d.INTER

    def mlp(w13, w2, m):
        g, u = w13[:m] @ x, w13[m:] @ x
        return w2 @ (g / (1 + np.exp(-g)) * u)
    assert np.allclose(mlp(w13, w2, mi), sum(mlp(a13, a2, mi // ranks) for a13, a2 in zip(s13, s2)), rtol=1e-10, atol=1e-12)


def test_shard_dims_refuses_uneven_splits():
    d = qdims(SMALL_MOE)
    assert Q.shard_dims(d, 1) is d
    with pytest.raises(ValueError):
        Q.shard_dims(d, 3)                     # 8 q heads do not split 3 ways
    with pytest.raises(ValueError):
        Q.shard_dims(qdims(SMALL_DENSE), 8)    # 4 q heads do not split 8 ways


def test_more_ranks_than_kv_heads_replicates_the_kv_head():
    """Qwen3-30B-A3B has 4 kv heads: on 8 ranks every rank takes 4 q heads and the ONE kv head they attend to (each kv
    head lives on two ranks).  Checked on the small MoE model at 4 ranks (2 kv heads) value by value, and on the
    30B-A3B shape by its dimensions."""
    big = Q.shard_dims(Q.load_dims("qwen3-30b-a3b"), 8)
    assert (big.NH, big.NKV, big.MI, big.VL) == (4, 1, 96, 151936 // 8) and Q.kv_replication(Q.load_dims("qwen3-30b-a3b"), 8) == 2
    assert Q.kv_replication(Q.load_dims("qwen3-30b-a3b"), 4) == 1 and Q.kv_replication(Q.load_dims("qwen3-8b"), 8) == 1
    od = SMALL_MOE
    d = qdims(od)
    ranks = 4
    assert Q.kv_replication(d, ranks) == 2
    sd = Q.shard_dims(d, ranks)
    assert (sd.NH, sd.NKV, sd.G) == (2, 1, 2)
    full = Q.pack_hf(d, O.SyntheticWeights(od, seed=3, gamma="ones").get, 64)
    shards = [Q.shard_weights(full, d, ranks, r) for r in range(ranks)]
    for s_ in shards:
        assert {k: tuple(v.shape) for k, v in s_.items()} == {k: tuple(v) for k, v in Q.weight_shapes(sd, 64).items()}
    nq, nk, hd = d.NH * d.HD, d.NKV * d.HD, d.HD
    w = full["0.wqkv"]
    for r, s_ in enumerate(shards):
        q_rows, k_rows, v_rows = s_["0.wqkv"][:2 * hd], s_["0.wqkv"][2 * hd:3 * hd], s_["0.wqkv"][3 * hd:]
        assert np.array_equal(q_rows, w[r * 2 * hd:(r + 1) * 2 * hd])
        kvh = (2 * r) // d.G                                             # the kv head of the rank's q heads
        assert np.array_equal(k_rows, w[nq + kvh * hd:nq + (kvh + 1) * hd]) and np.array_equal(v_rows, w[nq + nk + kvh * hd:nq + nk + (kvh + 1) * hd])
    # a rank's graph is a valid single-device program
    g, pool, sz = Q.build_graph(sd, lambda n: {"xrows": 1 << 30}.get(n, 4096), 64, ranks=ranks, rank=3)
    plan = compile_graph(g, "b200", {"POOL": len(pool.bytes())})
    assert verify_plan(plan) == [] and not simulate(plan).deadlock


@pytest.mark.parametrize("od", [SMALL_MOE, SMALL_DENSE])
def test_rank_graph_is_a_valid_single_device_program_with_flagged_grids(od):
    ranks, rank = 2, 1
    sd = Q.shard_dims(qdims(od), ranks)
    base = {"xrows": 1 << 30}
    g, pool, sz = Q.build_graph(sd, lambda n: base.get(n, 4096), 64, ranks=ranks, rank=rank)
    blob_pool = pool.bytes()
    plan = compile_graph(g, "b200", {"POOL": len(blob_pool)})
    assert verify_plan(plan) == []
    assert not simulate(plan).deadlock
    flagged = sorted(gr.name for gr in g.grids if gr.body.exchange)
    assert flagged == sorted([f"o_proj_{L}" for L in range(sd.L)] + [f"{'moe_down' if sd.moe else 'down'}_{L}" for L in range(sd.L)])
    # the blob carries the flag in the last word of each 48-byte type row
    blob = plan.to_blob([("impargs", len(blob_pool)), ("vl", 8)], blob_pool)
    n_types, n_tensors = struct.unpack_from("<I", blob, 20)[0], struct.unpack_from("<I", blob, 36)[0]
    toff = 64 + 64 * n_tensors
    flags = [struct.unpack_from("<i", blob, toff + 48 * i + 44)[0] for i in range(n_types)]
    by_id = {tid: name for name, tid in plan.type_ids.items()}
    assert sorted(by_id[i] for i, f in enumerate(flags) if f) == flagged
    # the exchanged grids name their block of flagged rows in `rows` and carry the flagged mode bit; the folds after
    # them read `ranks` rows from the same block
    rows = {r[0]: r for r in pool.rows}
    FL = 0x1000

    def field(grid, off, fmt):
        return struct.unpack_from(fmt, blob_pool, rows[grid][4] + off)[0]
    blk = lambda L, kind: base["xrows"] + (2 * L + kind) * ranks * sd.H * 4      # noqa: E731
    nxt, dn = ("router", "moe_down") if sd.moe else ("gate_up", "down")
    for L in range(sd.L):
        assert field(f"o_proj_{L}", 64, "<Q") == blk(L, 0) and field(f"o_proj_{L}", 104, "<i") & FL
        assert field(f"{nxt}_{L}", 64, "<Q") == blk(L, 0) and field(f"{nxt}_{L}", 96, "<i") == ranks and field(f"{nxt}_{L}", 104, "<i") & FL
        assert field(f"{dn}_{L}", 64, "<Q") == blk(L, 1) and field(f"{dn}_{L}", 104, "<i") & FL
    assert field("qkv_0", 96, "<i") == 0 and not field("qkv_0", 104, "<i") & FL
    assert field("qkv_1", 64, "<Q") == blk(0, 1) and field("qkv_1", 96, "<i") == ranks and field("qkv_1", 104, "<i") & FL
    assert field("lm_head", 64, "<Q") == blk(sd.L - 1, 1) and field("lm_head", 96, "<i") == ranks
    assert Q.argmax_offset(sd, ranks) == blk(sd.L, 0) - base["xrows"] and Q.exchange_bytes(sd, ranks) == Q.argmax_offset(sd, ranks) + Q.ARGMAX_BLOCK
    # the lm_head is split by vocabulary: this rank's rows and logits only
    assert sd.VL == sd.V // ranks and field("lm_head", 48, "<i") == sd.VL


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from etx_megakernel_b200.runtime import dist as D
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    got = D.gather_handles(bytes([rank]) * 64, dist)
    dist.barrier()
    q.put((rank, got))
    dist.destroy_process_group()


def test_two_ranks_pass_their_region_handles_around():
    mp = pytest.importorskip("torch.multiprocessing")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29633, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, got in out:
        assert got == [bytes([0]) * 64, bytes([1]) * 64]
