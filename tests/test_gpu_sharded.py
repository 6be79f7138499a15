"""The sharded (tensor-parallel) decode step on the GPU.

One GPU: a rank whose "peer" is its own exchange region (its rows and arrivals loop back to itself) must reproduce, bit
for bit, the same shard run as an ordinary single-rank program -- that covers the system-scope waits, the row copies,
the peer arrivals and the doubled counts inside ONE launch.  Two GPUs (skipped with fewer): two processes, one shard
each, against the whole model on one GPU and the oracle's tokens."""
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200.models import decode as D  # noqa: E402
from etx_megakernel_b200.models import qwen as Q  # noqa: E402
from etx_megakernel_b200.runtime import EtxbError, ExchangeRegion  # noqa: E402
from oracle import ref_decode as O  # noqa: E402
from tests.golden.cases import SMALL_DENSE, SMALL_MOE  # noqa: E402

FIELDS = ("name", "H", "NH", "NKV", "HD", "INTER", "L", "V", "eps", "theta", "tie", "bias", "qk_norm", "moe", "E", "TOPK", "MI", "norm_topk")
MAXLEN, N_PROMPT, N_GEN = 64, 6, 20


def qdims(od):
    return Q.Dims(**{f: getattr(od, f) for f in FIELDS})


def shard_on(od, ranks, rank, device, seed=1):
    d = qdims(od)
    full = Q.pack_hf(d, O.SyntheticWeights(od, seed=seed, gamma="ones").get, MAXLEN)
    return Q.shard_dims(d, ranks), D.to_device_weights(Q.shard_weights(full, d, ranks, rank), f"cuda:{device}")


def prompt_of(od):
    return np.random.default_rng(7).integers(0, od.V, N_PROMPT)


def long_prompt(od):
    return np.random.default_rng(8).integers(0, od.V, 24)


@pytest.mark.parametrize("od", [SMALL_MOE, SMALL_DENSE])
def test_rank_looped_back_to_itself_equals_the_plain_program(od):
    """Rank 0 of 2 whose "peer" mapping is its own region shifted by one row: what it publishes for the peer lands in row
    1 of its own blocks, so every fold adds the rank's rows twice.  With o_proj and down weights halved (exact in bf16)
    that is bit for bit the plain single-rank program."""
    sd, w = shard_on(od, 2, 0, 0)
    plain = D.DecodeProgram(sd, w, device=0, maxlen=MAXLEN)
    want = plain.generate(prompt_of(od), N_GEN)
    want_logits, want_resid = plain.read("logits"), plain.read("resid")
    lean = plain.session.status().kernel_variant
    plain.close()
    half = {k: (v * 0.5 if k.rsplit(".", 1)[-1] in ("wo", "w2", "wd") else v) for k, v in w.items()}
    for full_kernel in (0, 1):
        prog = D.DecodeProgram(sd, half, device=0, maxlen=MAXLEN, ranks=2, rank=0)
        with pytest.raises(EtxbError, match="set_exchange comes before"):
            prog.session.launch()                                  # a rank's plan does not run unconnected
        prog.region.peers[1] = prog.region.ptr + sd.H * 4
        prog.session.set_exchange(0, 2, prog.region)
        prog.region.peers = {}                                     # (nothing was opened: nothing to close)
        prog.session.set_option("full_kernel", full_kernel)
        got = prog.generate(prompt_of(od), N_GEN)
        assert prog.session.status().kernel_variant == (0 if full_kernel else lean)      # the lean kernels cover the sharded step
        assert got.tolist() == want.tolist()
        assert np.array_equal(prog.read("logits"), want_logits) and np.array_equal(prog.read("resid"), want_resid)
        with pytest.raises(EtxbError):
            prog.session.launch_unfused()
        prog.close()


@pytest.mark.parametrize("od", [SMALL_MOE, SMALL_DENSE])
def test_flagged_hand_off_on_one_rank_equals_the_plain_program(od):
    """One rank with the flagged hand-off (the folds poll the rows o_proj / down publish instead of waiting for those grids'
    events): the same arithmetic on the same values, so tokens, logits and hidden state are bit-identical to the plain
    program, on the lean and on the full kernel."""
    d = qdims(od)
    w = D.to_device_weights(Q.pack_hf(d, O.SyntheticWeights(od, seed=2, gamma="ones").get, MAXLEN), "cuda:0")
    plain = D.DecodeProgram(d, w, device=0, maxlen=MAXLEN)
    want, want_logits, want_resid = plain.generate(prompt_of(od), N_GEN), plain.read("logits"), plain.read("resid")
    plain.close()
    for full_kernel in (0, 1):
        prog = D.DecodeProgram(d, w, device=0, maxlen=MAXLEN, flagged=True)
        prog.session.set_option("full_kernel", full_kernel)
        got = prog.generate(prompt_of(od), N_GEN)
        assert got.tolist() == want.tolist()
        assert np.array_equal(prog.read("logits"), want_logits) and np.array_equal(prog.read("resid"), want_resid)
        prog.close()


def test_exchange_region_and_argument_checks():
    reg = ExchangeRegion(4096, 0)
    assert reg.ptr % 256 == 0 and len(reg.handle) == 64 and any(reg.handle)
    sd, w = shard_on(SMALL_MOE, 2, 0, 0)
    unsharded = D.DecodeProgram(sd, w, device=0, maxlen=MAXLEN)
    reg.peers[1] = reg.ptr
    with pytest.raises(EtxbError, match="marks no grid"):
        unsharded.session.set_exchange(0, 2, reg)              # the plan of a single-rank program exchanges nothing
    unsharded.close()
    prog = D.DecodeProgram(sd, w, device=0, maxlen=MAXLEN, ranks=2, rank=0)
    with pytest.raises(EtxbError):
        prog.session.set_exchange(0, 2, prog.region)           # no peer mapped yet
    with pytest.raises(EtxbError):
        prog.session.set_exchange(2, 2, prog.region)           # rank out of range
    # an exchanged grid whose block lies outside the region is refused when the records are built (before any launch)
    small = ExchangeRegion(4096, 0)
    small.peers[1] = small.ptr
    prog.session.set_exchange(0, 2, small)
    with pytest.raises(EtxbError, match="outside the exchange region"):
        prog.session.launch()
    small.peers, reg.peers = {}, {}
    prog.close(); small.close(); reg.close()


def test_a_peer_that_never_publishes_ends_in_a_timeout_status():
    """The bounded wait of the fold: the "peer" is a second region of this process that nothing reads or writes, so row 1
    never carries this step's flag; the step gives up at its deadline and reports it, the context stays usable."""
    sd, w = shard_on(SMALL_DENSE, 2, 0, 0)
    prog = D.DecodeProgram(sd, w, device=0, maxlen=MAXLEN, ranks=2, rank=0)
    other = ExchangeRegion(prog.region.nbytes, 0)
    prog.region.peers[1] = other.ptr
    prog.session.set_exchange(0, 2, prog.region)
    prog.region.peers = {}
    prog.session.set_option("timeout_ms", 200)
    with pytest.raises(EtxbError) as e:
        prog.generate(prompt_of(SMALL_DENSE), 2)
    assert e.value.status == "E_TIMEOUT"
    assert torch.zeros(4, device="cuda:0").sum().item() == 0.0     # the context is alive
    prog.close(); other.close()


# ------------------------------------------------------------------------------------------------ two GPUs, two processes
def _rank(rank, world, port, od_name, q):
    import torch.distributed as dist
    from etx_megakernel_b200.runtime import dist as RD
    od = {"moe": SMALL_MOE, "dense": SMALL_DENSE}[od_name]
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    sd, w = shard_on(od, world, rank, rank)
    prog = D.DecodeProgram(sd, w, device=rank, maxlen=MAXLEN, ranks=world, rank=rank)
    prog.session.set_option("timeout_ms", 5000)
    err = None
    try:
        RD.connect_ranks(prog, dist)
        forced = prog.generate(long_prompt(od), 1)                # every input token given: the states depend on no sampled token
        fl, fr = prog.read("logits"), prog.read("resid")
        dist.barrier()
        got = prog.generate(prompt_of(od), N_GEN)
        q.put((rank, got.tolist(), prog.read("logits"), (forced.tolist(), fl, fr)))
    except Exception as e:                                     # report, then leave together
        err = repr(e)
        q.put((rank, err, None, None))
    RD.close_ranks(prog, dist)
    dist.destroy_process_group()


@pytest.mark.parametrize("od_name,world", [("moe", 2), ("dense", 2), ("moe", 4), ("dense", 4)])
def test_two_ranks_on_two_gpus_match_the_whole_model(od_name, world):
    """world = 4 on these models (2 kv heads) is the case with more ranks than kv heads: every kv head lives on two ranks."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    od = {"moe": SMALL_MOE, "dense": SMALL_DENSE}[od_name]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank, args=(r, world, 29641 + (od_name == "dense") + 2 * world, od_name, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = sorted((q.get(timeout=300) for _ in procs), key=lambda t: t[0])
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    for rank, toks, logits, resid in out:
        assert logits is not None, f"rank {rank}: {toks}"
    # both ranks hold bit-identical hidden states (same rows added in the same order) and agree on every token
    # (the lm_head is split by vocabulary: a rank's logits are its half, the token is agreed on through the argmax exchange)
    for r in range(1, world):
        assert out[0][1] == out[r][1]
        assert out[0][3][0] == out[r][3][0] and np.array_equal(out[0][3][2], out[r][3][2])
    # against the whole model on one GPU with every input token given: hidden state and logits within the bf16 tolerance
    # (a rank rounds its partial rows to bf16 before they are added, the whole model rounds the whole row once)
    d = qdims(od)
    W = O.SyntheticWeights(od, seed=1, gamma="ones")
    whole = D.DecodeProgram(d, D.to_device_weights(Q.pack_hf(d, W.get, MAXLEN), "cuda:0"), device=0, maxlen=MAXLEN)
    wtok = whole.generate(long_prompt(od), 1).tolist()
    wl, wr = whole.read("logits"), whole.read("resid")
    vl = Q.shard_dims(d, world).VL
    assert vl == d.V // world
    fl, fr = np.concatenate([out[r][3][1][:vl] for r in range(world)]), out[0][3][2]
    el, er = np.abs(fl - wl).max() / np.abs(wl).max(), np.abs(fr - wr).max() / np.abs(wr).max()
    assert el <= 2e-2 and er <= 2e-2, f"logits off by {el:.4f}, hidden state by {er:.4f} (relative to the largest value)"
    top2 = np.sort(wl)[-2:]
    if top2[1] - top2[0] > 4e-2 * np.abs(wl).max():
        assert out[0][3][0] == wtok
    # and against the ORACLE with every input token given (teacher forcing): the ranks' hidden state and logits within the
    # bf16 tolerance of the CPU numerical path
    ref = O.Ref(od, W, MAXLEN)
    for t, tok in enumerate(long_prompt(od)):
        dump = []
        otok, ol = ref.step(int(tok), t, dump=dump, return_logits=True)
    eo_l, eo_h = np.abs(fl - ol).max() / np.abs(ol).max(), np.abs(fr - dump[-1]).max() / np.abs(dump[-1]).max()
    print("against the oracle: logits", eo_l, "hidden", eo_h, "token", out[0][3][0], "oracle", otok)
    assert eo_l <= 2e-2 and eo_h <= 2e-2, f"against the oracle: logits off by {eo_l:.4f}, hidden state by {eo_h:.4f}"
    # sampled tokens: equal to the whole model's until a step whose top-2 margin is inside that tolerance
    want = whole.generate(prompt_of(od), N_GEN).tolist()
    whole.close()
    print("relative error: logits", el, "hidden", er, "tokens equal for", next((i for i, (a, b) in enumerate(zip(out[0][1], want)) if a != b), N_GEN), "steps")
