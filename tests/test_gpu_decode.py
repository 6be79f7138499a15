"""The whole decode step on the GPU against the oracle: golden fixtures made by the reference, greedy tokens,
per-phase buffers of a single Qwen3-30B-A3B-shaped layer (BASELINE config 1), the host-buffer path, protocol checks
(every task runs exactly once per step) and the bounded wait."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200.models import decode as D  # noqa: E402
from etx_megakernel_b200.models import qwen as Q  # noqa: E402
from etx_megakernel_b200.runtime import EtxbError  # noqa: E402
from oracle import ref_decode as O  # noqa: E402
from tests.golden.cases import SMALL_DENSE, SMALL_MOE  # noqa: E402

BF16_REL = 2e-2


def qdims(od: O.Dims) -> Q.Dims:
    return Q.Dims(**{f: getattr(od, f) for f in ("name", "H", "NH", "NKV", "HD", "INTER", "L", "V", "eps", "theta", "tie", "bias",
                                                  "qk_norm", "moe", "E", "TOPK", "MI", "norm_topk")})


def make_program(od, W, maxlen, **kw):
    kw.setdefault("fused_attn", True)
    d = qdims(od)
    return D.DecodeProgram(d, D.to_device_weights(Q.pack_hf(d, W.get, maxlen), "cuda:0"), device=0, maxlen=maxlen, **kw)


def oracle_tokens(od, W, prompt, n_gen, ctx):
    ref = O.Ref(od, W, ctx)
    seq, gen = list(prompt), []
    for t in range(len(prompt) + n_gen - 1):
        nxt = ref.step(int(seq[t]), t)
        if t >= len(prompt) - 1:
            gen.append(nxt)
            if len(seq) <= t + 1:
                seq.append(nxt)
    return gen, ref


@pytest.mark.parametrize("dims,file", [(SMALL_MOE, "decode_small_moe.npz"), (SMALL_DENSE, "decode_small_dense.npz")])
def test_greedy_tokens_match_reference_fixture(golden_dir, dims, file):
    """Tokens the reference's own ref_numpy.py produced (fixture), the KV cache rows it wrote, and its residuals."""
    g = np.load(golden_dir / file)
    W = O.SyntheticWeights(dims, seed=int(g["seed"]), gamma=str(g["gamma"]))
    prompt, want = g["prompt"], g["gen"].tolist()
    prog = make_program(dims, W, 64)
    got = prog.generate(prompt, len(want))
    assert got.tolist() == want
    n = len(prompt) + len(want) - 1
    for L in range(dims.L):
        K, V = prog.read_kv(L, n)
        scale = np.abs(g["kc"][L]).max()
        assert np.abs(K - g["kc"][L]).max() <= BF16_REL * scale and np.abs(V - g["vc"][L]).max() <= BF16_REL * np.abs(g["vc"][L]).max()
        if L == 0:                                                        # layer 0 sees identical inputs: slot rows bit-exact
            assert np.mean(K == g["kc"][0]) > 0.99 and np.mean(V == g["vc"][0]) > 0.99
    toks, _ = prog.generate_host(prompt, len(want))
    assert toks.tolist() == want                                          # the host-buffer path gives the same tokens
    prog.close()


def oracle_run(od, W, prompt, n_gen, ctx):
    """Free-running greedy decode on the oracle; returns the generated ids and the bf16 logits of every generating step."""
    ref = O.Ref(od, W, ctx)
    seq, gen, logits = list(prompt), [], []
    for t in range(len(prompt) + n_gen - 1):
        nxt, lg = ref.step(int(seq[t]), t, return_logits=True)
        if t >= len(prompt) - 1:
            gen.append(nxt); logits.append(lg)
            if len(seq) <= t + 1:
                seq.append(nxt)
    return gen, logits


def check_greedy(od, W, prompt, n_gen, ctx, must_be_identical=False):
    """32 greedy tokens against the oracle.  Identical is the expectation; where a token differs, the oracle's own
    logits must show a near-tie between its choice and the device's (the two paths differ only in fp32 summation
    order, i.e. by at most a bf16 rounding of a logit): margin <= 2 bf16 ulps of the top logit -- the rule the
    reference applies to its own GPU runs (examples/vllm_llm/host.hip:930-946 counts small-margin mismatches as
    ties).  After a tie the comparison continues teacher-forced on the oracle's sequence."""
    want, logits = oracle_run(od, W, prompt, n_gen, ctx)
    prog = make_program(od, W, ctx)
    got = prog.generate(prompt, n_gen).tolist()
    margins = [float(np.sort(lg)[-1] - np.sort(lg)[-2]) for lg in logits]
    print(f"[greedy {od.name}] {n_gen} tokens, oracle top-1/top-2 margins min {min(margins):.4f} median {float(np.median(margins)):.4f}: "
          + ("identical" if got == want else f"first difference at token {next(i for i, (a, b) in enumerate(zip(got, want)) if a != b)}"))
    if got != want:
        assert not must_be_identical, f"tokens differ: {got} vs {want}"
        forced = list(prompt) + want[:-1]                                  # teacher forcing: the oracle's own sequence
        n = len(forced)
        tin = torch.zeros_like(prog.buf["token_in"]); tin[:n] = torch.tensor(forced, dtype=torch.int32)
        prog.buf["token_in"].copy_(tin)
        for t in range(n):
            prog.step(t, t, write_next=False, wait=(t == n - 1))
        out = prog.buf["token_out"][len(prompt) - 1:n].cpu().numpy().tolist()
        ties = 0
        for i, (g_tok, w_tok) in enumerate(zip(out, want)):
            if g_tok != w_tok:
                lg = logits[i]
                margin, ulp = float(lg[w_tok] - lg[g_tok]), float(abs(lg[w_tok])) * 2.0 ** -7
                print(f"[greedy {od.name}] teacher-forced token {i}: device {g_tok}, oracle {w_tok}, oracle margin {margin:.5f}, bf16 ulp {ulp:.5f}")
                assert margin <= 2 * ulp, f"token {i}: device chose {g_tok}, oracle {w_tok}, margin {margin} > 2 ulps ({ulp})"
                ties += 1
        assert ties <= 2, f"{ties} near-tie flips in {n_gen} tokens"
    prog.close()
    return got == want


def test_thirty_two_greedy_tokens_moe():
    """32 greedy tokens against the oracle on a 3-layer MoE model with the Qwen3 head geometry, four seeds: every
    difference must be a near-tie of the oracle's own logits, and most seeds must match token for token."""
    od = O.Dims(name="m", H=1024, NH=16, NKV=4, HD=128, INTER=0, L=3, V=4096, qk_norm=True, moe=True, E=32, TOPK=8, MI=256, norm_topk=True)
    identical = 0
    for seed in range(4):
        W = O.SyntheticWeights(od, seed=seed, gamma="ones")
        prompt = np.random.default_rng(seed).integers(0, od.V, 40)
        identical += check_greedy(od, W, prompt, 32, 96)
    print(f"[greedy m] {identical} of 4 seeds gave 32 tokens identical to the oracle's")
    assert identical >= 2, f"only {identical} of 4 seeds gave 32 identical tokens"


def test_unfused_attention_phases_and_separate_topk_give_the_same_tokens():
    """The graph with the reference's phase structure (prep -> attn -> reduce, stand-alone top-k) and the one with the
    general fused attention tile produce identical tokens and identical final buffers: those fusions change the schedule,
    not the arithmetic.  The grouped attention tile (partitions of 128 positions) sums in another order: same tokens,
    logits within the hidden-state tolerance (2e-2 relative to the largest logit)."""
    od = SMALL_MOE
    W = O.SyntheticWeights(od, seed=3, gamma="ones")
    prompt = np.random.default_rng(4).integers(0, od.V, 10)
    res = {}
    for name, kw in (("grouped", {}), ("general", {"fused_attn": "general"}), ("unfused", {"fused_attn": False, "fold_topk": False})):
        p = make_program(od, W, 64, **kw)
        if name == "grouped":
            assert p.sizing.attn[0] > 0, "the small model must take the grouped tile for this test to mean anything"
        res[name] = (p.generate(prompt, 12), p.read("logits"), *p.read_kv(1, 21))
        p.close()
    ta, la, ka, va = res["general"]; tb, lb, kb, vb = res["unfused"]
    assert ta.tolist() == tb.tolist() and np.array_equal(la, lb) and np.array_equal(ka, kb) and np.array_equal(va, vb)
    tg, lg, kg, vg = res["grouped"]
    assert tg.tolist() == ta.tolist()
    assert np.abs(lg - la).max() <= 2e-2 * np.abs(la).max()
    assert np.abs(kg - ka).max() <= 2e-2 * np.abs(ka).max() and np.abs(vg - va).max() <= 2e-2 * np.abs(va).max()


def test_lean_kernel_is_picked_for_decode_plans_and_matches_the_full_kernel():
    """The library runs fused decode plans on the lean kernel variant (only the tiles such a plan uses) and anything else
    on the full kernel; both give bit-identical results."""
    od = SMALL_MOE
    W = O.SyntheticWeights(od, seed=11, gamma="ones")
    prompt = np.random.default_rng(12).integers(0, od.V, 9)
    res = []
    for full in (0, 1):
        p = make_program(od, W, 64)
        p.session.set_option("full_kernel", full)
        res.append((p.generate(prompt, 10), p.read("logits"), *p.read_kv(1, 18)))
        gq = p.sizing.attn[0]
        assert p.session.status().kernel_variant == (0 if full else {1: 1, 2: 2, 4: 3, 8: 4}[gq])
        p.close()
    (ta, la, ka, va), (tb, lb, kb, vb) = res
    assert ta.tolist() == tb.tolist() and np.array_equal(la, lb) and np.array_equal(ka, kb) and np.array_equal(va, vb)
    for kw in ({"fused_attn": False, "fold_topk": False}, {"fused_attn": "general"}):      # plans with other tiles: the full kernel
        p = make_program(od, W, 64, **kw)
        assert p.session.status().kernel_variant == 0
        p.close()
    dense = make_program(SMALL_DENSE, O.SyntheticWeights(SMALL_DENSE, seed=1, gamma="ones"), 64)
    assert dense.session.status().kernel_variant == 0                                    # head_dim 64: the general attention tile
    dense.close()


def test_decode_across_partition_and_block_boundaries_up_to_the_last_cache_position():
    """A context that grows through the 128-position partition boundary of the grouped attention tile, through 16-position
    cache block boundaries, and ends on the very last position the cache has: tokens against the oracle (tie rule)."""
    od = O.Dims(name="edge", H=256, NH=4, NKV=2, HD=128, INTER=0, L=2, V=512, qk_norm=True, moe=True, E=8, TOPK=2, MI=64, norm_topk=True)
    W = O.SyntheticWeights(od, seed=21, gamma="ones")
    prompt = np.random.default_rng(22).integers(0, od.V, 118)
    check_greedy(od, W, prompt, 27, 144)                                    # positions 0 .. 143 = maxlen - 1


def test_launch_per_grid_baseline_gives_the_same_tokens():
    """The unfused baseline (one launch per grid) runs the same tiles in the same order: identical tokens, logits and cache."""
    od = SMALL_MOE
    W = O.SyntheticWeights(od, seed=5, gamma="ones")
    prompt = np.random.default_rng(6).integers(0, od.V, 9)
    res = []
    for unfused in (False, True):
        p = make_program(od, W, 64)
        res.append((p.generate(prompt, 10, unfused=unfused), p.read("logits"), *p.read_kv(1, 18)))
        if unfused:
            p.session.set_option("trace", 1)
            p.step(0, 20, False, unfused=True)
            assert (p.session.exec_counts() == 1).all()             # every task ran exactly once across the launches
        p.close()
    (ta, la, ka, va), (tb, lb, kb, vb) = res
    assert ta.tolist() == tb.tolist() and np.array_equal(la, lb) and np.array_equal(ka, kb) and np.array_equal(va, vb)


def test_program_from_a_pack_file_passes_the_golden_gate(tmp_path):
    """A vl.bin / vl.manifest directory (the reference packer's format) loaded back and run: same tokens as the weights it
    was written from, and the golden-file gate passes against the oracle's continuation."""
    from etx_megakernel_b200.models import packfile as PF
    od = SMALL_MOE
    W = O.SyntheticWeights(od, seed=7, gamma="ones")
    d = qdims(od)
    PF.write_vl(tmp_path, d, Q.pack_hf(d, W.get, 64), 64)
    d2, maxlen, packed = PF.read_vl(tmp_path, theta=od.theta)
    prompt = np.random.default_rng(8).integers(0, od.V, 12)
    prog = D.DecodeProgram(d2, PF.to_device(packed, "cuda:0"), device=0, maxlen=maxlen)
    got = prog.generate(prompt, 8).tolist()
    prog.close()
    direct = make_program(od, W, 64)
    assert got == direct.generate(prompt, 8).tolist()
    direct.close()
    # the golden file carries the oracle's continuation and its own top-1 / top-2 logit margins; the gate excuses a first
    # difference only where that margin is within two bf16 ulps of the top logit (the reference's tie rule)
    want, logits = oracle_run(od, W, prompt, 8, 64)
    top2 = [np.sort(lg)[-2:] for lg in logits]
    PF.write_golden(tmp_path / "golden_c12.txt", prompt, want, [float(t[1] - t[0]) for t in top2])
    _, gen, margins = PF.read_golden(tmp_path / "golden_c12.txt")
    assert gen == want
    tie = 2 * max(float(abs(t[1])) for t in top2) * 2.0 ** -7
    assert PF.check_golden(got, gen, margins, tie_margin=tie) == []
    assert PF.check_golden([w + 1 for w in want], gen, [m + 10 * tie + 1.0 for m in margins], tie_margin=tie) != []    # the gate does fail on a real difference


def test_thirty_two_greedy_tokens_dense_with_bias():
    od = O.Dims(name="dn", H=512, NH=8, NKV=2, HD=64, INTER=1536, L=3, V=2048, theta=1e4, tie=True, bias=True, qk_norm=False, moe=False)
    W = O.SyntheticWeights(od, seed=2, gamma="ones", std=0.05)
    prompt = np.random.default_rng(9).integers(0, od.V, 20)
    check_greedy(od, W, prompt, 32, 64)


def test_single_layer_qwen3_moe_config_one(golden_dir):
    """BASELINE config 1: one Qwen3-30B-A3B-shaped layer, batch 1, 1024 prior KV tokens, seed 0, against the output of
    the reference's CPU path (fixture) and, phase by phase, against the oracle: routing ids and the KV slot bit-exact,
    every bf16 vector within 2e-2 of the reference."""
    g = np.load(golden_dir / "layer_qwen3moe.npz")
    od = O.dims_from_config(O.QWEN3_30B_A3B, "qwen3-30b-a3b", layers=1)
    od.V, od.tie = 1, True
    W = O.SyntheticWeights(od, seed=0, gamma="normal")
    rng = np.random.default_rng(12345)
    S = 1024
    W.t["model.embed_tokens.weight"] = O.bfr(rng.standard_normal((1, od.H), dtype=np.float32))
    Kp = O.bfr(rng.standard_normal((S, od.NKV, od.HD), dtype=np.float32) * np.float32(0.02))
    Vp = O.bfr(rng.standard_normal((S, od.NKV, od.HD), dtype=np.float32) * np.float32(0.02))
    ref = O.Ref(od, W, S + 8)
    ref.kc[0, :S], ref.vc[0, :S] = Kp, Vp
    tr = {}
    out_ref = ref.layer(0, W.get("model.embed_tokens.weight")[0].copy(), S, tr)
    assert np.array_equal(out_ref, g["hidden_out"])                       # the oracle reproduces the reference fixture
    od.V = 8                                                             # the device argmax wants V % 8 == 0 rows to scan
    W.t["model.embed_tokens.weight"] = np.concatenate([W.t["model.embed_tokens.weight"], np.zeros((7, od.H), np.float32)])
    prog = make_program(od, W, 1072)
    prog.load_kv(0, Kp, Vp)
    prog.buf["token_in"][0] = 0
    prog.step(0, S, write_next=False)
    # the new KV slot: same bf16 values at the same paged address
    K, V = prog.read_kv(0, S + 1)
    assert np.array_equal(K[:S], Kp) and np.array_equal(V[:S], Vp)
    assert np.mean(K[S] == g["k_new"]) > 0.99 and np.abs(K[S] - g["k_new"]).max() <= BF16_REL * np.abs(g["k_new"]).max()
    assert np.mean(V[S] == g["v_new"]) > 0.99
    # routing: ids bit-exact, bf16 weights within one ulp
    assert prog.read("ti").tolist() == tr["ids"].tolist()
    assert np.all(np.abs(prog.read("tw") - tr["wts"]) <= np.abs(tr["wts"]) * 2.0 ** -7)
    acc = np.float32(0)
    for s_ in np.argsort(tr["ids"]):                                      # the expert combine: bf16 adds in ascending expert id
        acc = O.bfr(acc + tr["y"][s_])
    for name, want in (("attn_out", tr["attn"].reshape(-1)), ("o", tr["o"]), ("resid2", tr["resid2"]), ("o_norm", tr["xs2"]),
                       ("rlog", tr["rlog"]), ("mc2", tr["act"]), ("moe_out", acc)):
        got = prog.read(name).reshape(want.shape)
        scale = np.abs(want).max()
        assert np.abs(got - want).max() <= BF16_REL * scale, name
        assert np.mean(got == want) > 0.95, name
    # the layer output = residual the lm_head fold stores
    got = prog.read("resid")
    assert np.abs(got - g["hidden_out"]).max() <= BF16_REL * np.abs(g["hidden_out"]).max()
    assert np.mean(got == g["hidden_out"]) > 0.97
    prog.close()


def test_every_task_runs_exactly_once_and_trace_is_ordered():
    od = SMALL_MOE
    W = O.SyntheticWeights(od, seed=3, gamma="ones")
    prog = make_program(od, W, 64)
    prog.session.set_option("trace", 1)
    for t in range(3):
        prog.buf["token_in"][t] = 5 + t
        prog.step(t, t, write_next=False)
        assert np.all(prog.session.exec_counts() == 1)
    tr = prog.session.trace()
    assert np.all(tr[:, 1] >= tr[:, 0]) and np.all(tr[:, 2] >= tr[:, 1])
    # a consumer's "deps ready" stamp is never earlier than the end of its producers (qkv_0 waits for the prologue)
    plan = prog.plan
    first_qkv = plan.task_index[("qkv_0", (0,))]
    assert tr[first_qkv, 1] >= tr[plan.task_index[("prologue", (0,))], 2]
    assert prog.session.status().tasks_run == len(plan.tasks)
    prog.close()


def test_inconsistent_plan_is_rejected_before_launch():
    """Arrivals that do not add up to the declared count never reach the device: the library answers E_PLAN."""
    from etx_megakernel_b200.frontends import cuda_link
    from etx_megakernel_b200.ir import Graph
    from etx_megakernel_b200.passes import compile_graph
    from etx_megakernel_b200.runtime import Session
    g = Graph("stuck")
    g.tensor("impargs", (16,), role="weight", bytes_per_elem=1)
    g.etensor("E0", (1,), wait_count=1)
    g.etensor("E1", (1,), wait_count=1)
    g.call_device("a", (1,), cuda_link("", "nop"), args=["impargs"], consts=(0,), out_edges={"E0": "i->i"})
    g.call_device("b", (1,), cuda_link("", "nop"), args=["impargs"], consts=(0,), in_edges={"E0": "i->i"}, out_edges={"E1": "i->i"})
    plan = compile_graph(g, "b200", {})
    plan.task_out_words[0] = []                     # drop a's arrival: b would wait for a counter nobody bumps
    with pytest.raises(EtxbError) as e:
        Session(plan, {}, bytes(16))
    assert e.value.status == "E_PLAN"
    plan = compile_graph(g, "b200", {})
    plan.task_in_words[1] = [7]                     # a wait on an event that does not exist
    with pytest.raises(EtxbError) as e:
        Session(plan, {}, bytes(16))
    assert e.value.status == "E_PLAN"
    s = Session(compile_graph(g, "b200", {}), {}, bytes(16))     # the untouched plan runs
    s.run(5.0)
    s.close()


def test_wait_deadline_returns_status():
    """Device-side deadline: the consumer's producer is queued BEHIND it on the same worker (a plan the host-side
    verifier rejects; built here by hand), so the wait can only end by its deadline."""
    from etx_megakernel_b200.frontends import cuda_link
    from etx_megakernel_b200.ir import Graph
    from etx_megakernel_b200.passes import compile_graph
    from etx_megakernel_b200.passes.plan import verify_plan
    from etx_megakernel_b200.runtime import Session
    g = Graph("deadline")
    g.tensor("impargs", (16,), role="weight", bytes_per_elem=1)
    g.etensor("E0", (1,), wait_count=1)
    g.etensor("E1", (1,), wait_count=1)
    g.call_device("a", (1,), cuda_link("", "nop"), args=["impargs"], consts=(0,), out_edges={"E0": "i->i"})
    g.call_device("b", (1,), cuda_link("", "nop"), args=["impargs"], consts=(0,), in_edges={"E0": "i->i"}, out_edges={"E1": "i->i"})
    plan = compile_graph(g, "b200", {})
    plan.static_queues[(0, 0)] = [1, 0]              # consumer first, its producer behind it on the same worker
    plan.static_queues[(0, 1)] = []
    assert any("deadlock" in e for e in verify_plan(plan))
    s = Session(plan, {}, bytes(16))
    s.set_option("timeout_ms", 200)
    with pytest.raises(EtxbError) as e:
        s.run(5.0)
    assert e.value.status == "E_TIMEOUT"
    st = s.status()
    assert st.ctrl & 2 and st.stuck_event == 0
    plan2 = compile_graph(g, "b200", {})             # the same device context runs a healthy plan afterwards
    s2 = Session(plan2, {}, bytes(16))
    s2.run(5.0)
    s2.close(); s.close()


def test_a_step_after_an_abandoned_step_is_correct():
    """A step that is abandoned (here: the host watchdog aborts it almost at once) may stop in the middle of an attention
    phase and leave the merge-election counters of the fused attention grids off a multiple of their partition count.
    The library realigns them when it recovers, so the session goes on to produce the tokens a fresh session produces.
    To make the misalignment certain the counters are also knocked off by hand before the aborted step."""
    od = SMALL_MOE
    W = O.SyntheticWeights(od, seed=13, gamma="ones")
    prompt = np.random.default_rng(14).integers(0, od.V, 9)
    fresh = make_program(od, W, 64)
    want = fresh.generate(prompt, 10).tolist()
    fresh.close()
    prog = make_program(od, W, 64)
    assert prog.generate(prompt, 10).tolist() == want
    prog.buf["attn_counters"] += 1                    # every election now fires one arrival early ...
    torch.cuda.synchronize()
    prog.session.set_step(tok=0, pos=0, write_next=0)
    prog.session.launch()
    try:
        prog.session.wait(1e-7)                       # ... and this step is aborted by the host watchdog (or finishes first)
    except EtxbError as e:
        assert e.status in ("E_ABORTED", "E_TIMEOUT")
    else:
        prog.close()
        pytest.skip("the step finished before the host watchdog looked at it")
    assert prog.generate(prompt, 10).tolist() == want  # counters realigned: same tokens as the fresh session
    prog.close()


def test_full_size_model_properties():
    """Qwen3-30B-A3B at its full size (48 layers, random weights generated on the device): the oracle cannot follow at
    this size in seconds, so size-independent properties stand in -- the single launch, the launch-per-grid baseline,
    the full kernel variant and the host-buffer entry all produce the same greedy tokens, twice."""
    d = Q.load_dims("qwen3-30b-a3b")
    dev = torch.device("cuda:0")
    w = D.random_packed_weights(d, 128, dev, seed=0, gamma="ones")
    prompt = np.random.default_rng(3).integers(0, d.V, 24)
    runs = {}
    for name in ("lean", "lean again", "full kernel", "launch per grid"):
        prog = D.DecodeProgram(d, w, device=0, maxlen=128)
        if name == "full kernel":
            prog.session.set_option("full_kernel", 1)
        assert prog.session.status().kernel_variant == (0 if name == "full kernel" else {1: 1, 2: 2, 4: 3, 8: 4}[prog.sizing.attn[0]])
        runs[name] = prog.generate(prompt, 8, unfused=(name == "launch per grid")).tolist()
        if name == "lean":
            logits = prog.read("logits")
            assert np.isfinite(logits).all() and logits.std() > 0
            host, _ = prog.session.decode_host(np.asarray(prompt, np.int32), len(prompt) + 8 - 1, 0)
            runs["host buffers"] = host[len(prompt) - 1:].tolist()
        prog.close()
    first = runs["lean"]
    assert len(set(first)) > 1, "degenerate generation"
    for name, toks in runs.items():
        assert toks == first, f"{name}: {toks} != {first}"
