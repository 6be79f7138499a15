"""Batched decode on the GPU (several sequences per step in one persistent launch) against the oracle run per sequence:
greedy tokens per column (identical, or a first difference inside the oracle's own two-ulp logit margin -- the reference's
tie rule, examples/vllm_llm/host.hip:930-946), routing ids bit-exact, hidden state and logits within bf16 tolerance,
columns independent of their neighbours, expert lists with more tokens than one tensor-core pass holds."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200.models import batched as BT  # noqa: E402
from etx_megakernel_b200.models import decode as D  # noqa: E402
from etx_megakernel_b200.models import qwen as Q  # noqa: E402
from oracle import ref_decode as O  # noqa: E402
from tests.golden.cases import SMALL_MOE  # noqa: E402

BF16_REL = 2e-2
FIELDS = ("name", "H", "NH", "NKV", "HD", "INTER", "L", "V", "eps", "theta", "tie", "bias", "qk_norm", "moe", "E", "TOPK", "MI", "norm_topk")
MID = O.Dims(name="mid_moe", H=1024, NH=16, NKV=4, HD=128, INTER=0, L=3, V=4096, qk_norm=True, moe=True, E=32, TOPK=8, MI=384, norm_topk=True)


def qdims(od):
    return Q.Dims(**{f: getattr(od, f) for f in FIELDS})


def program(od, W, B, maxlen, engine="tc"):
    d = qdims(od)
    prog = BT.BatchProgram(d, D.to_device_weights(Q.pack_hf(d, W.get, maxlen), "cuda:0"), B, device=0, maxlen=maxlen, engine=engine)
    assert prog.info["engine"] == engine
    return prog


def oracle_column(od, W, prompt, n_gen, ctx):
    ref = O.Ref(od, W, ctx)
    seq, gen, logits = list(prompt), [], []
    for t in range(len(prompt) + n_gen - 1):
        nxt, lg = ref.step(int(seq[t]), t, return_logits=True)
        if t >= len(prompt) - 1:
            gen.append(nxt); logits.append(lg)
            if len(seq) <= t + 1:
                seq.append(nxt)
    return gen, logits


def check_columns(name, got, od, W, prompts, n_gen, ctx):
    identical = 0
    for b, prompt in enumerate(prompts):
        want, logits = oracle_column(od, W, prompt, n_gen, ctx)
        g = got[b].tolist()
        if g == want:
            identical += 1
            continue
        i = next(k for k, (x, y) in enumerate(zip(g, want)) if x != y)
        lg = logits[i]
        margin, ulp = float(lg[want[i]] - lg[g[i]]), float(abs(lg[want[i]])) * 2.0 ** -7
        print(f"[{name}] column {b}: first difference at token {i}: device {g[i]}, oracle {want[i]}, oracle margin {margin:.5f}, bf16 ulp {ulp:.5f}")
        assert margin <= 2 * ulp, f"column {b} token {i}: device chose {g[i]}, oracle {want[i]}, margin {margin} > 2 ulps ({ulp})"
    print(f"[{name}] {identical} of {len(prompts)} columns gave {n_gen} tokens identical to the oracle's")
    return identical


@pytest.mark.parametrize("od,B,engine", [(SMALL_MOE, 4, "tc"), (MID, 8, "tc"), (MID, 32, "tc"), (MID, 40, "tc"), (SMALL_MOE, 4, "mma"), (MID, 32, "mma")])
def test_batched_greedy_tokens_per_column(od, B, engine):
    """Both engines of the batched grids: tcgen05.mma (TMA tensor copies, accumulators in tensor memory; 40 columns = two
    passes of the dense grids) and the mma.sync tiles."""
    W = O.SyntheticWeights(od, seed=31, gamma="ones")
    prompts = np.random.default_rng(B).integers(0, od.V, (B, 12))
    prog = program(od, W, B, 64, engine)
    got = prog.generate(prompts, 12)
    prog.close()
    identical = check_columns(f"{od.name} x{B} {engine}", got, od, W, prompts, 12, 64)
    assert identical >= (B + 1) // 2, f"only {identical} of {B} columns identical"


def test_columns_do_not_depend_on_their_neighbours():
    """The same prompt in every column gives the same tokens and bit-identical logits in every column; the same prompt next
    to different neighbours gives the same tokens as alone."""
    od = SMALL_MOE
    W = O.SyntheticWeights(od, seed=32, gamma="ones")
    rng = np.random.default_rng(5)
    one = rng.integers(0, od.V, 10)
    prog = program(od, W, 8, 64)
    same = prog.generate(np.tile(one, (8, 1)), 8)
    logits = prog.read("logits")
    assert all(same[b].tolist() == same[0].tolist() for b in range(8))
    assert all(np.array_equal(logits[b], logits[0]) for b in range(8))
    mixed = np.stack([one] + [rng.integers(0, od.V, 10) for _ in range(7)])
    got = prog.generate(mixed, 8)
    assert got[0].tolist() == same[0].tolist()
    prog.close()


def test_whole_sequence_attention_agrees_with_the_partitioned_form():
    """20 sequences of a 150-token prompt (two partitions of 128 positions) through ONE layer, so that nothing but the
    attention phase separates the two forms: at B = 20 the attention grid has one task per (sequence, kv head) that
    walks the partitions itself with its products on the tensor cores (bf16 q / K / V, the probabilities as a bf16 value
    plus the bf16 of its rounding error, fp32 accumulation); at B = 10 it has one task per partition on the fp32 pipes
    and a merge through flagged partials.  Same partition boundaries and merge order, sums in another order: the KV
    caches are bit-identical, the attention output agrees within 2 bf16 ulps per element with >= 90 % of the elements
    identical.  (Through several MoE layers a one-ulp difference can flip a near-tie routing decision, which is why the
    multi-layer comparisons are made against the oracle with its tie rule, not between the two forms.)"""
    from dataclasses import replace
    od = replace(MID, L=1)
    W = O.SyntheticWeights(od, seed=35, gamma="ones")
    prompts = np.random.default_rng(8).integers(0, od.V, (20, 150))
    whole = program(od, W, 20, 192)
    assert whole.info["attn_whole"] and whole.info["attn"][2] == 2
    whole.generate(prompts, 1)
    att, kc, vc = whole.read("attn_out"), whole.read("kc"), whole.read("vc")
    whole.close()
    for half in range(2):
        part = program(od, W, 10, 192)
        assert not part.info["attn_whole"]
        part.generate(prompts[10 * half: 10 * half + 10], 1)
        patt, pkc, pvc = part.read("attn_out"), part.read("kc"), part.read("vc")
        part.close()
        nblk = pkc.shape[1] // 10
        assert np.array_equal(kc[:, 10 * half * nblk: (10 * half + 10) * nblk], pkc) and np.array_equal(vc[:, 10 * half * nblk: (10 * half + 10) * nblk], pvc)
        g, w = att[10 * half: 10 * half + 10], patt
        scale = np.abs(w).max()
        ulp = np.maximum(np.abs(w) * 2.0 ** -7, scale / 4096)
        same = float(np.mean(g == w))
        print(f"whole-sequence vs partitioned attention, columns {10 * half}..{10 * half + 9}: max diff {np.abs(g - w).max() / scale:.2e} of scale, {same:.1%} identical")
        assert np.all(np.abs(g - w) <= 2 * ulp) and same >= 0.9


def test_one_batched_step_against_the_oracle_state():
    """One teacher-forced step at a short context, B = 8: routing ids of the last layer exact (a swap of two experts only inside the oracle's own near tie), routing weights
    within 2e-2, final hidden state and logits of every column within 2e-2 of the oracle's."""
    od, B, P = MID, 8, 9
    W = O.SyntheticWeights(od, seed=33, gamma="ones")
    prompts = np.random.default_rng(6).integers(0, od.V, (B, P))
    prog = program(od, W, B, 64)
    prog.generate(prompts, 1)
    hid, logits, ids, wts = prog.read("resid"), prog.read("logits"), prog.read("ti"), prog.read("tw")
    prog.close()
    for b in range(B):
        ref = O.Ref(od, W, 64)
        for t in range(P):
            dump, tr = [], {}
            _, lg = ref.step(int(prompts[b, t]), t, dump=dump, trace=tr, return_logits=True)
        if ids[b].tolist() != tr["ids"].tolist():
            # the columns' inputs to the last router differ from the oracle's by fp32 summation order (two layers of
            # tensor-core sums against BLAS sums), so two experts whose logits the oracle itself puts within two bf16 ulps
            # of each other may swap; anything else is an error
            ours, theirs = set(ids[b].tolist()) - set(tr["ids"].tolist()), set(tr["ids"].tolist()) - set(ids[b].tolist())
            assert len(ours) == len(theirs) <= 1, f"column {b}: routing ids {ids[b].tolist()} vs {tr['ids'].tolist()}"
            if ours:
                a, c = tr["rlog"][ours.pop()], tr["rlog"][theirs.pop()]
                print(f"[batched step] column {b}: one expert swapped, oracle logits {a:.5f} / {c:.5f}")
                assert abs(a - c) <= 2 * max(abs(a), abs(c)) * 2.0 ** -7, f"column {b}: routing ids differ beyond a near tie"
        else:
            assert np.all(np.abs(wts[b] - tr["wts"]) <= BF16_REL * np.abs(tr["wts"]).max())      # (a smooth function of logits that carry three layers of summation-order noise)
        eh = np.abs(hid[b] - dump[-1]).max() / np.abs(dump[-1]).max()
        el = np.abs(logits[b] - lg).max() / np.abs(lg).max()
        assert eh <= BF16_REL and el <= BF16_REL, f"column {b}: hidden {eh:.4f}, logits {el:.4f}"


@pytest.mark.parametrize("engine", ["tc", "mma"])
def test_an_expert_with_more_tokens_than_one_pass(engine):
    """Every column sees the same token, so all B = 12 columns select the same experts: each expert's list holds 12 entries,
    more than the 8 tokens of an mma.sync pass and of the tensor-core tile's M = 64 form.  Tokens equal the
    single-sequence program's (tie rule aside: compared on logits); the routing is the same in every column, the active
    experts counted per layer and step are the top-k ones, and (mma.sync engine, whose routing tile writes them) the
    per-expert lists are complete."""
    od, B = SMALL_MOE, 12
    W = O.SyntheticWeights(od, seed=34, gamma="ones")
    prompt = np.random.default_rng(7).integers(0, od.V, 6)
    prog = program(od, W, B, 64, engine)
    got = prog.generate(np.tile(prompt, (B, 1)), 6)
    ecount, elist, ids = prog.read("ecount"), prog.read("elist"), prog.read("ti")
    active = prog.active_experts()
    blog = prog.read("logits")
    prog.close()
    assert all(sorted(ids[b].tolist()) == sorted(ids[0].tolist()) for b in range(B))
    assert len(set(active.tolist())) == 1 and active[0] == od.TOPK * (len(prompt) + 6 - 1)      # top-k experts per layer and step
    if engine == "mma":
        assert sorted(np.nonzero(ecount)[0].tolist()) == sorted(ids[0].tolist()) and set(ecount[ecount > 0].tolist()) == {B}
        for e in np.nonzero(ecount)[0]:
            assert sorted((int(v) >> 8) for v in elist[e, :B]) == list(range(B))
    d = qdims(od)
    single = D.DecodeProgram(d, D.to_device_weights(Q.pack_hf(d, W.get, 64), "cuda:0"), device=0, maxlen=64)
    want = single.generate(prompt, 6)
    slog = single.read("logits")
    single.close()
    assert np.abs(blog[0] - slog).max() <= BF16_REL * np.abs(slog).max()
    if got[0].tolist() != want.tolist():
        top2 = np.sort(slog)[-2:]
        assert top2[1] - top2[0] <= 4 * abs(top2[1]) * 2.0 ** -7
