"""The benchmarked models at their full size against the oracle (BASELINE configs 3 and 4): 36-layer Qwen3-8B and 48-layer
Qwen3-30B-A3B with random-init weights generated on the device.  The oracle reads the same weights through a lazy
provider (tests/device_weights.py), so it runs the very model the kernel runs.

Per model: (1) a short random prompt and greedy tokens, free-running on both sides -- identical, or where a token
differs the oracle's own logit margin between the two candidates is at most 2 bf16 ulps (the reference's tie rule,
examples/vllm_llm/host.hip:930-946) and the comparison goes on teacher-forced; (2) teacher-forced steps at context
1024 over the same random KV cache, layer by layer on the oracle's own inputs (first, middle, last layer): layer output
within 2e-2 of its largest magnitude and >= 50 % of the elements bit-identical (what is left are single bf16 roundings
that fell the other way), KV slot written in place.  What matched
and every margin are printed (pytest -s / the captured output of a failing run)."""
import os
import time

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200.models import decode as D  # noqa: E402
from etx_megakernel_b200.models import qwen as Q  # noqa: E402
from oracle import ref_decode as O  # noqa: E402
from tests.device_weights import DeviceWeights  # noqa: E402

BF16_REL = 2e-2
CFG = {"qwen3-30b-a3b": O.QWEN3_30B_A3B, "qwen3-8b": O.QWEN3_8B}


def greedy_against_oracle(name, d, w, n_prompt, n_gen, maxlen=128):
    od = O.dims_from_config(CFG[name], name)
    prompt = np.random.default_rng(5).integers(0, d.V, n_prompt)
    prog = D.DecodeProgram(d, w, device=0, maxlen=maxlen)
    got = prog.generate(prompt, n_gen).tolist()
    ref = O.Ref(od, DeviceWeights(d, w), maxlen)
    seq, want, logits = list(prompt), [], []
    t0 = time.perf_counter()
    for t in range(n_prompt + n_gen - 1):
        nxt, lg = ref.step(int(seq[t]), t, return_logits=True)
        if t >= n_prompt - 1:
            want.append(nxt); logits.append(lg)
            if len(seq) <= t + 1:
                seq.append(nxt)
    print(f"[{name}] oracle: {n_prompt + n_gen - 1} steps in {time.perf_counter() - t0:.1f} s")
    margins = [float(np.sort(lg)[-1] - np.sort(lg)[-2]) for lg in logits]
    print(f"[{name}] top-1 / top-2 logit margins of the oracle: min {min(margins):.4f} median {np.median(margins):.4f}")
    if got == want:
        print(f"[{name}] {n_gen} greedy tokens identical to the oracle's")
    else:
        forced = list(prompt) + want[:-1]                                  # teacher forcing on the oracle's sequence
        n = len(forced)
        tin = torch.zeros_like(prog.buf["token_in"]); tin[:n] = torch.tensor(forced, dtype=torch.int32)
        prog.buf["token_in"].copy_(tin)
        for t in range(n):
            prog.step(t, t, write_next=False, wait=(t == n - 1))
        out = prog.buf["token_out"][n_prompt - 1:n].cpu().numpy().tolist()
        ties = []
        for i, (g_tok, w_tok) in enumerate(zip(out, want)):
            if g_tok != w_tok:
                lg = logits[i]
                margin, ulp = float(lg[w_tok] - lg[g_tok]), float(abs(lg[w_tok])) * 2.0 ** -7
                ties.append((i, g_tok, w_tok, margin, ulp))
        print(f"[{name}] free-running tokens differ from the oracle's at {sum(a != b for a, b in zip(got, want))} of {n_gen} places; "
              f"teacher-forced: {len(ties)} differences (token, device, oracle, margin, bf16 ulp): {ties}")
        for i, g_tok, w_tok, margin, ulp in ties:
            assert margin <= 2 * ulp, f"token {i}: device chose {g_tok}, oracle {w_tok}, margin {margin} > 2 ulps ({ulp})"
        assert len(ties) <= 2, f"{len(ties)} near-tie flips in {n_gen} tokens"
    prog.close()


def layers_at_context(name, d, w, context=1024, steps=2):
    """Layer by layer at a long context.  A random-init MoE stack amplifies a one-ulp difference (a flipped 8th expert)
    from layer to layer, so the whole 48-layer hidden state is not a meaningful comparison at any tolerance (measured:
    bit-identical after 2 layers, 0.6 % off after 4, unrelated after 16 -- and the same between any two correct
    implementations).  Instead every checked layer gets the ORACLE's input for that layer: a one-layer program holding
    that layer's weights and KV cache, with the oracle's hidden state as its embedding row.  First, middle and last layer;
    the last one also checks the final norm + lm_head rows it is given.  The full-depth error is printed for the record."""
    from dataclasses import replace
    od = O.dims_from_config(CFG[name], name)
    maxlen = context + 16
    W = DeviceWeights(d, w)
    ref = O.Ref(od, W, maxlen)
    rng = np.random.default_rng(17)
    for L in range(d.L):
        ref.kc[L, :context] = O.bfr(rng.standard_normal((context, d.NKV, d.HD), dtype=np.float32) * np.float32(0.02))
        ref.vc[L, :context] = O.bfr(rng.standard_normal((context, d.NKV, d.HD), dtype=np.float32) * np.float32(0.02))
    whole = D.DecodeProgram(d, w, device=0, maxlen=maxlen)
    for L in range(d.L):
        whole.load_kv(L, ref.kc[L, :context], ref.vc[L, :context])
    d1 = replace(d, L=1, V=8, tie=False)
    toks = rng.integers(0, d.V, steps)
    for i, tok in enumerate(toks):
        pos = context + i
        dump = []
        want_tok, want_logits = ref.step(int(tok), pos, dump=dump, return_logits=True)
        inputs = [W.get("model.embed_tokens.weight")[int(tok)]] + dump[:-1]
        for L in sorted({0, d.L // 2, d.L - 1}):
            w1 = {k: w[k] for k in ("final_norm", "cos_sin")}
            w1["lm_head"] = w["lm_head"][:8].contiguous()
            emb = torch.zeros((8, d.H), dtype=torch.bfloat16, device="cuda:0")
            emb[0] = torch.from_numpy(inputs[L]).to("cuda:0").to(torch.bfloat16)
            w1["embed"] = emb
            for k in w:
                if k.startswith(f"{L}."):
                    w1["0." + k.split(".", 1)[1]] = w[k]
            one = D.DecodeProgram(d1, w1, device=0, maxlen=maxlen)
            one.load_kv(0, ref.kc[L, :pos], ref.vc[L, :pos])
            one.buf["token_in"][0] = 0
            torch.cuda.synchronize()                                      # the session launches on its own stream
            one.step(0, pos, write_next=False)
            got, want = one.read("resid"), dump[L]
            err, same = float(np.abs(got - want).max() / np.abs(want).max()), float(np.mean(got == want))
            msg = f"[{name}] context {pos}, layer {L} on the oracle's input: max err {err:.2e} of scale, {same:.1%} of elements identical"
            if L == d.L - 1:
                el = float(np.abs(one.read("logits")[:8] - want_logits[:8]).max() / np.abs(want_logits).max())
                msg += f"; first 8 logits max err {el:.2e}"
                assert el <= BF16_REL
            print(msg)
            assert err <= BF16_REL and same >= 0.5, msg
            Kd, Vd = one.read_kv(0, pos + 1)
            assert np.array_equal(Kd[:pos], ref.kc[L, :pos]) and np.mean(Kd[pos] == ref.kc[L, pos]) > 0.97 and np.mean(Vd[pos] == ref.vc[L, pos]) > 0.97
            one.close()
        whole.buf["token_in"][i] = int(tok)
        torch.cuda.synchronize()
        whole.step(i, pos, write_next=False)
        hid = whole.read("resid")
        print(f"[{name}] context {pos}, all {d.L} layers free-running (for the record, not asserted): hidden max err "
              f"{float(np.abs(hid - dump[-1]).max() / np.abs(dump[-1]).max()):.2e}, token {int(whole.buf['token_out'][i].item())} vs oracle {want_tok}")
    whole.close()


# The oracle takes a few seconds per token at these sizes (numpy on the host, weights fetched from the device), so the
# default run is short; ETXB_FULLSIZE_LONG=1 runs 16 prompt + 32 greedy tokens per model (several minutes each).
LONG = os.environ.get("ETXB_FULLSIZE_LONG", "0") == "1"


@pytest.mark.parametrize("name,n_prompt,n_gen", [("qwen3-30b-a3b", 16 if LONG else 6, 32 if LONG else 10), ("qwen3-8b", 16 if LONG else 4, 32 if LONG else 8)])
def test_full_size_model_against_the_oracle(name, n_prompt, n_gen):
    d = Q.load_dims(name)
    w = D.random_packed_weights(d, 1040, torch.device("cuda:0"), seed=0, gamma="ones")
    greedy_against_oracle(name, d, w, n_prompt, n_gen, maxlen=1040)
    layers_at_context(name, d, w, context=1024, steps=3 if LONG else 2)
    del w
    torch.cuda.empty_cache()
