"""DeepSeek-V2 family on the GPU: the absorbed latent-attention tile and a small model (dense layer + shared-expert MoE
layers) against the CPU oracle (oracle/ref_mla.py, pinned by tests/golden/mla_layer.npz), through the C ABI."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200 import ops  # noqa: E402
from etx_megakernel_b200.importer import argblock  # noqa: E402
from etx_megakernel_b200.models import dsv2 as M  # noqa: E402
from etx_megakernel_b200.ops import mla as op_mla  # noqa: E402
from etx_megakernel_b200.runtime import op_launch  # noqa: E402
from oracle import ref_mla as R  # noqa: E402
from oracle.ref_decode import bfr, f32_to_bf16_bits  # noqa: E402
from tests.test_mla_host import oracle_dims  # noqa: E402

ENT = ops.all_entries()
DEV = "cuda:0"
BF16_REL = 2e-2          # tolerance for bf16 vectors (max error relative to the largest value, fp32 accumulation)


def dev_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(f32_to_bf16_bits(np.asarray(a, np.float32))).view(np.int16)).to(DEV).view(torch.bfloat16)


def host(t):
    torch.cuda.synchronize()
    return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()


@pytest.mark.parametrize("NH,ctx", [(4, 0), (4, 37), (16, 300), (16, 1027)])
def test_latent_attention_tile_against_the_oracle(NH, ctx):
    """A task per (head, 128 positions) over a context of `ctx` cached positions + the new one (1, 3 and 9 partitions; the
    new position first in its partition or in the middle): the cache row the tile writes is the oracle's bit for bit
    (latent RMSNorm in numpy's summation order, interleaved rope with fp32 YaRN tables), the attention output within
    the bf16 tolerance of the oracle's (fp32 sums in another order, softmax merged over partitions)."""
    d = M.MlaDims(name="t", H=NH * 128, NH=NH, C=512, DN=128, DR=64, DV=128, MI=128, E=4, TOPK=2, NS=0, DENSE_LAYERS=0, DENSE_INTER=0, L=1, V=256)
    od = oracle_dims(d)
    maxlen = ctx + 8
    lw = R.synthetic_layer(od, seed=10 + ctx)
    lw.o_proj = np.eye(d.H, dtype=np.float32)                 # the oracle's attention() then returns bf16(out) itself
    cos, sin = R.yarn_tables(od, maxlen)
    rng = np.random.default_rng(ctx)
    cache = np.zeros((maxlen, d.ROW), np.float32)
    for t in range(ctx):
        R.attention(od, lw, bfr(rng.standard_normal(d.H).astype(np.float32)), cache, t, cos, sin)
    x = bfr(rng.standard_normal(d.H).astype(np.float32))
    before = cache.copy()
    want = R.attention(od, lw, x, cache, ctx, cos, sin)
    xn = R.rmsnorm2(x, lw.input_layernorm, d.eps)
    qkv = np.concatenate([bfr(lw.q_proj @ xn), bfr(lw.kv_a_proj_with_mqa @ xn)])
    t_qkv, t_ln, t_w = dev_bf16(qkv), dev_bf16(lw.kv_a_layernorm), dev_bf16(lw.kv_b_proj)
    t_cs = torch.from_numpy(M.yarn_table(d, maxlen)).to(DEV)
    t_cache = dev_bf16(before)
    t_pos = torch.tensor([ctx], dtype=torch.int64, device=DEV)
    t_out = torch.zeros(NH * d.DV, dtype=torch.bfloat16, device=DEV)
    nparts = op_mla.partitions(maxlen)
    t_tmp = torch.zeros((op_mla.tmp_pairs(NH, d.C, maxlen), 2), dtype=torch.float32, device=DEV)
    blob = argblock.pack_named(ENT["mla_attn"], (NH * (nparts + op_mla.FINISHERS), 1, 1), qkv=t_qkv.data_ptr(), kvln=t_ln.data_ptr(), cos_sin=t_cs.data_ptr(), wkvb=t_w.data_ptr(),
                               cache=t_cache.data_ptr(), positions=t_pos.data_ptr(), out=t_out.data_ptr(), NH=NH, C=d.C, DN=d.DN, DR=d.DR, DV=d.DV,
                               maxlen=maxlen, scale=d.scale, eps=d.eps, tmp=t_tmp.data_ptr(), max_parts=nparts, tag=3)
    op_launch("mla_attn", blob, NH * (nparts + op_mla.FINISHERS))
    got_cache, got = host(t_cache), host(t_out)
    assert np.array_equal(got_cache[ctx], cache[ctx]), "the new cache row differs from the oracle's"
    assert np.array_equal(got_cache[:ctx], before[:ctx]) and not got_cache[ctx + 1:].any()
    scale = np.abs(want).max()
    err = np.abs(got - want).max() / scale
    print(f"mla_attn NH={NH} ctx={ctx}: max err {err:.5f} of scale, {np.mean(got == want) * 100:.1f} % of elements identical")
    assert err <= BF16_REL and np.mean(got == want) >= 0.9


def small_model(seed=0):
    d = M.MlaDims(name="mla_small", H=512, NH=4, C=512, DN=128, DR=64, DV=128, MI=128, E=8, TOPK=2, NS=2, DENSE_LAYERS=1, DENSE_INTER=384, L=3, V=1024)
    rng = np.random.default_rng(seed)
    layers = [R.synthetic_layer(oracle_dims(d, dense=d.dense(L)), seed=100 * seed + L) for L in range(d.L)]
    embed = bfr(rng.standard_normal((d.V, d.H)).astype(np.float32) * np.float32(0.5))
    final_norm = bfr(1 + 0.1 * rng.standard_normal(d.H).astype(np.float32))
    lm_head = bfr(rng.standard_normal((d.V, d.H)).astype(np.float32) * np.float32(0.05))
    return d, layers, embed, final_norm, lm_head


def oracle_decode(d, layers, embed, final_norm, lm_head, prompt, n_gen, maxlen):
    """Greedy decode with the oracle's layers; returns (tokens, per-step logits, per-step final hidden, last trace)."""
    ods = [oracle_dims(d, dense=d.dense(L)) for L in range(d.L)]
    cos, sin = R.yarn_tables(ods[0], maxlen)
    caches = [np.zeros((maxlen, d.ROW), np.float32) for _ in range(d.L)]
    seq, gen, logits, hidden, trace = list(prompt), [], [], [], {}
    for t in range(len(prompt) + n_gen - 1):
        x = embed[seq[t]].copy()
        for L in range(d.L):
            trace = {}
            x = R.layer(ods[L], layers[L], x, caches[L], t, cos, sin, trace)
        lg = bfr(lm_head @ R.rmsnorm2(x, final_norm, d.eps))
        if t >= len(prompt) - 1:
            nxt = int(np.argmax(lg))
            gen.append(nxt); logits.append(lg); hidden.append(x)
            if t + 1 >= len(prompt):
                seq.append(nxt)
    return gen, logits, hidden, trace


def test_small_model_against_the_oracle():
    """A dense layer and two MoE layers with two shared experts: teacher-forced hidden state and logits within the bf16
    tolerance of the oracle at every generated position, routing of the last layer equal to the oracle's (as a set; the
    shared experts in the last slots), greedy tokens equal unless the oracle's own margin between the two candidates is
    within 4 bf16 ulps of the logit."""
    d, layers, embed, final_norm, lm_head = small_model(1)
    maxlen, P, G = 64, 9, 8
    packed = {"embed": embed, "final_norm": final_norm, "lm_head": lm_head}
    for L in range(d.L):
        packed.update(M.pack_layer(d, L, layers[L]))
    prog = M.MlaProgram(d, M.to_device(d, packed, maxlen, DEV), device=0, maxlen=maxlen)
    prompt = np.random.default_rng(5).integers(0, d.V, P)
    want_tok, want_logits, want_hidden, trace = oracle_decode(d, layers, embed, final_norm, lm_head, prompt, G, maxlen)
    got = prog.generate(prompt, G).tolist()
    # teacher forcing: the oracle's tokens as input, state compared at the last position
    forced = list(prompt) + want_tok[:-1]
    prog2_tok = prog.generate(forced, 1).tolist()
    hid, lg, ids, wts = prog.read("resid"), prog.read("logits"), prog.read("ti"), prog.read("tw")
    ckv = prog.read("ckv")
    prog.close()
    eh = np.abs(hid - want_hidden[-1]).max() / np.abs(want_hidden[-1]).max()
    el = np.abs(lg - want_logits[-1]).max() / np.abs(want_logits[-1]).max()
    print(f"mla small model: hidden err {eh:.4f}, logits err {el:.4f} of scale; tokens {got} vs {want_tok}")
    assert eh <= BF16_REL and el <= BF16_REL
    assert ids[d.TOPK:].tolist() == [d.E, d.E + 1] and np.all(wts[d.TOPK:] == 1.0)
    if sorted(ids[:d.TOPK].tolist()) == sorted(trace["ids"].tolist()):
        order = np.argsort(ids[:d.TOPK]); worder = np.argsort(trace["ids"])
        assert np.all(np.abs(wts[:d.TOPK][order] - trace["wts"][worder]) <= BF16_REL * np.abs(trace["wts"]).max())
    assert np.isfinite(ckv).all() and np.abs(ckv[:, :len(forced)]).max() > 0 and not ckv[:, len(forced):].any()
    for i, (a, b) in enumerate(zip(got, want_tok)):
        if a != b:
            lgi = want_logits[i]
            assert abs(lgi[a] - lgi[b]) <= 4 * abs(lgi[b]) * 2.0 ** -7, f"token {i}: {a} vs {b}, margin {lgi[b] - lgi[a]}"
            break                                              # after a near-tie split the sequences differ legitimately
    assert prog2_tok[0] == want_tok[-1] or abs(want_logits[-1][prog2_tok[0]] - want_logits[-1][want_tok[-1]]) <= 4 * abs(want_logits[-1][want_tok[-1]]) * 2.0 ** -7


def test_blocks_outside_the_tile_are_refused():
    from etx_megakernel_b200.runtime.lib import EtxbError
    t = torch.zeros(64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(ValueError, match="mla_attn"):
        argblock.pack_named(ENT["mla_attn"], (2, 1, 1), qkv=t.data_ptr(), kvln=t.data_ptr(), cos_sin=t.data_ptr(), wkvb=t.data_ptr(), cache=t.data_ptr(),
                            positions=t.data_ptr(), out=t.data_ptr(), NH=2, C=1024, DN=128, DR=64, DV=128, maxlen=64, scale=0.1, eps=1e-6, tmp=t.data_ptr(), max_parts=1, tag=0)
    good = argblock.pack_named(ENT["mla_attn"], (2 * 5, 1, 1), qkv=t.data_ptr(), kvln=t.data_ptr(), cos_sin=t.data_ptr(), wkvb=t.data_ptr(), cache=t.data_ptr(),
                               positions=t.data_ptr(), out=t.data_ptr(), NH=2, C=512, DN=128, DR=64, DV=128, maxlen=64, scale=0.1, eps=1e-6, tmp=t.data_ptr(), max_parts=1, tag=0)
    bad = bytearray(good)
    bad[60:64] = (2048).to_bytes(4, "little")                 # C beyond the tile's shared-memory layout, patched past the Python check
    with pytest.raises(EtxbError, match="mla_attn"):
        op_launch("mla_attn", bytes(bad), 2 * 5)
