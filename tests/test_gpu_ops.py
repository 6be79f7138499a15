"""Parity of the single tiles against the CPU oracle, through the C ABI (etxb_op_launch with the tiles' own
argument blocks).  Integer / index work is compared bit for bit, bf16 vectors within the tolerance stated per test."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200 import ops  # noqa: E402
from etx_megakernel_b200.importer import argblock  # noqa: E402
from etx_megakernel_b200.models import qwen as Q  # noqa: E402
from etx_megakernel_b200.runtime import op_launch  # noqa: E402
from oracle import ref_decode as O  # noqa: E402
from oracle import topk_wave as TW  # noqa: E402

ENT = ops.all_entries()
DEV = "cuda:0"
BF16_REL = 2e-2          # north-star tolerance for bf16 vectors (max relative error, fp32 accumulation)


def dev_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(O.f32_to_bf16_bits(a)).view(np.int16)).to(DEV).view(torch.bfloat16)


def host(t):
    torch.cuda.synchronize()
    return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()


def assert_bf16_close(got, want, what, min_exact=0.98, per_element=True):
    """max |got - want| <= BF16_REL * max|want| (the reference's own check uses 2 bf16 ulps with a floor of scale/4096,
    examples/vllm_llm/host.hip:954-1141), and nearly every element identical: only fp32 summation order differs."""
    scale = float(np.max(np.abs(want))) or 1.0
    err = float(np.max(np.abs(got - want)))
    assert err <= BF16_REL * scale, f"{what}: max abs err {err} vs scale {scale}"
    ulp = np.maximum(np.abs(want) * 2.0 ** -7, scale / 4096)
    if per_element:
        assert np.all(np.abs(got - want) <= 2 * ulp + 1e-30), f"{what}: an element is off by more than 2 bf16 ulps"
    exact = float(np.mean(got == want))
    assert exact >= min_exact, f"{what}: only {exact:.4f} of the elements are bit-identical"


def gemv_case(M, K, N, seed, tasks=148):
    rng = np.random.default_rng(seed)
    W = O.bfr(rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))
    x = O.bfr(rng.standard_normal((M, K), dtype=np.float32))
    Wd, xd = dev_bf16(W), dev_bf16(x)
    out = torch.zeros((M, N), dtype=torch.bfloat16, device=DEV)
    rpt = -(-N // tasks)
    t = -(-N // rpt)
    blob = argblock.pack_named(ENT["dsl_gemv"], (t, 1, 1), W=Wd.data_ptr(), x=xd.data_ptr(), out=out.data_ptr(), M=N, K=K, rpt=rpt,
                               tpe=1, nb=M, sx=K, sout=N)
    op_launch("gemv", blob, t)
    return host(out), O.gemv(W, x)


@pytest.mark.parametrize("M,K,N", [(1, 256, 64), (1, 2048, 128), (2, 1024, 300), (1, 768, 2048), (4, 4096, 1024), (8, 4096, 1536),
                                   (1, 1408, 100), (1, 12288, 512)])
def test_gemv_small_shapes(M, K, N):
    got, want = gemv_case(M, K, N, seed=1)
    assert_bf16_close(got, want, f"gemv M={M} K={K} N={N}")


@pytest.mark.parametrize("M", [1, 2, 4, 8])
def test_gemv_sweep_shape(M):
    """BASELINE config 2: K = 4096 -> N = 12288, M tokens, seed 1."""
    got, want = gemv_case(M, 4096, 12288, seed=1)
    assert_bf16_close(got, want, f"sweep M={M}")


def test_gemv_transposed_sweep_shape():
    got, want = gemv_case(1, 12288, 4096, seed=1)
    assert_bf16_close(got, want, "sweep K=12288")


def test_gemv_is_deterministic_and_linear():
    """Size-independent properties at the lm_head shape: same bits on a rerun; W.(2x) == 2 (W.x) exactly in bf16."""
    rng = np.random.default_rng(1)
    N, K = 151936, 4096
    Wd = torch.empty((N, K), dtype=torch.bfloat16, device=DEV).normal_(0, 0.02)
    x = O.bfr(rng.standard_normal((1, K), dtype=np.float32))
    outs = []
    for xx in (x, x, 2 * x):
        xd = dev_bf16(xx)
        out = torch.zeros((1, N), dtype=torch.bfloat16, device=DEV)
        rpt = -(-N // 592)
        t = -(-N // rpt)
        op_launch("gemv", argblock.pack_named(ENT["dsl_gemv"], (t, 1, 1), W=Wd.data_ptr(), x=xd.data_ptr(), out=out.data_ptr(),
                                              M=N, K=K, rpt=rpt, tpe=1, nb=1, sx=K, sout=N), t)
        outs.append(host(out))
    assert np.array_equal(outs[0], outs[1])
    assert np.array_equal(2 * outs[0], outs[2])
    ref = host(Wd[:4096].float() @ torch.from_numpy(x[0]).to(DEV))
    assert_bf16_close(outs[0][0, :4096], O.bfr(ref), "lm_head rows vs torch fp32", min_exact=0.95)


@pytest.mark.parametrize("R,K", [(0, 2048), (1, 2048), (8, 2048), (4, 512), (8, 4096), (1, 1408)])
def test_norm_fold_is_bit_exact(R, K):
    """x = rmsnorm(bf16(resid + rows added in bf16 in ascending expert id)): every value identical to the oracle for
    K = 128 * 2^j (numpy's summation order is reproduced), within 1 ulp otherwise."""
    rng = np.random.default_rng(R * 100 + K)
    resid = O.bfr(rng.standard_normal(K, dtype=np.float32))
    rows = O.bfr(rng.standard_normal((max(R, 1), K), dtype=np.float32) * np.float32(0.3))
    ln = O.bfr(1 + 0.1 * rng.standard_normal(K, dtype=np.float32))
    ids = rng.permutation(64)[:max(R, 1)].astype(np.int32)
    Wm = O.bfr(rng.standard_normal((32, K), dtype=np.float32) * np.float32(0.02))
    acc = np.float32(0)
    for s in np.argsort(ids)[:R]:
        acc = O.bfr(acc + rows[s])
    z = O.bfr(resid + acc) if R else resid
    xs = O.rmsnorm(z, ln, 1e-6)
    d = {k: dev_bf16(v) for k, v in dict(resid=resid, rows=rows, ln=ln, W=Wm).items()}
    idd = torch.from_numpy(ids).to(DEV)
    rout = torch.zeros(K, dtype=torch.bfloat16, device=DEV)
    xout = torch.zeros(K, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(32, dtype=torch.bfloat16, device=DEV)
    blob = argblock.pack_named(ENT["dsl_gemv_fold"], (4, 1, 1), W=d["W"].data_ptr(), x=xout.data_ptr(), out=out.data_ptr(), M=32, K=K,
                               rpt=8, tpe=1, rows=d["rows"].data_ptr() if R else 0, resid_in=d["resid"].data_ptr(), resid_out=rout.data_ptr(),
                               ln=d["ln"].data_ptr(), R=R, eps=1e-6, ids=idd.data_ptr() if R > 1 else 0, mode=1, nb=1)
    op_launch("gemv", blob, 4)
    assert np.array_equal(host(rout), z)
    pow2 = K >= 128 and K & (K - 1) == 0
    if pow2:
        assert np.array_equal(host(xout), xs)
    else:
        assert_bf16_close(host(xout), xs, "normed x")
    assert_bf16_close(host(out), O.bfr(Wm @ xs), "folded gemv", min_exact=0.9)


def test_topk_against_reference_rows(golden_dir):
    """Golden rows produced by the reference's bit-level model (etx/ops/topk_key32.py ref_topk): ids exact (NaN-free
    rows), weights within 2e-6 relative (device expf and a 32-lane butterfly instead of numpy exp and 64 lanes)."""
    g = np.load(golden_dir / "topk_rows.npz")
    for row, (E, K, renorm), ids, wts in zip(g["rows"], g["meta"], g["ids"], g["wts"]):
        E, K = int(E), int(K)
        lg = torch.from_numpy(row[:E].astype(np.uint16).view(np.int16)).to(DEV).view(torch.bfloat16)
        w = torch.zeros(16, dtype=torch.float32, device=DEV); i = torch.zeros(16, dtype=torch.int32, device=DEV)
        te = torch.zeros(16, dtype=torch.int32, device=DEV)
        blob = argblock.pack_named(ENT["dsl_topk"], (1, 1, 1), logits=lg.data_ptr(), wts=w.data_ptr(), ids=i.data_ptr(), tei=te.data_ptr(),
                                   E=E, K=K, mode=int(renorm), nbsv=0)
        op_launch("topk", blob, 1)
        assert host(i)[:K].tolist() == ids[:K].tolist()
        assert host(te)[:K].tolist() == list(range(K))
        np.testing.assert_allclose(host(w)[:K], wts[:K], rtol=4e-6, atol=1e-30)


def test_topk_matches_decode_oracle_with_bf16_weights():
    rng = np.random.default_rng(2)
    for _ in range(20):
        bits = TW.bf16_bits(rng.normal(0, 1, 128).astype(np.float32))
        ids, wts = O.softmax_topk(TW.bf16_to_f32(bits), 8, True)
        lg = torch.from_numpy(bits.view(np.int16)).to(DEV).view(torch.bfloat16)
        w = torch.zeros(8, dtype=torch.float32, device=DEV); i = torch.zeros(8, dtype=torch.int32, device=DEV)
        blob = argblock.pack_named(ENT["dsl_topk"], (1, 1, 1), logits=lg.data_ptr(), wts=w.data_ptr(), ids=i.data_ptr(), tei=0,
                                   E=128, K=8, mode=1 | 0x100, nbsv=0)
        op_launch("topk", blob, 1)
        assert host(i).tolist() == ids.tolist()
        gw = host(w)
        assert np.all(np.abs(gw - wts) <= np.abs(wts) * 2.0 ** -7)          # at most one bf16 ulp (expf vs numpy exp)
        assert np.mean(gw == wts) >= 0.5                                    # and mostly the very same bf16 value


@pytest.mark.parametrize("NH,NKV,HD,qk_norm", [(32, 4, 128, True), (8, 2, 128, True), (4, 2, 64, False), (32, 8, 128, True)])
def test_attnprep_bit_exact(NH, NKV, HD, qk_norm):
    """q / k norm + rope and the cache slot writes: integer addressing and every bf16 value identical to the oracle."""
    rng = np.random.default_rng(NH + HD)
    maxlen, pos = 80, 37
    nblk = -(-maxlen // 16)
    qkv = O.bfr(rng.standard_normal((NH + 2 * NKV, HD), dtype=np.float32))
    qn = O.bfr(1 + 0.1 * rng.standard_normal(HD, dtype=np.float32)); kn = O.bfr(1 + 0.1 * rng.standard_normal(HD, dtype=np.float32))
    cos, sin = O.rope_tables(1e6, HD, maxlen)
    q, k, v = qkv[:NH], qkv[NH:NH + NKV], qkv[NH + NKV:]
    if qk_norm:
        q = np.stack([O.rmsnorm(h, qn, 1e-6) for h in q]); k = np.stack([O.rmsnorm(h, kn, 1e-6) for h in k])
    q = np.stack([O.apply_rope(h, cos[pos], sin[pos]) for h in q]); k = np.stack([O.apply_rope(h, cos[pos], sin[pos]) for h in k])
    ks, vs = O.paged_shapes(nblk, NKV, HD)
    kc_ref = np.full(ks, 7.0, np.float32); vc_ref = np.full(vs, 7.0, np.float32)
    O.paged_write(kc_ref, vc_ref, k, v, pos)
    d_qkv = dev_bf16(qkv); d_qn, d_kn = dev_bf16(qn), dev_bf16(kn)
    cs = torch.from_numpy(Q.rope_table(1e6, HD, maxlen).view(np.int16)).to(DEV).view(torch.bfloat16)
    kc = torch.full(ks, 7.0, dtype=torch.bfloat16, device=DEV); vc = torch.full(vs, 7.0, dtype=torch.bfloat16, device=DEV)
    p64 = torch.tensor([pos], dtype=torch.int64, device=DEV)
    blob = argblock.pack_named(ENT["dsl_attnprep"], (NKV, 1, 1), qkv=d_qkv.data_ptr(), qw=d_qn.data_ptr() if qk_norm else 0,
                               kw=d_kn.data_ptr() if qk_norm else 0, cos_sin=cs.data_ptr(), positions=p64.data_ptr(), kc=kc.data_ptr(),
                               vc=vc.data_ptr(), slot_mapping=p64.data_ptr(), NH=NH, NKV=NKV, HD=HD, eps=1e-6, BS=16, X=8)
    op_launch("attnprep", blob, NKV)
    out = host(d_qkv)
    assert np.array_equal(out[:NH], q) and np.array_equal(out[NH:NH + NKV], k) and np.array_equal(out[NH + NKV:], v)
    assert np.array_equal(host(kc), kc_ref) and np.array_equal(host(vc), vc_ref)      # the slot and nothing else


@pytest.mark.parametrize("NH,NKV,HD,seq", [(32, 4, 128, 1025), (8, 2, 128, 1), (8, 2, 128, 33), (4, 2, 64, 100), (32, 8, 128, 640)])
def test_paged_attention(NH, NKV, HD, seq):
    rng = np.random.default_rng(seq)
    G = NH // NKV
    maxlen = ((seq + 31) // 32) * 32 + 32
    nblk, parts = maxlen // 16, maxlen // 32
    K = O.bfr(rng.standard_normal((seq, NKV, HD), dtype=np.float32) * np.float32(0.5))
    V = O.bfr(rng.standard_normal((seq, NKV, HD), dtype=np.float32))
    q = O.bfr(rng.standard_normal((NH, HD), dtype=np.float32))
    scale = np.float32(1.0 / np.sqrt(HD))
    want = np.zeros((NH, HD), np.float32)
    for h in range(NH):
        s = (K[:, h // G] @ q[h]) * scale
        s = s - s.max(); pr = np.exp(s); pr = pr / pr.sum()
        want[h] = O.bfr(pr @ V[:, h // G])
    kc, vc = O.paged_from_contig(K, V, nblk)
    perm = rng.permutation(nblk).astype(np.int32)                         # a non-identity block table
    kcp, vcp = np.zeros_like(kc), np.zeros_like(vc)
    kcp[perm] = kc; vcp[perm] = vc
    d_kc, d_vc, d_q = dev_bf16(kcp), dev_bf16(vcp), dev_bf16(q)
    bt = torch.from_numpy(perm).to(DEV); sl = torch.tensor([seq], dtype=torch.int32, device=DEV)
    es = torch.zeros((NH, parts), dtype=torch.float32, device=DEV); ml = torch.zeros_like(es)
    tmp = torch.zeros((NH, parts, HD), dtype=torch.float32, device=DEV); out = torch.zeros((NH, HD), dtype=torch.bfloat16, device=DEV)
    common = dict(q=d_q.data_ptr(), kc=d_kc.data_ptr(), vc=d_vc.data_ptr(), block_tables=bt.data_ptr(), seq_lens=sl.data_ptr(),
                  exp_sums=es.data_ptr(), max_logits=ml.data_ptr(), tmp_out=tmp.data_ptr(), out=out.data_ptr(), scale=float(scale),
                  NH=NH, NKV=NKV, HD=HD, BS=16, X=8, max_parts=parts, max_blocks=nblk)
    op_launch("attn", argblock.pack_named(ENT["attn_decode"], (parts * NKV, 1, 1), **common), parts * NKV)
    op_launch("attn_reduce", argblock.pack_named(ENT["attn_reduce"], (NH, 1, 1), **common), NH)
    assert_bf16_close(host(out), want, f"attention seq={seq}", min_exact=0.9)


@pytest.mark.parametrize("NH,NKV,HD,qk_norm,seq,gq", [
    (32, 4, 128, True, 1025, 0), (32, 4, 128, True, 1024, 0), (8, 2, 128, True, 1, 0), (8, 2, 128, True, 33, 0), (4, 2, 64, False, 100, 0),
    (32, 8, 128, True, 640, 0), (16, 2, 128, True, 97, 0),
    # the grouped form: gq q heads x 128 positions per task
    (32, 4, 128, True, 1025, 2), (32, 4, 128, True, 1024, 2), (32, 4, 128, True, 1041, 8), (8, 2, 128, True, 1, 1), (8, 2, 128, True, 129, 4),
    (32, 8, 128, False, 640, 2), (32, 8, 128, True, 128, 4), (16, 2, 128, True, 257, 8), (4, 4, 128, True, 77, 1)])
def test_attention_phase_fused(NH, NKV, HD, qk_norm, seq, gq):
    """The one-phase attention tile (norm + rope + cache write of the new position, split-KV attention, merge) against the
    oracle, in its general form (merge by the last task to finish) and its grouped form (merge by the last partition's
    task over flagged partials): new cache slot bit-exact, output within bf16 tolerance; run twice on the same buffers to
    cover the modulo arithmetic of the election counters and the step flags of the partials."""
    rng = np.random.default_rng(seq + NH)
    G = NH // NKV
    pos = seq - 1
    plen = 128 if gq else 32
    maxlen = ((seq + plen - 1) // plen) * plen + plen
    nblk, parts = maxlen // 16, maxlen // plen
    ntask, ncnt = (parts * (NH // gq), NH // gq) if gq else (parts * NKV, NKV)
    K = O.bfr(rng.standard_normal((seq, NKV, HD), dtype=np.float32) * np.float32(0.5))
    V = O.bfr(rng.standard_normal((seq, NKV, HD), dtype=np.float32))
    qkv = O.bfr(rng.standard_normal((NH + 2 * NKV, HD), dtype=np.float32))
    qn = O.bfr(1 + 0.1 * rng.standard_normal(HD, dtype=np.float32)); kn = O.bfr(1 + 0.1 * rng.standard_normal(HD, dtype=np.float32))
    cos, sin = O.rope_tables(1e6, HD, maxlen)
    q, k, v = qkv[:NH], qkv[NH:NH + NKV], qkv[NH + NKV:]
    if qk_norm:
        q = np.stack([O.rmsnorm(h, qn, 1e-6) for h in q]); k = np.stack([O.rmsnorm(h, kn, 1e-6) for h in k])
    q = np.stack([O.apply_rope(h, cos[pos], sin[pos]) for h in q]); k = np.stack([O.apply_rope(h, cos[pos], sin[pos]) for h in k])
    K[pos], V[pos] = k, v
    scale = np.float32(1.0 / np.sqrt(HD))
    want = np.zeros((NH, HD), np.float32)
    for h in range(NH):
        s = (K[:, h // G] @ q[h]) * scale
        s = s - s.max(); pr = np.exp(s); pr = pr / pr.sum()
        want[h] = O.bfr(pr @ V[:, h // G])
    Kold, Vold = K.copy(), V.copy()
    Kold[pos], Vold[pos] = 9.0, 9.0                                       # stale slot contents the tile must overwrite
    kc0, vc0 = O.paged_from_contig(Kold, Vold, nblk)
    kc_ref, vc_ref = O.paged_from_contig(K, V, nblk)
    d_kc, d_vc, d_qkv = dev_bf16(kc0), dev_bf16(vc0), dev_bf16(qkv)
    d_qn, d_kn = dev_bf16(qn), dev_bf16(kn)
    cs = torch.from_numpy(Q.rope_table(1e6, HD, maxlen).view(np.int16)).to(DEV).view(torch.bfloat16)
    bt = torch.arange(nblk, dtype=torch.int32, device=DEV); sl = torch.tensor([seq], dtype=torch.int32, device=DEV)
    p64 = torch.tensor([pos], dtype=torch.int64, device=DEV)
    es = torch.zeros((NH, parts), dtype=torch.float32, device=DEV); ml = torch.zeros_like(es)
    tmp = torch.zeros((NH, parts, ops.attn.GQ_PARTIAL_FLOATS if gq else HD), dtype=torch.float32, device=DEV)
    out = torch.zeros((NH, HD), dtype=torch.bfloat16, device=DEV)
    cnt = torch.zeros(ncnt, dtype=torch.int32, device=DEV)
    blob = argblock.pack_named(ENT["attn_fused"], (ntask, 1, 1), qkv=d_qkv.data_ptr(), qw=d_qn.data_ptr() if qk_norm else 0,
                               kw=d_kn.data_ptr() if qk_norm else 0, cos_sin=cs.data_ptr(), kc=d_kc.data_ptr(), vc=d_vc.data_ptr(),
                               block_tables=bt.data_ptr(), seq_lens=sl.data_ptr(), positions=p64.data_ptr(), slot_mapping=p64.data_ptr(),
                               exp_sums=es.data_ptr(), max_logits=ml.data_ptr(), tmp_out=tmp.data_ptr(), out=out.data_ptr(),
                               counters=cnt.data_ptr(), scale=float(scale), eps=1e-6, NH=NH, NKV=NKV, HD=HD, BS=16, X=8, max_parts=parts,
                               gq=gq, part_len=plen if gq else 0)
    for rerun in range(2):
        out.zero_()
        op_launch("attn_fused", blob, ntask)
        assert np.array_equal(host(d_kc), kc_ref) and np.array_equal(host(d_vc), vc_ref)
        assert_bf16_close(host(out), want, f"fused attention seq={seq} run {rerun}", min_exact=0.9)
        assert host(cnt).tolist() == [0 if gq else parts * (rerun + 1)] * ncnt        # (the grouped form elects nobody: its merger is fixed)
        assert np.array_equal(host(d_qkv), qkv)                          # the fused tile leaves qkv as the GEMV wrote it


@pytest.mark.parametrize("E,TOPK,MI,H,fold", [(16, 4, 128, 512, True), (128, 8, 768, 2048, True), (128, 8, 768, 2048, False), (8, 2, 256, 256, True)])
def test_moe_block(E, TOPK, MI, H, fold):
    """router logits -> top-k -> gate/up with SiLU*mul -> down scaled by the bf16 routing weight, against the oracle's
    MoE block (examples/llm/ref_numpy.py:133-148).  Routing ids bit-exact."""
    rng = np.random.default_rng(E + MI)
    xs = O.bfr(rng.standard_normal(H, dtype=np.float32))
    logits = O.bfr(rng.standard_normal(E, dtype=np.float32))
    w13 = O.bfr(rng.standard_normal((E, 2 * MI, H), dtype=np.float32) * np.float32(0.02))
    w2 = O.bfr(rng.standard_normal((E, H, MI), dtype=np.float32) * np.float32(0.02))
    ids, wts = O.softmax_topk(logits, TOPK, True)
    act_ref = np.zeros((TOPK, MI), np.float32); y_ref = np.zeros((TOPK, H), np.float32)
    for s, (e, we) in enumerate(zip(ids.tolist(), wts.tolist())):
        g = O.bfr(w13[e, :MI] @ xs); u = O.bfr(w13[e, MI:] @ xs)
        act_ref[s] = O.bfr(O.bfr(O.silu(g)) * u)
        y_ref[s] = O.bfr(O.bfr(w2[e] @ act_ref[s]) * np.float32(we))
    d_x, d_lg, d_w13, d_w2 = dev_bf16(xs), dev_bf16(logits), dev_bf16(w13), dev_bf16(w2)
    ti = torch.zeros(TOPK, dtype=torch.int32, device=DEV); tw = torch.zeros(TOPK, dtype=torch.float32, device=DEV)
    act = torch.zeros((TOPK, MI), dtype=torch.bfloat16, device=DEV); y = torch.zeros((TOPK, H), dtype=torch.bfloat16, device=DEV)
    if not fold:
        op_launch("topk", argblock.pack_named(ENT["dsl_topk"], (1, 1, 1), logits=d_lg.data_ptr(), wts=tw.data_ptr(), ids=ti.data_ptr(), tei=0,
                                              E=E, K=TOPK, mode=1 | 0x100, nbsv=0), 1)
    tpe = 5
    rpt = -(-MI // tpe)
    up = argblock.pack_named(ENT["dsl_moe_up_fold" if fold else "dsl_moe_up"], (TOPK * tpe, 1, 1), W=d_w13.data_ptr(), x=d_x.data_ptr(),
                             out=act.data_ptr(), ids=ti.data_ptr(), wts=tw.data_ptr(), estride=2 * MI * H, M=MI, K=H, rpt=rpt, tpe=tpe,
                             R=TOPK, mode=(3 | 0x100) if fold else 0, E=E, logits=d_lg.data_ptr(), nb=1)
    op_launch("moe_up", up, TOPK * tpe)
    rpt2 = -(-H // tpe)
    dn = argblock.pack_named(ENT["dsl_moe_down"], (TOPK * tpe, 1, 1), W=d_w2.data_ptr(), x=act.data_ptr(), out=y.data_ptr(), ids=ti.data_ptr(),
                             wts=tw.data_ptr(), estride=H * MI, M=H, K=MI, rpt=rpt2, tpe=tpe, R=TOPK, nb=1)
    op_launch("moe_down", dn, TOPK * tpe)
    assert host(ti).tolist() == ids.tolist()
    assert np.all(np.abs(host(tw) - wts) <= np.abs(wts) * 2.0 ** -7)
    assert_bf16_close(host(act), act_ref, "moe_up act", min_exact=0.97)
    assert_bf16_close(host(y), y_ref, "moe_down y", min_exact=0.95)


@pytest.mark.parametrize("E,TOPK,MI,H,spt", [(128, 8, 768, 2048, 2), (16, 4, 128, 512, 4), (128, 8, 768, 2048, 8), (64, 6, 1408, 2048, 3)])
def test_moe_block_grouped_slots_and_summed_down(E, TOPK, MI, H, spt):
    """Several expert slots per gate+up task, and the down form that covers every slot and writes the expert combine
    (bf16 adds in ascending expert id, examples/llm/ref_numpy.py:142-148) instead of one row per slot."""
    rng = np.random.default_rng(E * 7 + spt)
    xs = O.bfr(rng.standard_normal(H, dtype=np.float32))
    logits = O.bfr(rng.standard_normal(E, dtype=np.float32))
    w13 = O.bfr(rng.standard_normal((E, 2 * MI, H), dtype=np.float32) * np.float32(0.02))
    w2 = O.bfr(rng.standard_normal((E, H, MI), dtype=np.float32) * np.float32(0.02))
    ids, wts = O.softmax_topk(logits, TOPK, True)
    act_ref = np.zeros((TOPK, MI), np.float32)
    acc = np.float32(0)
    ys = {}
    for s, (e, we) in enumerate(zip(ids.tolist(), wts.tolist())):
        g = O.bfr(w13[e, :MI] @ xs); u = O.bfr(w13[e, MI:] @ xs)
        act_ref[s] = O.bfr(O.bfr(O.silu(g)) * u)
        ys[e] = O.bfr(O.bfr(w2[e] @ act_ref[s]) * np.float32(we))
    for e in sorted(ys):
        acc = O.bfr(acc + ys[e])
    d_x, d_lg, d_w13, d_w2 = dev_bf16(xs), dev_bf16(logits), dev_bf16(w13), dev_bf16(w2)
    ti = torch.zeros(TOPK, dtype=torch.int32, device=DEV); tw = torch.zeros(TOPK, dtype=torch.float32, device=DEV)
    act = torch.zeros((TOPK, MI), dtype=torch.bfloat16, device=DEV); out = torch.zeros(H, dtype=torch.bfloat16, device=DEV)
    tpe = 7
    rpt = -(-MI // tpe); tpe = -(-MI // rpt)
    groups = TOPK // spt
    mode = (3 | 0x100) | (spt << 16)
    up = argblock.pack_named(ENT["dsl_moe_up_fold"], (groups * tpe, 1, 1), W=d_w13.data_ptr(), x=d_x.data_ptr(), out=act.data_ptr(), ids=ti.data_ptr(),
                             wts=tw.data_ptr(), estride=2 * MI * H, M=MI, K=H, rpt=rpt, tpe=tpe, R=TOPK, mode=mode, E=E, logits=d_lg.data_ptr(), nb=1)
    op_launch("moe_up", up, groups * tpe)
    tpe2 = 9
    rpt2 = -(-H // tpe2); tpe2 = -(-H // rpt2)
    dn = argblock.pack_named(ENT["dsl_moe_down_fold"], (tpe2, 1, 1), W=d_w2.data_ptr(), x=act.data_ptr(), out=out.data_ptr(), ids=ti.data_ptr(),
                             wts=tw.data_ptr(), estride=H * MI, M=H, K=MI, rpt=rpt2, tpe=tpe2, R=TOPK, mode=(3 | 0x100) | (TOPK << 16) | 0x400,
                             E=E, logits=d_lg.data_ptr(), nb=1)
    op_launch("moe_down", dn, tpe2)
    assert host(ti).tolist() == ids.tolist()
    assert_bf16_close(host(act), act_ref, "grouped moe_up act", min_exact=0.97)
    # a sum of eight rounded terms can cancel: the 2-ulp bound is relative to the terms, not to the (smaller) sum
    assert_bf16_close(host(out), acc, "summed moe_down", min_exact=0.9, per_element=False)
    assert np.all(np.abs(host(out) - acc) <= 4 * 2.0 ** -8 * max(np.abs(y).max() for y in ys.values()))


def test_argument_block_rejected_before_launch():
    with pytest.raises(ValueError):
        argblock.pack_named(ENT["dsl_gemv"], (4, 1, 1), W=1, x=2, out=3, M=64, K=100, rpt=16, nb=1)     # K % 8
    with pytest.raises(ValueError):
        argblock.pack_named(ENT["dsl_gemv"], (2, 1, 1), W=1, x=2, out=3, M=64, K=128, rpt=16, nb=1)     # rows left unwritten
    with pytest.raises(ValueError):
        argblock.pack_named(ENT["dsl_gemv"], (4, 1, 1), W=1, x=2, out=3, M=64, K=128, rpt=16, nb=3)     # unsupported column count


# ------------------------------------------------------------------------------------------------ argument-block limits, NaN rows, protocol demo
@pytest.mark.parametrize("bad", [dict(K=12296), dict(K=0), dict(K=2044), dict(rpt=0), dict(mode=1, K=8200), dict(mode=2, E=300, R=8), dict(mode=0x30000, rpt=1024)])
def test_blocks_outside_the_tile_limits_are_refused_before_launch(bad):
    """A GEMV-family block a device loop could not get through (a row longer than a ring stage, a zero row length, more
    results than the tile holds ...) never reaches the GPU: the C entry point answers E_UNSUPPORTED from its host-side
    check.  Nothing is launched, so the test needs no valid pointers."""
    import struct
    from etx_megakernel_b200.runtime import EtxbError
    f = dict(W=4096, x=4096, out=4096, M=64, K=2048, rpt=1, tpe=64, nb=1, mode=0, E=0, R=0, logits=4096)
    body = "moe_up" if bad.get("mode", 0) & 0xff0000 else "gemv"
    blob = bytearray(argblock.pack_named(ENT["dsl_moe_up" if body == "moe_up" else "dsl_gemv"], (64, 1, 1), **f))
    # the Python packer has its own guard (ops.gemv.check_shape), so the out-of-range values are patched into the packed
    # bytes: what a C or C++ host that fills the 160-byte block by hand could pass
    offsets = {name: off for name, _, off, _ in ops.gemv.PARAMS}
    for name, value in bad.items():
        struct.pack_into("<i", blob, offsets[name], value)
    with pytest.raises(EtxbError) as e:
        op_launch(body, bytes(blob), 64)
    assert e.value.status == "E_UNSUPPORTED" and "outside the tile" in str(e.value)
    fa = dict(qkv=4096, cos_sin=4096, kc=4096, vc=4096, block_tables=4096, seq_lens=4096, positions=4096, slot_mapping=4096, exp_sums=4096,
              max_logits=4096, tmp_out=4096, out=4096, counters=4096, scale=1.0, eps=1e-6, NH=32, NKV=4, HD=128, BS=16, X=8, max_parts=9,
              gq=2, part_len=128)
    ablob = bytearray(argblock.pack_named(ENT["attn_fused"], (9 * 16, 1, 1), **fa))
    struct.pack_into("<i", ablob, 152, 3)                                   # gq = 3 does not divide the 8 q heads of a kv head
    with pytest.raises(EtxbError) as e:
        op_launch("attn_fused", bytes(ablob), 144)
    assert e.value.status == "E_UNSUPPORTED"
    assert torch.zeros(2, device=DEV).sum().item() == 0.0


def test_topk_rows_with_nan_follow_the_reference_model(golden_dir):
    """Rows with NaN logits as the reference's model of its wave path pins them (etx/ops/topk_key32.py ref_topk; the
    rows were produced by it): every probability is NaN, no round finds a candidate, so every id is 0x7fffffff and every
    weight -1 (renormalised: 1 / K)."""
    g = np.load(golden_dir / "topk_rows.npz")
    nan_rows = [n for n, row in enumerate(g["rows"]) if np.isnan(TW.bf16_to_f32(row[:g["meta"][n][0]])).any()]
    assert nan_rows, "the fixture holds rows with NaN logits"
    for n in nan_rows:
        E, K, renorm = (int(v) for v in g["meta"][n])
        lg = torch.from_numpy(g["rows"][n].view(np.int16)).to(DEV).view(torch.bfloat16)
        w = torch.zeros(16, dtype=torch.float32, device=DEV); i = torch.zeros(16, dtype=torch.int32, device=DEV)
        blob = argblock.pack_named(ENT["dsl_topk"], (1, 1, 1), logits=lg.data_ptr(), wts=w.data_ptr(), ids=i.data_ptr(), tei=0,
                                   E=E, K=K, mode=renorm, nbsv=0)
        op_launch("topk", blob, 1)
        assert host(i)[:K].tolist() == g["ids"][n][:K].tolist() == [0x7FFFFFFF] * K
        np.testing.assert_allclose(host(w)[:K], g["wts"][n][:K], rtol=1e-6)


def test_split_k_demo_program_runs_through_a_session():
    """The protocol demo of the reference (etx/operators/splitk_sum.py: partial sums -> per-row event -> final sum) on
    the persistent kernel: tile bodies 10 / 11 through a Session, every task exactly once, sums against numpy."""
    from etx_megakernel_b200.operators import splitk_sum as S
    from etx_megakernel_b200.passes import compile_graph
    from etx_megakernel_b200.runtime import Session
    n, cols, chunks = 96, 256, 4
    rng = np.random.default_rng(5)
    A = rng.standard_normal((n, cols)).astype(np.float32)
    a = torch.from_numpy(A).to(DEV); parts = torch.zeros((n, chunks), dtype=torch.float32, device=DEV); out = torch.zeros(n, dtype=torch.float32, device=DEV)
    g, pool = S.build_program(n, cols, chunks, a.data_ptr(), parts.data_ptr(), out.data_ptr())
    plan = compile_graph(g, "b200", {})
    s = Session(plan, {}, pool)
    s.set_option("trace", 1)
    for _ in range(2):                                                      # twice: the counters carry over from step to step
        out.zero_()
        s.run(10.0)
        assert (s.exec_counts() == 1).all() and s.status().kernel_variant == 0
        np.testing.assert_allclose(host(parts), A.reshape(n, chunks, cols // chunks).sum(-1), rtol=1e-5, atol=1e-5)
        np.testing.assert_allclose(host(out), A.sum(-1), rtol=1e-5, atol=1e-4)
    s.close()
