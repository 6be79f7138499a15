"""The oracle against the reference's own outputs (fixtures made by tests/golden/make_golden.py, which runs
examples/llm/ref_numpy.py, etx/ops/topk_key32.py and etx/bench/numerical.py of the reference unmodified)."""
import zlib

import numpy as np
import pytest

from oracle import moe_block as MB
from oracle import ref_decode as O
from oracle import topk_wave as TW
from tests.golden.cases import SMALL_DENSE, SMALL_MOE


def _crc(W):
    c = 0
    for k in sorted(W.t):
        c = zlib.crc32(np.ascontiguousarray(W.t[k]).tobytes(), c)
    return c


@pytest.mark.parametrize("dims,file,n_prompt", [(SMALL_MOE, "decode_small_moe.npz", 8), (SMALL_DENSE, "decode_small_dense.npz", 6)])
def test_decode_tokens_and_residuals_bit_exact(golden_dir, dims, file, n_prompt):
    g = np.load(golden_dir / file)
    W = O.SyntheticWeights(dims, seed=int(g["seed"]), gamma=str(g["gamma"]))
    assert _crc(W) == int(g["weights_crc"]), "synthetic weights are not the bytes the fixture was made with"
    n_gen = len(g["gen"])
    ref = O.Ref(dims, W, n_prompt + n_gen + 8)
    seq, gen, dumps = list(g["prompt"]), [], []
    for t in range(n_prompt + n_gen - 1):
        nxt = ref.step(int(seq[t]), t, dumps if t == n_prompt - 1 else None)
        if t >= n_prompt - 1:
            gen.append(nxt)
            if len(seq) <= t + 1:
                seq.append(nxt)
    assert gen == g["gen"].tolist()
    assert np.array_equal(np.stack(dumps), g["layers"])                 # same code path, same BLAS: bit-exact
    n = n_prompt + n_gen - 1
    assert np.array_equal(ref.kc[:, :n], g["kc"]) and np.array_equal(ref.vc[:, :n], g["vc"])


def test_single_layer_config_one(golden_dir):
    """BASELINE config 1 (Qwen3-30B-A3B layer, 1024 prior tokens) against the reference's output."""
    g = np.load(golden_dir / "layer_qwen3moe.npz")
    d = O.dims_from_config(O.QWEN3_30B_A3B, "qwen3-30b-a3b", layers=1)
    d.V, d.tie = 1, True
    W = O.SyntheticWeights(d, seed=0, gamma="normal")
    rng = np.random.default_rng(12345)
    S = 1024
    W.t["model.embed_tokens.weight"] = O.bfr(rng.standard_normal((1, d.H), dtype=np.float32))
    assert _crc(W) == int(g["weights_crc"])
    ref = O.Ref(d, W, S + 8)
    ref.kc[0, :S] = O.bfr(rng.standard_normal((S, d.NKV, d.HD), dtype=np.float32) * np.float32(0.02))
    ref.vc[0, :S] = O.bfr(rng.standard_normal((S, d.NKV, d.HD), dtype=np.float32) * np.float32(0.02))
    out = ref.layer(0, W.get("model.embed_tokens.weight")[0].copy(), S)
    assert np.array_equal(out, g["hidden_out"])
    assert np.array_equal(ref.kc[0, S], g["k_new"]) and np.array_equal(ref.vc[0, S], g["v_new"])


def test_wave_topk_matches_reference_model(golden_dir):
    g = np.load(golden_dir / "topk_rows.npz")
    for row, (E, K, renorm), ids, wts in zip(g["rows"], g["meta"], g["ids"], g["wts"]):
        i, w = TW.wave_topk(row[:E], int(K), bool(renorm), lanes=64)
        assert i == ids[:K].tolist()
        assert np.array_equal(np.array(w, np.float32), wts[:K], equal_nan=True)


def test_wave_topk_ids_do_not_depend_on_lane_count(golden_dir):
    g = np.load(golden_dir / "topk_rows.npz")
    for row, (E, K, renorm), ids, wts in zip(g["rows"], g["meta"], g["ids"], g["wts"]):
        i, w = TW.wave_topk(row[:E], int(K), bool(renorm), lanes=32)
        assert i == ids[:K].tolist()
        np.testing.assert_allclose(np.array(w, np.float32), wts[:K], rtol=2e-6, atol=1e-30)


def test_softmax_topk_ties_and_agreement_with_wave_model():
    rng = np.random.default_rng(11)
    for _ in range(50):
        bits = TW.bf16_bits(rng.normal(0, 1, 128).astype(np.float32))
        ids, wts = O.softmax_topk(TW.bf16_to_f32(bits), 8, True)
        wi, ww = TW.wave_topk(bits, 8, True, lanes=32)
        assert ids.tolist() == wi
        np.testing.assert_allclose(wts, O.bfr(np.array(ww, np.float32)), rtol=2 ** -7)
    ids, _ = O.softmax_topk(np.zeros(128, np.float32), 8, True)
    assert ids.tolist() == list(range(8))                               # ties -> the smallest ids


def test_moe_block_known_answers(golden_dir):
    g = np.load(golden_dir / "moe_block.npz")
    assert bool(g["suite_passed"]) and int(g["suite_cases"]) == 24
    for E, K in ((8, 2), (128, 8)):
        for renorm in (False, True):
            tag = f"E{E}K{K}R{int(renorm)}"
            data = MB.fixture(experts=E, top_k=K, renormalize=renorm)
            assert np.array_equal(data["x"], g[tag + "_x"]) and np.array_equal(data["router"], g[tag + "_router"])
            out, written, sel = MB.block_fp32(data)
            ref, ids = MB.block_scalar64(data)
            assert sel == g[tag + "_sel"].tolist() == ids == g[tag + "_ids"].tolist()
            np.testing.assert_allclose(ref, g[tag + "_scalar"], rtol=1e-12)
            np.testing.assert_allclose(out, g[tag + "_vector"], rtol=1e-6)
            assert MB.check_output(out, ref, written) == []


@pytest.mark.parametrize("renorm", [True, False])
def test_moe_block_ties_choose_smallest_id_and_faults_are_rejected(renorm):
    data = MB.fixture(renormalize=renorm)
    data["router"][:] = 0
    out, written, sel = MB.block_fp32(data)
    ref, ids = MB.block_scalar64(data)
    assert ids == sel == [0, 1] and MB.check_output(out, ref, written) == []
    for fault in ("nan", "inf", "hole", "wrong_value", "wrong_topk"):
        bad, mask = out.copy(), written.copy()
        if fault in ("nan", "inf"):
            bad[-1] = float(fault)
        elif fault == "hole":
            mask[-1] = False
        elif fault == "wrong_value":
            bad[-1] += 1
        else:
            bad, mask, _ = MB.block_fp32({**MB.fixture(renormalize=renorm), "top_k": 1})
            ref, _ = MB.block_scalar64(MB.fixture(renormalize=renorm))
        assert MB.check_output(bad, ref, mask), fault
    with pytest.raises(ValueError):
        MB.check_output([1], [2], [True], atol=float("inf"))


def test_paged_cache_layout_round_trip():
    rng = np.random.default_rng(5)
    ctx, nkv, hd = 37, 2, 128
    K = rng.standard_normal((ctx, nkv, hd)).astype(np.float32); V = rng.standard_normal((ctx, nkv, hd)).astype(np.float32)
    kc, vc = O.paged_from_contig(K, V, nblocks=4)
    assert kc.shape == (4, nkv, hd // 8, 16, 8) and vc.shape == (4, nkv, hd, 16)
    # element addressing of the reference tile: key [blk][h][d/8][off][d%8], value [blk][h][d][off]
    t, h, dd = 21, 1, 77
    assert kc[t // 16, h, dd // 8, t % 16, dd % 8] == K[t, h, dd] and vc[t // 16, h, dd, t % 16] == V[t, h, dd]
    K2, V2 = O.paged_to_contig(kc, vc, ctx)
    assert np.array_equal(K, K2) and np.array_equal(V, V2)


def test_byte_ledger_matches_reference_figures():
    """6.1845 GB per step and 115.878 MB per layer at context 1024 (docs/qwen/BANDWIDTH-2026-10-07.md:24)."""
    d = O.dims_from_config(O.QWEN3_30B_A3B)
    b = O.step_bytes(d, 1024)
    assert abs(b["layer"] / 1e6 - 115.878) < 0.01
    assert abs(b["total"] / 1e9 - 6.1845) < 0.001
    d8 = O.dims_from_config(O.QWEN3_8B)
    assert abs(O.step_bytes(d8, 1024)["total"] / 1e9 - 15.288) < 0.002


def test_mla_oracle_matches_the_reference_fixture(golden_dir):
    """oracle/ref_mla.py (absorbed MLA + DeepSeek MoE / dense layer) against outputs of the NumPy reference archived in
    the reference tree (tests/golden/make_golden.py: mla_case): layer outputs and latent cache rows bit-exact over 24
    decode positions, YaRN tables and softmax scale equal."""
    from oracle import ref_mla as M
    from tests.golden.cases import MLA_SMALL
    g = np.load(golden_dir / "mla_layer.npz")
    n = int(g["n"])
    for tag, dense in (("moe", 0), ("dense", int(g["dense_inter"]))):
        d = M.MlaDims(**MLA_SMALL, dense_inter=dense)
        L = M.synthetic_layer(d, seed=int(g["seed"]))
        cos, sin = M.yarn_tables(d, n)
        assert np.array_equal(cos.astype(np.float32), g[f"{tag}_cos"]) and np.array_equal(sin.astype(np.float32), g[f"{tag}_sin"])
        assert d.scale == float(g[f"{tag}_scale"])
        rng = np.random.default_rng(int(g["xseed"]))
        cache = np.zeros((n, d.kv_lora + d.qk_rope), np.float32)
        for pos in range(n):
            x = O.bfr(rng.standard_normal(d.hidden, dtype=np.float32))
            tr = {}
            y = M.layer(d, L, x, cache, pos, cos, sin, tr)
            assert np.array_equal(y, g[f"{tag}_y"][pos]), (tag, pos)
            if not dense:
                assert len(set(tr["ids"].tolist())) == d.top_k and abs(float(tr["wts"].sum())) <= 1.0 + 1e-6
        assert np.array_equal(cache, g[f"{tag}_cache"])
    full = M.MlaDims(**M.DSV2_LITE)
    assert full.q_head == 192 and abs(M.layer_bytes(full, 1025) - 167.38e6) / 167.38e6 < 0.01          # the reference's 167.38 MB per MoE layer
