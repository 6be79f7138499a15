#!/usr/bin/env python3
"""Generate the golden fixtures in this directory by running the REFERENCE's own CPU code.

Run where the reference checkout is available ($ETX_REFERENCE, default: a directory `reference` beside this repository):

    python tests/golden/make_golden.py

It imports, unmodified:
  examples/llm/ref_numpy.py   (Ref.step, bfr, rmsnorm, rope_tables, apply_rope)  -> decode_*.npz, layer_qwen3moe.npz
  etx/ops/topk_key32.py       (ref_topk, bf16_bits)                               -> topk_rows.npz
  etx/bench/numerical.py      (fixture, vectorized, scalar_reference)             -> moe_block.npz
and drives them with the seeded synthetic weights of oracle/ref_decode.py (weights are regenerated from the seed
by the tests, a checksum is stored).  The fixtures travel; the reference does not.
"""
from __future__ import annotations

import os
import sys
import zlib
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
REF = Path(os.environ.get("ETX_REFERENCE", str(ROOT.parent / "reference")))
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(REF))

from oracle import ref_decode as O                         # noqa: E402

from examples.llm import model as RM                       # noqa: E402  (reference)
from examples.llm import ref_numpy as RN                   # noqa: E402  (reference)
from etx.ops import topk_key32 as RTK                      # noqa: E402  (reference)
from etx.bench import numerical as RNUM                    # noqa: E402  (reference)


def ref_dims(d: O.Dims):
    return RM.Dims(name=d.name, H=d.H, NH=d.NH, NKV=d.NKV, HD=d.HD, INTER=d.INTER, L=d.L, V=d.V, eps=d.eps,
                   theta=d.theta, tie=d.tie, bias=d.bias, qk_norm=d.qk_norm, moe=d.moe, E=d.E, TOPK=d.TOPK,
                   MI=d.MI, norm_topk=d.norm_topk)


def reference_model(d: O.Dims, W, ctx: int):
    """A reference `Ref` without a checkpoint directory: __init__ wants safetensors, so build it by hand."""
    r = RN.Ref.__new__(RN.Ref)
    r.d, r.W, r.ctx = ref_dims(d), W, ctx
    r.cos, r.sin = RN.rope_tables(d.theta, d.HD, ctx)
    r.kc = np.zeros((d.L, ctx, d.NKV, d.HD), np.float32)
    r.vc = np.zeros((d.L, ctx, d.NKV, d.HD), np.float32)
    return r


def checksum(W) -> int:
    c = 0
    for k in sorted(W.t):
        c = zlib.crc32(np.ascontiguousarray(W.t[k]).tobytes(), c)
    return c


from tests.golden.cases import SMALL_DENSE, SMALL_MOE    # noqa: E402


def decode_case(d: O.Dims, seed: int, n_prompt: int, n_gen: int, gamma: str, out: str):
    W = O.SyntheticWeights(d, seed=seed, gamma=gamma)
    ctx = n_prompt + n_gen + 8
    ref = reference_model(d, W, ctx)
    rng = np.random.default_rng(seed + 1000)
    prompt = rng.integers(0, d.V, n_prompt)
    seq, gen, dumps = list(prompt), [], []
    for t in range(n_prompt + n_gen - 1):
        nxt = ref.step(int(seq[t]), t, dumps if t == n_prompt - 1 else None)
        if t >= n_prompt - 1:
            gen.append(nxt)
            if len(seq) <= t + 1:
                seq.append(nxt)
    np.savez_compressed(HERE / out, seed=seed, gamma=gamma, prompt=prompt, gen=np.array(gen), layers=np.stack(dumps),
                        kc=ref.kc[:, : n_prompt + n_gen - 1], vc=ref.vc[:, : n_prompt + n_gen - 1],
                        weights_crc=checksum(W))
    print(out, "gen", gen)


def layer_case():
    """BASELINE config 1: one Qwen3-30B-A3B-shaped layer, batch 1, 1024 prior tokens, everything N(0, 0.02) bf16
    (norm gammas too), input hidden N(0, 1), seed 0.  The input hidden rides in as the single embedding row."""
    d = O.dims_from_config(O.QWEN3_30B_A3B, "qwen3-30b-a3b", layers=1)
    d.V, d.tie = 1, True
    W = O.SyntheticWeights(d, seed=0, gamma="normal")
    rng = np.random.default_rng(12345)
    S = 1024
    W.t["model.embed_tokens.weight"] = O.bfr(rng.standard_normal((1, d.H), dtype=np.float32))
    ref = reference_model(d, W, S + 8)
    ref.kc[0, :S] = O.bfr(rng.standard_normal((S, d.NKV, d.HD), dtype=np.float32) * np.float32(0.02))
    ref.vc[0, :S] = O.bfr(rng.standard_normal((S, d.NKV, d.HD), dtype=np.float32) * np.float32(0.02))
    dumps = []
    ref.step(0, S, dumps)
    np.savez_compressed(HERE / "layer_qwen3moe.npz", hidden_in=W.t["model.embed_tokens.weight"][0], hidden_out=dumps[0],
                        k_new=ref.kc[0, S], v_new=ref.vc[0, S], weights_crc=checksum(W))
    print("layer_qwen3moe.npz |out| max", float(np.abs(dumps[0]).max()))


def topk_case():
    rng = np.random.default_rng(7)
    rows, meta, ids, wts = [], [], [], []
    for E, K in ((128, 8), (64, 6), (8, 2), (128, 1), (128, 16)):
        for renorm in (False, True):
            for kind in range(7):
                if kind < 3:
                    v = rng.normal(0, 3 if kind else 1, E).astype(np.float32)
                elif kind == 3:
                    v = rng.integers(-2, 3, E).astype(np.float32)                  # heavy ties
                elif kind == 4:
                    v = rng.normal(0, 30, E).astype(np.float32); v[rng.random(E) < 0.1] = -np.inf
                elif kind == 5:
                    v = np.zeros(E, np.float32)                                     # all equal: ids 0..K-1
                else:
                    v = rng.normal(0, 1, E).astype(np.float32); v[rng.integers(0, E)] = np.nan   # a NaN logit: no candidate in any round
                bits = RTK.bf16_bits(v)
                i, w = RTK.ref_topk(bits, K, renorm)
                row = np.zeros(128, np.uint16); row[:E] = bits
                rows.append(row); meta.append((E, K, int(renorm)))
                ids.append(np.pad(np.array(i, np.int64), (0, 16 - K))); wts.append(np.pad(np.array(w, np.float32), (0, 16 - K)))
    np.savez_compressed(HERE / "topk_rows.npz", rows=np.stack(rows), meta=np.array(meta), ids=np.stack(ids), wts=np.stack(wts))
    print("topk_rows.npz", len(rows), "rows")


def moe_block_case():
    out = {}
    for n, (E, K) in enumerate(((8, 2), (128, 8))):
        for renorm in (False, True):
            data = RNUM.fixture(experts=E, top_k=K, renormalize=renorm)
            ref, ref_ids = RNUM.scalar_reference(data)
            act, written, sel = RNUM.vectorized(data)
            tag = f"E{E}K{K}R{int(renorm)}"
            out[tag + "_x"] = data["x"]; out[tag + "_router"] = data["router"]
            out[tag + "_scalar"] = ref; out[tag + "_vector"] = act
            out[tag + "_ids"] = np.array(ref_ids); out[tag + "_sel"] = np.array(sel)
    suite = RNUM.acceptance_suite()
    out["suite_passed"] = np.array(suite["passed"]); out["suite_cases"] = np.array(len(suite["cases"]))
    np.savez_compressed(HERE / "moe_block.npz", **out)
    print("moe_block.npz", suite["passed"], len(suite["cases"]))


MLA_FILE = "examples/dsv2lite/results/2026-10-14-k1/b_alld4r0l1kvs_stamps/fleet_src/host/reference_decode.py"


def mla_case():
    """One absorbed-MLA + MoE layer and one dense layer, 24 decode positions each, run by the NumPy reference archived in
    the reference tree (bf16 rounding on).  Inputs and weights are regenerated from the seeds by the test."""
    import importlib.util
    from oracle import ref_mla as M
    from tests.golden.cases import MLA_SMALL
    spec = importlib.util.spec_from_file_location("fleet_reference_decode", REF / MLA_FILE)
    R = importlib.util.module_from_spec(spec)
    sys.modules["fleet_reference_decode"] = R
    spec.loader.exec_module(R)
    out, n = {}, 24
    for tag, dense in (("moe", 0), ("dense", 96)):
        d = M.MlaDims(**MLA_SMALL, dense_inter=dense)
        L = M.synthetic_layer(d, seed=5)
        cfg = R.ModelConfig(hidden=d.hidden, heads=d.heads, kv_lora_rank=d.kv_lora, qk_nope=d.qk_nope, qk_rope=d.qk_rope, v_head=d.v_head,
                            moe_inter=d.moe_inter, n_routed=d.n_routed, top_k=d.top_k, bf16=True)
        kw = dict(input_layernorm=L.input_layernorm, q_proj=L.q_proj, kv_a_proj_with_mqa=L.kv_a_proj_with_mqa, kv_a_layernorm=L.kv_a_layernorm,
                  kv_b_proj=L.kv_b_proj, o_proj=L.o_proj, post_attention_layernorm=L.post_attention_layernorm)
        if dense:
            kw.update(mlp_gate=L.mlp["gate"], mlp_up=L.mlp["up"], mlp_down=L.mlp["down"])
        else:
            kw.update(gate_weight=L.mlp["router"], experts_gate=L.mlp["egate"], experts_up=L.mlp["eup"], experts_down=L.mlp["edown"],
                      shared_gate=L.mlp["sgate"], shared_up=L.mlp["sup"], shared_down=L.mlp["sdown"])
        W = R.LayerWeights(**kw)
        cos, sin = R.yarn_cos_sin(d.qk_rope, n, cfg.rope_theta, cfg.rope_factor, cfg.rope_original_max, cfg.beta_fast, cfg.beta_slow,
                                  cfg.mscale, cfg.mscale_all_dim)
        rng = np.random.default_rng(1)
        cache = np.zeros((n, d.kv_lora + d.qk_rope), np.float32)
        ys = []
        for pos in range(n):
            x = O.bfr(rng.standard_normal(d.hidden, dtype=np.float32))
            ys.append(R.decoder_layer(cfg, W, x, cache, pos, cos, sin))
        out.update({f"{tag}_y": np.stack(ys), f"{tag}_cache": cache, f"{tag}_cos": cos.astype(np.float32), f"{tag}_sin": sin.astype(np.float32),
                    f"{tag}_scale": np.float64(cfg.softmax_scale)})
    np.savez_compressed(HERE / "mla_layer.npz", seed=5, xseed=1, n=n, dense_inter=96, **out)
    print("mla_layer.npz", {k: v.shape for k, v in out.items() if hasattr(v, "shape")})


if __name__ == "__main__":
    if "--mla-only" in sys.argv:
        mla_case()
        raise SystemExit(0)
    if "--topk-only" in sys.argv:
        topk_case()
        raise SystemExit(0)
    mla_case()
    decode_case(SMALL_MOE, seed=3, n_prompt=8, n_gen=8, gamma="ones", out="decode_small_moe.npz")
    decode_case(SMALL_DENSE, seed=4, n_prompt=6, n_gen=6, gamma="normal", out="decode_small_dense.npz")
    topk_case()
    moe_block_case()
    layer_case()
