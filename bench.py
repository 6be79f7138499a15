#!/usr/bin/env python3
"""Headline benchmark: Qwen3-30B-A3B-shaped bf16 greedy decode at batch 1, one persistent launch per token.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--layers L] [--prompt P]

A step is one decode step (one token through all layers + lm_head + argmax) at context >= P (default 1024: the
prompt is fed token by token through the same kernel first, as the reference's host does).  Prints ONE JSON line:
value = ms per token with every input resident in HBM (K launches back to back, the next token never leaves the
device), e2e = the same through the C ABI's host-buffer decode (token id host->device and device->host every step),
roofline = algorithmic bytes of a step / measured launch time against the measured HBM copy peak, cpu_baseline = the
oracle (numpy restatement of the reference's CPU path) timed on this box's cores on a bounded sample.
With --impl reference the CPU path itself is the thing measured (same metric / config), on rank 0 only.
N > 1: ONE request sharded over the N GPUs (tensor parallel: the ranks exchange partial rows inside the kernel; strong
scaling, value = the request's ms/token); --shard replicas runs N independent requests instead (no exchange; value stays
one request's ms/token, the job's aggregate tokens/s is in config).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC, UNIT = "decode_ms_per_token_bs1", "ms/token"
DRAM_TRAFFIC_CAPTURE = (862.60e6, 854.11e6)   # (dram bytes read + written, algorithmic bytes) of the captured 2-layer launch
DRAM_TRAFFIC_CAPTURE_BS32 = (3053.90e6, 2931.44e6)   # the same for the captured 2-layer batched step (32 sequences)
MODEL = "qwen3-30b-a3b"          # the configuration the metric is quoted on; --model qwen3-8b reports the dense config beside it


def oracle_cfg(O):
    return {"qwen3-30b-a3b": O.QWEN3_30B_A3B, "qwen3-8b": O.QWEN3_8B}[MODEL]


def workload(layers: int, prompt: int) -> str:
    return f"{MODEL} decode bs1, {layers} layers, prompt {prompt} random ids, then greedy tokens"


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 100 ms while the kernel runs (prompt feed and timed region)."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------------------------------------------ CPU arm
def oracle_sample(dims_cfg, layers_total: int, context: int, get_layer_weights, lm_head, final_norm, embed_row, seconds: float = 12.0):
    """Time the oracle on a bounded sample: `ls` layers of the model at `context` prior tokens, a few decode steps, plus
    the lm_head GEMV; scaled to the whole model (layers_total layers).  Returns (ms per token estimate, description)."""
    from oracle import ref_decode as O
    ls = 2
    od = O.dims_from_config(dims_cfg, MODEL, layers=ls)
    t = {}
    for L in range(ls):
        t.update(get_layer_weights(L))
    t["model.norm.weight"], t["lm_head.weight"] = final_norm, lm_head
    t["model.embed_tokens.weight"] = embed_row[None, :]
    ref = O.Ref(od, O.DictWeights(t), context + 64)
    rng = np.random.default_rng(0)
    ref.kc[:, :context] = O.bfr(rng.standard_normal((ls, context, od.NKV, od.HD), dtype=np.float32) * np.float32(0.02))
    ref.vc[:, :context] = O.bfr(rng.standard_normal((ls, context, od.NKV, od.HD), dtype=np.float32) * np.float32(0.02))
    x0 = t["model.embed_tokens.weight"][0]
    xs = O.rmsnorm(x0, final_norm, od.eps)
    layer_s, head_s, n = [], [], 0
    t_end = time.perf_counter() + seconds
    while n < 3 or (time.perf_counter() < t_end and n < 40):
        a = time.perf_counter()
        x = x0.copy()
        for L in range(ls):
            x = ref.layer(L, x, context + n)
        b = time.perf_counter()
        logits = O.bfr(lm_head @ xs)
        int(np.argmax(logits))
        c = time.perf_counter()
        if n >= 1:                                                        # first pass warms the page cache / BLAS threads
            layer_s.append((b - a) / ls); head_s.append(c - b)
        n += 1
    ms = (float(np.median(layer_s)) * layers_total + float(np.median(head_s))) * 1e3
    return ms, f"{len(layer_s)} decode steps of {ls} layers + lm_head at context {context}, median per-layer time x {layers_total} layers"


def host_cores() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def use_all_cores() -> int:
    """Give numpy's BLAS every core this process may run on (a launcher such as torchrun exports OMP_NUM_THREADS=1, which
    would otherwise pin the CPU arm to one thread) and return the thread count it then reports."""
    try:
        from threadpoolctl import threadpool_info, threadpool_limits
        threadpool_limits(limits=host_cores())
        return max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        return 1


def blas_threads() -> int:
    try:
        from threadpoolctl import threadpool_info
        return max([p.get("num_threads", 1) for p in threadpool_info()] or [1])
    except Exception:
        return 1


def run_reference(args, rank: int, world: int):
    """The reference's CPU implementation of the path (its numpy path restated in oracle/) on this box's host cores."""
    if rank != 0:
        return
    if MODEL == "deepseek-v2-lite":
        return run_reference_mla(args)
    from oracle import ref_decode as O
    use_all_cores()
    cfg = oracle_cfg(O)
    layers_total = args.layers or cfg["num_hidden_layers"]
    od = O.dims_from_config(cfg, MODEL, layers=2)
    W = O.SyntheticWeights(O.Dims(**{**od.__dict__, "V": 8}), seed=0, gamma="ones")
    rng = np.random.default_rng(1)
    lm = O.bfr(rng.standard_normal((cfg["vocab_size"], od.H), dtype=np.float32) * np.float32(0.02))

    def layer_w(L):
        return {k: v for k, v in W.t.items() if k.startswith(f"model.layers.{L}.")}
    vals = []
    for i in range(args.warmup + args.steps):
        ms, sample = oracle_sample(cfg, layers_total, args.prompt, layer_w, lm, W.t["model.norm.weight"], W.t["model.embed_tokens.weight"][0],
                                   seconds=max(2.0, 60.0 / max(1, args.warmup + args.steps)))
        if i >= args.warmup:
            vals.append(ms)
    v = float(np.median(vals))
    cores = blas_threads()
    B = max(1, args.batch)
    metric, unit, hib, work = METRIC, UNIT, False, workload(layers_total, args.prompt)
    if B > 1:                                                              # the CPU path decodes one sequence at a time: its tok/s does not grow with the batch
        metric, unit, hib, v = f"decode_tok_per_s_bs{B}", "tok/s", True, 1000.0 / v
        work = f"{MODEL} decode bs{B}, {layers_total} layers, {B} prompts of {args.prompt} random ids, then greedy tokens"
        sample += "; one sequence at a time"
    print(json.dumps({"impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": 1000.0 / v if B > 1 else v, "higher_is_better": hib, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": work, "parallelism": "cpu", "norm_gamma": "ones"},
                      "cpu_baseline": {"value": v, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
                      "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


# ------------------------------------------------------------------------------------------------ DeepSeek-V2-Lite (latent attention)
def run_mla(args, rank: int, world: int, local_rank: int):
    """--model deepseek-v2-lite: the same measurement for the latent-attention / shared-expert model (one GPU per request;
    N > 1 runs N independent requests)."""
    import torch
    import etx_megakernel_b200  # noqa: F401
    from etx_megakernel_b200.models import dsv2 as M
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    d = M.load_dims("deepseek-v2-lite", layers=args.layers or None)
    P, K, Wm = args.prompt, args.steps, args.warmup
    maxlen = ((P + Wm + K + 40 + 15) // 16) * 16
    weights = M.random_weights(d, maxlen, dev, seed=rank)
    prog = M.MlaProgram(d, weights, device=local_rank, maxlen=maxlen, steps=maxlen)
    prompt = np.random.default_rng(1000 + rank).integers(0, d.V, P)
    tin = torch.zeros_like(prog.buf["token_in"]); tin[:P] = torch.tensor(prompt, dtype=torch.int32)
    prog.buf["token_in"].copy_(tin)
    clk = ClockSampler(local_rank)
    clk.__enter__()
    try:
        t0 = time.perf_counter()
        for t in range(P + Wm):
            prog.step(t, t, write_next=t + 1 >= P, wait=(t % 128 == 127))
        prog.session.wait(120.0)
        torch.cuda.synchronize(dev)
        prefill_s = time.perf_counter() - t0
        stream = torch.cuda.Stream(dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if dist:
            dist.barrier()
        torch.cuda.synchronize(dev)
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(K):
                t = P + Wm + i
                prog.session.set_step(tok=t, pos=t, write_next=1)
                prog.session.launch(stream.cuda_stream)
            e1.record(stream)
        torch.cuda.synchronize(dev)
        prog.session.wait(120.0)
        if dist:
            dist.barrier()
        dev_ms = e0.elapsed_time(e1) / K
        gen_dev = prog.buf["token_out"][P + Wm - 1:P + Wm + K].cpu().numpy()
        h0 = time.perf_counter()
        toks_host, _ = prog.session.decode_host(np.asarray([int(gen_dev[0])], np.int32), K, P + Wm)
        host_ms = (time.perf_counter() - h0) * 1e3 / K
    finally:
        clk.__exit__(None, None, None)
    clocks = clk.summary()
    same_tokens = bool(np.array_equal(toks_host, gen_dev[1:K + 1]))
    from etx_megakernel_b200.runtime.dist import slowest
    dev_ms, host_ms = slowest([dev_ms, host_ms], dist, dev)
    ctx = P + Wm + K // 2
    ledger = M.step_bytes(d, ctx)
    peak, peak_src = measured_peaks()
    achieved = ledger["total"] / (dev_ms * 1e-3) / 1e9
    line = {"metric": METRIC, "value": dev_ms, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm, "ms_per_step": dev_ms, "higher_is_better": False,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"deepseek-v2-lite decode bs1, {d.L} layers ({d.DENSE_LAYERS} dense), prompt {P} random ids, then greedy tokens",
                       "prefill": "the prompt is fed token by token through the same kernel", "context": ctx,
                       "parallelism": "single" if world == 1 else f"replicas x{world} (independent requests)", "norm_gamma": "ones",
                       "l2": f"each step streams {ledger['total'] / 1e9:.1f} GB (> 126 MB L2)", "prefill_s": round(prefill_s, 2),
                       "host_tokens_equal_device_tokens": same_tokens},
            "e2e": {"value": host_ms, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4}, "gpu_launches": K, "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                         "algorithmic_bytes_per_launch": ledger["total"], "kernel": "etxb_megakernel",
                         "ledger": "per layer: q / kv_a / kv_b / o projections + latent cache + (router + (top-k + shared) experts | dense MLP); + lm_head"}}
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = mla_cpu_baseline(d, weights, ctx)
    if rank == 0:
        print(json.dumps(line))
    prog.close()
    if dist:
        dist.destroy_process_group()


def run_reference_mla(args):
    """--impl reference --model deepseek-v2-lite: the oracle's layers on the host cores with random weights of the model's
    shapes (a pool of 8 routed experts stands for the 64: what a step multiplies is the same)."""
    import etx_megakernel_b200  # noqa: F401
    from etx_megakernel_b200.models import dsv2 as M
    from oracle import ref_mla as R
    cores = use_all_cores()
    d = M.load_dims("deepseek-v2-lite", layers=args.layers or None)
    ctx = args.prompt + args.warmup + args.steps // 2
    rng = np.random.default_rng(0)
    w = lambda *shape: R.bfr(rng.standard_normal(shape, dtype=np.float32) * np.float32(0.02))   # noqa: E731

    class Pool:
        def __init__(self, mats):
            self.mats = mats

        def __getitem__(self, e):
            return self.mats[int(e) % len(self.mats)]
    one = np.ones
    att = lambda: (one(d.H, np.float32), w(d.NH * d.QH, d.H), w(d.ROW, d.H), one(d.C, np.float32), w(d.NH * (d.DN + d.DV), d.C), w(d.H, d.NH * d.DV),   # noqa: E731
                   one(d.H, np.float32))
    dense, moe = R.MlaLayer(*att()), R.MlaLayer(*att())
    dense.mlp = {"gate": w(d.DENSE_INTER, d.H), "up": w(d.DENSE_INTER, d.H), "down": w(d.H, d.DENSE_INTER)}
    si = d.MI * d.NS
    moe.mlp = {"router": w(d.E, d.H), "egate": Pool([w(d.MI, d.H) for _ in range(8)]), "eup": Pool([w(d.MI, d.H) for _ in range(8)]),
               "edown": Pool([w(d.H, d.MI) for _ in range(8)]), "sgate": w(si, d.H), "sup": w(si, d.H), "sdown": w(d.H, si)}
    lm = w(d.V, d.H)
    cos, sin = R.yarn_tables(mla_oracle_dims(R, d, False), ctx + 8)
    cache = rng.standard_normal((ctx + 8, d.ROW)).astype(np.float32)
    x = rng.standard_normal(d.H).astype(np.float32)

    def step():
        t0 = time.perf_counter()
        R.layer(mla_oracle_dims(R, d, True), dense, x, cache, ctx, cos, sin)
        t1 = time.perf_counter()
        R.layer(mla_oracle_dims(R, d, False), moe, x, cache, ctx, cos, sin)
        t2 = time.perf_counter()
        lm @ x
        t3 = time.perf_counter()
        return 1e3 * (d.DENSE_LAYERS * (t1 - t0) + (d.L - d.DENSE_LAYERS) * (t2 - t1) + (t3 - t2))
    for _ in range(args.warmup):
        step()
    v = float(np.mean([step() for _ in range(args.steps)]))
    print(json.dumps({"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": v, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"deepseek-v2-lite decode bs1, {d.L} layers ({d.DENSE_LAYERS} dense), prompt {args.prompt} random ids, then greedy tokens",
                                 "parallelism": "cpu", "norm_gamma": "ones"},
                      "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                       "sample": f"per step: the dense layer once, one MoE layer once, the lm_head product, at context {ctx}; scaled to {d.L} layers"},
                      "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


class _LazyExperts:
    """m["egate"][e]-style access to one expert's rows of a packed device tensor (fetched when asked for)."""

    def __init__(self, t, rows):
        self.t, self.rows = t, rows

    def __getitem__(self, e):
        a = self.t[e]
        return (a[self.rows] if self.rows is not None else a).float().cpu().numpy()


def mla_oracle_layer(R, d, weights, L):
    """The oracle's layer object of layer L over the device's packed weights (experts fetched lazily)."""
    g = lambda n: weights[f"{L}.{n}"].float().cpu().numpy()                 # noqa: E731
    wqa = g("wqa")
    lw = R.MlaLayer(g("ln1"), wqa[:d.NH * d.QH], wqa[d.NH * d.QH:], g("kvln"), g("wkvb"), g("wo"), g("ln2"))
    if d.dense(L):
        wgu = g("wgu")
        lw.mlp = {"gate": wgu[:d.DENSE_INTER], "up": wgu[d.DENSE_INTER:], "down": g("wd")}
    else:
        w13, w2 = weights[f"{L}.w13"], weights[f"{L}.w2"]
        sh = [w13[d.E + i].float().cpu().numpy() for i in range(d.NS)]
        lw.mlp = {"router": g("wr"), "egate": _LazyExperts(w13, slice(0, d.MI)), "eup": _LazyExperts(w13, slice(d.MI, 2 * d.MI)), "edown": _LazyExperts(w2, None),
                  "sgate": np.concatenate([s[:d.MI] for s in sh]), "sup": np.concatenate([s[d.MI:] for s in sh]),
                  "sdown": np.concatenate([w2[d.E + i].float().cpu().numpy() for i in range(d.NS)], axis=1)}
    return lw


def mla_oracle_dims(R, d, dense):
    return R.MlaDims(hidden=d.H, heads=d.NH, kv_lora=d.C, qk_nope=d.DN, qk_rope=d.DR, v_head=d.DV, moe_inter=d.MI, n_routed=d.E, top_k=d.TOPK, n_shared=d.NS,
                     dense_inter=d.DENSE_INTER if dense else 0, eps=d.eps, theta=d.theta, rope_factor=d.rope_factor, rope_original_max=d.rope_original_max,
                     beta_fast=d.beta_fast, beta_slow=d.beta_slow, mscale=d.mscale, mscale_all_dim=d.mscale_all_dim, norm_topk=d.norm_topk)


def mla_cpu_baseline(d, weights, ctx, budget_s: float = 20.0):
    """The oracle (oracle/ref_mla.py) on the host cores: a few decode steps of the dense layer and of one MoE layer at the
    bench's context + the lm_head product, scaled to the model's layer counts."""
    from oracle import ref_mla as R                                        # the checker, timed: the one CPU leg of this bench
    cores = use_all_cores()
    x = np.random.default_rng(0).standard_normal(d.H).astype(np.float32)
    cos, sin = R.yarn_tables(mla_oracle_dims(R, d, False), ctx + 8)
    per = {}
    for kind, L in (("dense", 0 if d.DENSE_LAYERS else None), ("moe", d.DENSE_LAYERS if d.L > d.DENSE_LAYERS else None)):
        if L is None:
            per[kind] = 0.0
            continue
        od, lw = mla_oracle_dims(R, d, kind == "dense"), mla_oracle_layer(R, d, weights, L)
        cache = np.random.default_rng(1).standard_normal((ctx + 8, d.ROW)).astype(np.float32)
        ts = []
        t_end = time.perf_counter() + budget_s / 2
        while len(ts) < 3 or (time.perf_counter() < t_end and len(ts) < 12):
            t0 = time.perf_counter()
            R.layer(od, lw, x, cache, ctx, cos, sin)
            ts.append(time.perf_counter() - t0)
        per[kind] = float(np.median(ts))
    lm = weights["lm_head"].float().cpu().numpy()
    t0 = time.perf_counter()
    for _ in range(3):
        lm @ x
    t_lm = (time.perf_counter() - t0) / 3
    ms = 1e3 * (d.DENSE_LAYERS * per["dense"] + (d.L - d.DENSE_LAYERS) * per["moe"] + t_lm)
    return {"value": ms, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"median of a few decode steps of the dense layer and of one MoE layer at context {ctx} + the lm_head product, scaled to {d.L} layers"}


# ------------------------------------------------------------------------------------------------ GPU arm
def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import etx_megakernel_b200  # noqa: F401
    from etx_megakernel_b200.models import decode as D
    from etx_megakernel_b200.models import qwen as Q
    from oracle import ref_decode as O                                     # cpu_baseline leg and the byte ledger only
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    d = Q.load_dims(MODEL, layers=args.layers or None)
    P, K, Wm = args.prompt, args.steps, args.warmup
    maxlen = ((P + Wm + K + 40 + 15) // 16) * 16
    tp, why_not = 1, None
    if world > 1 and args.shard in ("auto", "tp"):
        try:
            Q.shard_dims(d, world)
            tp = world
        except ValueError as e:                                            # the model does not split this many ways
            if args.shard == "tp":
                raise
            why_not = str(e)
    if tp > 1:
        # one request over all ranks: every rank draws the whole model from the same seed, keeps its shard, and the ranks
        # meet inside the kernel at the row-parallel grids (no collective library call on the data path)
        from etx_megakernel_b200.runtime import dist as RD
        whole = D.random_packed_weights(d, maxlen, dev, seed=0, gamma="ones")
        weights = Q.shard_weights(whole, d, tp, rank)
        del whole
        torch.cuda.empty_cache()
        prog = D.DecodeProgram(Q.shard_dims(d, tp), weights, device=local_rank, maxlen=maxlen, steps=maxlen, ranks=tp, rank=rank)
        prog.session.set_option("timeout_ms", 10000)
        RD.connect_ranks(prog, dist)
    else:
        weights = D.random_packed_weights(d, maxlen, dev, seed=rank, gamma="ones")
        prog = D.DecodeProgram(d, weights, device=local_rank, maxlen=maxlen, steps=maxlen, flagged=args.flagged)
    prompt = np.random.default_rng(1000 + (0 if tp > 1 else rank)).integers(0, d.V, P)
    # prefill: the prompt token by token through the same kernel (fills the KV caches), plus W warm-up decode steps
    tin = torch.zeros_like(prog.buf["token_in"]); tin[:P] = torch.tensor(prompt, dtype=torch.int32)
    prog.buf["token_in"].copy_(tin)
    # the clock sampler runs from the prompt feed (the same kernel back to back: the same load) through the timed region,
    # so that the few hundred milliseconds of the timed steps are not its only samples
    clk = ClockSampler(local_rank)
    clk.__enter__()
    t0 = time.perf_counter()
    for t in range(P + Wm):
        prog.step(t, t, write_next=t + 1 >= P, wait=(t % 128 == 127))
    prog.session.wait(120.0)
    torch.cuda.synchronize(dev)
    prefill_s = time.perf_counter() - t0
    # timed region: exactly K steps, back to back, CUDA events on the launching stream, barrier on both sides
    stream = torch.cuda.Stream(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist:
        dist.barrier()
    torch.cuda.synchronize(dev)
    try:
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(K):
                t = P + Wm + i
                prog.session.set_step(tok=t, pos=t, write_next=1)
                prog.session.launch(stream.cuda_stream)
            e1.record(stream)
        torch.cuda.synchronize(dev)
        prog.session.wait(120.0)
        if dist:
            dist.barrier()
        dev_ms = e0.elapsed_time(e1) / K
        # end to end through the host-buffer entry point: the same K positions, token ids through host memory
        gen_dev = prog.buf["token_out"][P + Wm - 1:P + Wm + K].cpu().numpy()      # argmax of steps P+Wm-1 .. P+Wm+K-1
        first = int(gen_dev[0])
        h0 = time.perf_counter()
        toks_host, ms_host = prog.session.decode_host(np.asarray([first], np.int32), K, P + Wm)
        host_ms = (time.perf_counter() - h0) * 1e3 / K
        # the unfused baseline: the same steps as one launch per grid (what the single launch is compared with)
        Ku = 0 if tp > 1 else min(K, 4)                                          # (a sharded session runs as the single launch only)
        u0, u1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            u0.record(stream)
            for i in range(Ku):
                t = P + Wm + i
                prog.session.set_step(tok=t, pos=t, write_next=1)
                prog.session.launch_unfused(stream.cuda_stream)
            u1.record(stream)
        torch.cuda.synchronize(dev)
        prog.session.wait(120.0)
        unfused_ms = u0.elapsed_time(u1) / Ku if Ku else None
        gen_unfused = prog.buf["token_out"][P + Wm:P + Wm + Ku].cpu().numpy()
    finally:
        clk.__exit__(None, None, None)
    clocks = clk.summary()
    same_tokens = bool(np.array_equal(toks_host, gen_dev[1:K + 1]))
    from etx_megakernel_b200.runtime.dist import slowest
    dev_ms, host_ms = slowest([dev_ms, host_ms], dist, dev)
    ctx = P + Wm + K // 2
    ledger = O.step_bytes(O.dims_from_config(oracle_cfg(O), MODEL, layers=d.L), ctx)
    peak, peak_src = measured_peaks()
    achieved = ledger["total"] / (dev_ms * 1e-3) / 1e9
    # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel on a 2-layer
    # model (DRAM_TRAFFIC_CAPTURE: measured bytes, algorithmic bytes of the captured launch), scaled to this launch by its
    # algorithmic bytes -- a capture of the 61 GB launch itself is outside what a profiler run should hold
    traffic = ledger["total"] * (DRAM_TRAFFIC_CAPTURE[0] / DRAM_TRAFFIC_CAPTURE[1])
    jobs = 1 if tp > 1 else world                                                # sequences decoded at once by the whole job
    peak_all = peak * (tp if tp > 1 else 1)
    line = {"metric": METRIC, "value": dev_ms, "unit": UNIT, "n_gpus": world, "steps": K, "warmup": Wm, "ms_per_step": dev_ms,
            "higher_is_better": False, "scaling": "strong" if tp > 1 else "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload(d.L, P), "prefill": "the prompt is fed token by token through the same kernel",
                       "context": ctx, "parallelism": "single" if world == 1 else f"tp{tp} (one request over {tp} GPUs, in-kernel exchange of partial rows"
                                      + (f", kv heads replicated x{Q.kv_replication(d, tp)}" if Q.kv_replication(d, tp) > 1 else "") + ")" if tp > 1
                       else f"replicas x{world} (independent requests; value is one request's latency" + (f"; not sharded: {why_not}" if why_not else "") + ")",
                       "norm_gamma": "ones", "l2": f"each step streams {ledger['total'] / 1e9:.1f} GB (> 126 MB L2)",
                       "tokens_per_s": 1000.0 / dev_ms * jobs, "prefill_s": round(prefill_s, 2), "host_tokens_equal_device_tokens": same_tokens,
                       "unfused_baseline": {"ms_per_token": unfused_ms, "launches_per_token": len(prog.plan.graph.grids), "steps": Ku,
                                            "same_tokens": bool(np.array_equal(gen_unfused, gen_dev[1:Ku + 1])),
                                            "what": "the same tiles, one kernel launch per grid on one stream"}},
            "e2e": {"value": host_ms, "unit": UNIT, "h2d_bytes_per_step": 4, "d2h_bytes_per_step": 4},
            "gpu_launches": K, "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak_all, "unit": "GB/s", "frac": achieved / peak_all, "traffic": traffic,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": ledger["total"], "kernel": "etxb_megakernel"}}
    if rank == 0 and world == 1 and not args.no_cpu:
        def layer_w(L):
            return Q.unpack_layer_hf(d, lambda n: weights[n].view(torch.int16).cpu().numpy().view(np.uint16), L)
        f = lambda t: (t.view(torch.int16).cpu().numpy().view(np.uint16).astype(np.uint32) << 16).view(np.float32)     # noqa: E731
        use_all_cores()
        ms, sample = oracle_sample(oracle_cfg(O), d.L, P, layer_w, f(weights["lm_head"]), f(weights["final_norm"]), f(weights["embed"][int(prompt[0])]))
        line["cpu_baseline"] = {"value": ms, "unit": UNIT, "cores": blas_threads(), "kind": "port", "sample": sample}
    if tp > 1:
        RD.close_ranks(prog, dist)
    else:
        prog.close()
    if world == 1 and d.moe and args.bs32_leg and MODEL == "qwen3-30b-a3b":
        # the other half of the metric ("tok/s @bs32") on the same weights, as an extra key of the same line
        line["batched"] = batched_leg(d, weights, 32, P + Wm + K, dev, local_rank, O, peak)
    if rank == 0:
        print(json.dumps(line))
    if dist:
        dist.destroy_process_group()


def batched_leg(d, weights, B, pos0, dev, local_rank, O, peak, K=8, Wm=3):
    """B sequences per step through the batched program (python bench.py --batch B measures the same with a real prefill and
    the host-buffer loop): here a random KV cache stands for the prefill -- a step streams the same bytes -- so the leg
    adds a second, not a minute, to the default run."""
    import torch
    from etx_megakernel_b200.models import batched as BT
    maxlen = int(weights["cos_sin"].shape[0])
    K = max(1, min(K, maxlen - pos0 - Wm - 1))
    prog = BT.BatchProgram(d, weights, B, device=local_rank, maxlen=maxlen, steps=64)
    prog.buf["kc"].normal_(0, 0.02); prog.buf["vc"].normal_(0, 0.02)
    prog.buf["token_in"].random_(0, d.V)
    torch.cuda.synchronize(dev)
    for i in range(Wm):
        prog.step(i, pos0 + i, write_next=True)
    prog.active_experts()
    stream = torch.cuda.Stream(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    with torch.cuda.stream(stream):
        e0.record(stream)
        for i in range(K):
            prog.session.set_step(tok=Wm + i, pos=pos0 + Wm + i, write_next=1)
            prog.session.launch(stream.cuda_stream)
        e1.record(stream)
    torch.cuda.synchronize(dev)
    prog.session.wait(300.0)
    ms = e0.elapsed_time(e1) / K
    active = prog.active_experts() / K
    prog.close()
    ledger = O.step_bytes(O.dims_from_config(oracle_cfg(O), MODEL, layers=d.L), pos0 + Wm + K // 2, batch=B, active_experts=float(np.mean(active)))
    achieved = ledger["total"] / (ms * 1e-3) / 1e9
    return {"metric": f"decode_tok_per_s_bs{B}", "value": B * 1000.0 / ms, "unit": "tok/s", "ms_per_step": ms, "steps": K, "warmup": Wm, "gpu_launches": K,
            "active_experts_per_layer": float(np.mean(active)), "context": pos0 + Wm + K // 2,
            "kv": "random-filled cache in place of a prefill (bench.py --batch 32 runs the prompts through the kernel and the host-buffer loop)",
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "algorithmic_bytes_per_launch": ledger["total"]}}


def run_batch(args, rank: int, world: int, local_rank: int):
    """--batch B: B sequences per step in one persistent launch (the "tok/s @bs32" half of the metric).  One GPU per
    process; N > 1 runs N independent batches (replicas).  value = tokens per second of the whole job."""
    import torch
    import etx_megakernel_b200  # noqa: F401
    from etx_megakernel_b200.models import batched as BT
    from etx_megakernel_b200.models import decode as D
    from etx_megakernel_b200.models import qwen as Q
    from etx_megakernel_b200.runtime.dist import slowest
    from oracle import ref_decode as O                                     # the byte ledger and the cpu_baseline leg only
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback for the product path")
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    d = Q.load_dims(MODEL, layers=args.layers or None)
    B, P, K, Wm = args.batch, args.prompt, args.steps, args.warmup
    maxlen = ((P + Wm + 2 * K + 40 + 15) // 16) * 16
    weights = D.random_packed_weights(d, maxlen, dev, seed=rank, gamma="ones")
    prog = BT.BatchProgram(d, weights, B, device=local_rank, maxlen=maxlen, steps=maxlen)
    prompts = np.random.default_rng(1000 + rank).integers(0, d.V, (B, P))
    tin = torch.zeros_like(prog.buf["token_in"]); tin[:P] = torch.from_numpy(prompts.T.copy()).to(torch.int32)
    prog.buf["token_in"].copy_(tin)
    torch.cuda.synchronize(dev)
    clk = ClockSampler(local_rank)
    clk.__enter__()
    t0 = time.perf_counter()
    for t in range(P + Wm):                                               # prefill: the prompts position by position through the same kernel
        prog.step(t, t, write_next=t + 1 >= P, wait=(t % 64 == 63))
    prog.session.wait(300.0)
    torch.cuda.synchronize(dev)
    prefill_s = time.perf_counter() - t0
    prog.active_experts()
    stream = torch.cuda.Stream(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if dist:
        dist.barrier()
    torch.cuda.synchronize(dev)
    try:
        with torch.cuda.stream(stream):
            e0.record(stream)
            for i in range(K):
                t = P + Wm + i
                prog.session.set_step(tok=t, pos=t, write_next=1)
                prog.session.launch(stream.cuda_stream)
            e1.record(stream)
        torch.cuda.synchronize(dev)
        prog.session.wait(300.0)
        if dist:
            dist.barrier()
        dev_ms = e0.elapsed_time(e1) / K
        active = prog.active_experts() / K                                 # per layer: experts that had a token, averaged over the timed steps
        gen_dev = prog.buf["token_out"][P + Wm - 1:P + Wm + K].cpu().numpy()     # [K + 1][B]
        # end to end with host buffers: every step the B token ids go host -> device from pinned memory and the B results
        # come back, through the session's launch / wait (the call a host integration makes)
        h_in = torch.empty(B, dtype=torch.int32).pin_memory(); h_out = torch.empty(B, dtype=torch.int32).pin_memory()
        h_in.copy_(torch.from_numpy(gen_dev[0].astype(np.int32)))
        toks_host = np.zeros((K, B), np.int32)
        slot_in, slot_out = prog.buf["token_in"][0], prog.buf["token_out"][0]
        h0 = time.perf_counter()
        with torch.cuda.stream(stream):
            for i in range(K):
                slot_in.copy_(h_in, non_blocking=True)
                prog.session.set_step(tok=0, pos=P + Wm + i, write_next=0)
                prog.session.launch(stream.cuda_stream)
                h_out.copy_(slot_out, non_blocking=True)
                stream.synchronize()
                prog.session.wait(300.0)
                toks_host[i] = h_out.numpy()
                h_in.copy_(h_out)
        host_ms = (time.perf_counter() - h0) * 1e3 / K
    finally:
        clk.__exit__(None, None, None)
    clocks = clk.summary()
    same_tokens = bool(np.array_equal(toks_host, gen_dev[1:K + 1]))
    dev_ms, host_ms = slowest([dev_ms, host_ms], dist, dev)
    ctx = P + Wm + K // 2
    od = O.dims_from_config(oracle_cfg(O), MODEL, layers=d.L)
    ledger = O.step_bytes(od, ctx, batch=B, active_experts=float(np.mean(active)))
    peak, peak_src = measured_peaks()
    achieved = ledger["total"] / (dev_ms * 1e-3) / 1e9
    # DRAM bytes per launch: scaled from the ncu capture of the 2-layer batched step (32 sequences) by algorithmic bytes
    traffic = ledger["total"] * (DRAM_TRAFFIC_CAPTURE_BS32[0] / DRAM_TRAFFIC_CAPTURE_BS32[1])
    line = {"metric": f"decode_tok_per_s_bs{B}", "value": world * B * 1000.0 / dev_ms, "unit": "tok/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "ms_per_step": dev_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{MODEL} decode bs{B}, {d.L} layers, {B} prompts of {P} random ids, then greedy tokens", "batch": B, "context": ctx,
                       "prefill": "the prompts are fed position by position through the same kernel", "prefill_s": round(prefill_s, 2),
                       "parallelism": "single" if world == 1 else f"replicas x{world} (independent batches)", "norm_gamma": "ones",
                       "active_experts_per_layer": {"mean": float(np.mean(active)), "min": float(np.min(active)), "max": float(np.max(active)),
                                                    "what": "experts with at least one token, measured by the routing tile over the timed steps"},
                       "l2": f"each step streams {ledger['total'] / 1e9:.1f} GB (> 126 MB L2)", "host_tokens_equal_device_tokens": same_tokens},
            "e2e": {"value": world * B * 1000.0 / host_ms, "unit": "tok/s", "h2d_bytes_per_step": 4 * B, "d2h_bytes_per_step": 4 * B},
            "gpu_launches": K, "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                         "peak_source": peak_src, "algorithmic_bytes_per_launch": ledger["total"], "kernel": "etxb_megakernel",
                         "ledger": "dense weights once + (measured active experts) x 3 x MI x H x 2 per layer + B x KV + lm_head"}}
    if rank == 0 and world == 1 and not args.no_cpu:
        def layer_w(L):
            return Q.unpack_layer_hf(d, lambda n: weights[n].view(torch.int16).cpu().numpy().view(np.uint16), L)
        f = lambda t: (t.view(torch.int16).cpu().numpy().view(np.uint16).astype(np.uint32) << 16).view(np.float32)     # noqa: E731
        use_all_cores()
        ms, sample = oracle_sample(oracle_cfg(O), d.L, P, layer_w, f(weights["lm_head"]), f(weights["final_norm"]), f(weights["embed"][int(prompts[0, 0])]))
        line["cpu_baseline"] = {"value": 1000.0 / ms, "unit": "tok/s", "cores": blas_threads(), "kind": "port",
                                "sample": sample + "; the CPU path decodes one sequence at a time, so its tok/s does not grow with the batch"}
    prog.close()
    if rank == 0:
        print(json.dumps(line))
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default=MODEL, choices=["qwen3-30b-a3b", "qwen3-8b", "deepseek-v2-lite"],
                    help="qwen3-8b: the dense configuration; deepseek-v2-lite: latent attention + shared-expert MoE (both reported beside the headline)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (debugging only; 0 = all)")
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--flagged", type=int, default=0, help="one GPU: hand o_proj / down outputs to the next norm fold as flagged words (1) or through events (0)")
    ap.add_argument("--bs32-leg", type=int, default=1, help="N = 1, the headline model: also time the batched step at 32 sequences and report it under \"batched\" (0: skip)")
    ap.add_argument("--sweep", action="store_true", help="the stand-alone GEMV sweep instead of the decode step: one JSON line per shape (GB/s against the measured HBM peak)")
    ap.add_argument("--batch", type=int, default=1, help="sequences per step (1: the headline ms/token; 8 / 32: tok/s through the batched step)")
    ap.add_argument("--shard", default="auto", choices=["auto", "tp", "replicas"],
                    help="N > 1: ONE request sharded over the N GPUs (tp; auto = tp when the model splits N ways, else replicas) or N independent requests (replicas)")
    a = ap.parse_args()
    globals()["MODEL"] = a.model
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    if a.sweep:
        if rank == 0:
            import etx_megakernel_b200  # noqa: F401  (registers the package under its importable name)
            from etx_megakernel_b200.ops import gemv_sweep
            gemv_sweep.main()
    elif a.model == "deepseek-v2-lite" and a.impl != "reference":
        run_mla(a, rank, world, local)
    elif a.impl == "reference":
        run_reference(a, rank, world)
    elif a.batch > 1:
        run_batch(a, rank, world, local)
    else:
        run_ours(a, rank, world, local)


if __name__ == "__main__":
    main()
