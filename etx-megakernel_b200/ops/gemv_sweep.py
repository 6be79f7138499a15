"""The stand-alone bf16 GEMV sweep (M tokens x K -> N) as ETX programs on one B200, with GB/s against the HBM roofline.

Shapes: M in {1, 2, 4, 8}, K = 4096, N = 12288; M = 1, K = 12288, N = 4096; M = 1, K = 4096, N = 151936 (lm_head).
Weights ~ N(0, 0.02), activations ~ N(0, 1), fp32 accumulation, seed 1.  M = 1 runs as a one-grid graph through the
persistent kernel (plan -> session -> launches, the path a decode program takes); M > 1 runs the column-batched kernel
through `etxb_op_launch`; the rows marked "tc" (M = 8, 32) run the tcgen05 tile of the batched decode step as a one-grid
graph through the persistent kernel (TMA tensor copies, accumulators in tensor memory, K cut in slices where the matrix
has too few 256-row blocks for the workers).  Between timed launches a buffer larger than L2 is written, so every launch streams its
weights from HBM.  Algorithmic bytes per launch: 2 N K + 2 M K + 2 M N.

    python -m etx_megakernel_b200.ops.gemv_sweep            # prints one line per shape
"""
from __future__ import annotations

import json

import numpy as np

SHAPES = [(1, 4096, 12288), (2, 4096, 12288), (4, 4096, 12288), (8, 4096, 12288), (1, 12288, 4096), (1, 4096, 151936),
          (8, 4096, 12288, "tc"), (32, 4096, 12288, "tc"), (32, 2048, 151936, "tc")]


def run(shapes=SHAPES, iters: int = 12, device: int = 0, peak_gbs: float | None = None) -> list:
    import torch

    from .. import ops
    from ..frontends import cuda_link
    from ..importer import argblock
    from ..ir import Graph
    from ..machine import load_machine
    from ..passes import compile_graph
    from ..runtime import Session, op_launch
    ent = ops.all_entries()
    m = load_machine("b200")
    dev = torch.device("cuda", device)
    g0 = torch.Generator(device=dev); g0.manual_seed(1)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.Stream(dev)                                # launches and the timing events share this stream
    out_rows = []
    for shape in shapes:
        M, K, N = shape[:3]
        tc = len(shape) > 3 and shape[3] == "tc"
        W = torch.empty((N, K), dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=g0)
        x = torch.randn((M, K), device=dev, generator=g0).bfloat16()
        out = torch.zeros((M, N), dtype=torch.bfloat16, device=dev)
        session = None
        if not tc:
            tasks, rpt = m.gemv_tasks(N, waves=4 if N > 65536 else 1)
            blob = argblock.pack_named(ent["dsl_gemv"], (tasks, 1, 1), W=W.data_ptr(), x=x.data_ptr(), out=out.data_ptr(), M=N, K=K, rpt=rpt,
                                       tpe=1, nb=M, sx=K, sout=N)
        if tc:
            from . import batch as _batch
            tasks, rpt, S = _batch.split_k(N, K, m.workers())
            part = torch.zeros((S * N * M,), dtype=torch.float32, device=dev)
            count = torch.zeros((tasks // S,), dtype=torch.int32, device=dev)
            blob = argblock.pack_named(ent["gemv_tc"], (tasks, 1, 1), W=W.data_ptr(), x=x.data_ptr(), out=out.data_ptr(), M=N, K=K, rpt=rpt, tpe=S, nb=M,
                                       sx=K, sout=N, rows=part.data_ptr() if S > 1 else 0, resid_in=count.data_ptr() if S > 1 else 0)
            g = Graph(f"gemv_tc_{M}x{K}x{N}")
            g.tensor("impargs", (len(blob),), role="weight", bytes_per_elem=1)
            g.etensor("E_done", (1,), wait_count=tasks)
            g.call_device("gemv", (tasks,), cuda_link("", "etx_tile_gemv_tc", stream_after=""), args=["impargs"], consts=(0,),
                          out_edges={"E_done": "i->(0)"})
            session = Session(compile_graph(g, m, {}), {}, blob, device)

            def launch():
                session.launch(stream.cuda_stream)
        elif M == 1:
            g = Graph(f"gemv_{K}x{N}")
            g.tensor("impargs", (len(blob),), role="weight", bytes_per_elem=1)
            g.etensor("E_done", (1,), wait_count=tasks)
            g.call_device("gemv", (tasks,), cuda_link("", "etx_tile_dsl_gemv", stream_after=""), args=["impargs"], consts=(0,),
                          out_edges={"E_done": "i->(0)"})
            plan = compile_graph(g, m, {})
            session = Session(plan, {}, blob, device)

            def launch():
                session.launch(stream.cuda_stream)
        else:
            def launch():
                op_launch("gemv", blob, tasks, stream=stream.cuda_stream)
        ts = []
        for i in range(iters + 2):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            with torch.cuda.stream(stream):
                flush.zero_()
                e0.record(stream); launch(); e1.record(stream)
            torch.cuda.synchronize(dev)
            if session is not None:
                session.wait(30.0)
            if i >= 2:
                ts.append(e0.elapsed_time(e1) * 1e3)
        us = float(np.median(ts))
        want = (x.float() @ W.float().t())
        err = float((out.float() - want).abs().max() / want.abs().max())
        nbytes = 2 * N * K + 2 * M * K + 2 * M * N
        row = {"M": M, "K": K, "N": N, "engine": "tcgen05" if tc else ("fma ring" if M == 1 else "mma.sync"), "tasks": tasks, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1), "bytes": nbytes,
               "max_rel_err_vs_fp32": err}
        if peak_gbs:
            row["of_peak"] = round(row["gbs"] / peak_gbs, 3)
        out_rows.append(row)
        if session is not None:
            session.close()
        del W, x, out
    return out_rows


def main() -> int:
    import pathlib
    peak = None
    p = pathlib.Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        peak = float(json.loads(p.read_text()).get("hbm_gbs", 0)) or None
    for row in run(peak_gbs=peak):
        print(json.dumps(row))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
