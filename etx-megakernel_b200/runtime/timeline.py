"""Per-task trace of one decode step -> schedule tables and the critical path (the role of etx/tools/timeline.py).

Input: the plan and one row of device stamps per task.  `etxb_trace` gives eight uint64 per task in task-id order
{taken, dependencies ready, body done, worker, four in-body marks} in nanoseconds of the GPU's global timer; the
simulator (`sim.protocol.simulate`) gives the same three times in microseconds.  Output:

  * per grid: tasks, when the last task became ready / finished, median wait and body time, the in-body marks;
  * the critical path: from the task that finished last, step to whichever finished later -- the producer that
    completed its dependencies, or the previous task on the same worker -- until nothing precedes; the span splits
    into task bodies, dependency gaps (arrival -> the waiter saw it) and queue gaps, summed by grid;
  * `raw_rows()`: the reference's ETX_TRACE_RAW layout, nine int64 per task {type, coord[0..3], taken, ready, done,
    worker} (examples/vllm_llm/host.hip:1147-1155 writes it; here the tick is 1 ns, there 10 ns).

    python -m etx_megakernel_b200.runtime.timeline --layers 2 --context 1024          # traced step on cuda:0
    python -m etx_megakernel_b200.runtime.timeline --layers 2 --sim                   # simulated schedule, no GPU
"""
from __future__ import annotations

import argparse
from dataclasses import dataclass

import numpy as np

from ..passes.plan import Plan


@dataclass
class Step:
    task: int
    grid: str
    body_us: float
    gap_us: float
    via: str            # "dependency" | "queue" | "start"


class Timeline:
    def __init__(self, plan: Plan, taken_us, ready_us, done_us, worker=None, marks_us=None):
        n = len(plan.tasks)
        self.plan = plan
        self.taken, self.ready, self.done = (np.asarray(a, np.float64).reshape(n) for a in (taken_us, ready_us, done_us))
        self.worker = np.asarray(worker, np.int64).reshape(n) if worker is not None else self._queue_workers()
        self.marks = np.asarray(marks_us, np.float64).reshape(n, -1) if marks_us is not None else np.full((n, 0), np.nan)
        self.t0 = float(self.taken.min()) if n else 0.0

    # ---- constructors
    @classmethod
    def from_trace(cls, plan: Plan, rows) -> "Timeline":
        """rows: (n_tasks, 8) uint64 as returned by Session.trace(), task-id order, nanoseconds."""
        r = np.asarray(rows).astype(np.int64).reshape(len(plan.tasks), 8)
        marks = np.where(r[:, 4:8] > 0, r[:, 4:8] / 1e3, np.nan)
        return cls(plan, r[:, 0] / 1e3, r[:, 1] / 1e3, r[:, 2] / 1e3, r[:, 3], marks)

    @classmethod
    def from_sim(cls, plan: Plan, sim) -> "Timeline":
        if sim.deadlock:
            raise ValueError("the simulated schedule deadlocked: " + "; ".join(sim.blocked[:4]))
        ids = range(len(plan.tasks))
        return cls(plan, [sim.taken[i] for i in ids], [sim.ready[i] for i in ids], [sim.done[i] for i in ids])

    def _queue_workers(self):
        w = np.zeros(len(self.plan.tasks), np.int64)
        for (dev, k), q in self.plan.static_queues.items():
            w[list(q)] = k
        return w

    # ---- tables
    @property
    def span_us(self) -> float:
        return float(self.done.max() - self.t0) if len(self.done) else 0.0

    def by_grid(self) -> list:
        out = []
        for g in self.plan.graph.grids:
            ids = [self.plan.task_index[(g.name, c)] for c in self.plan.inst.tasks[g.name]]
            rd, dn, tk = self.ready[ids], self.done[ids], self.taken[ids]
            row = {"grid": g.name, "tasks": len(ids), "last_ready": float(rd.max() - self.t0), "last_done": float(dn.max() - self.t0),
                   "phase": float(dn.max() - rd.max()), "wait": float(np.median(rd - tk)), "body": float(np.median(dn - rd)),
                   "body_max": float((dn - rd).max())}
            if self.marks.shape[1]:
                with np.errstate(all="ignore"):
                    rel = self.marks[ids] - rd[:, None]
                    row["marks"] = [float(np.nanmedian(rel[:, k])) if np.isfinite(rel[:, k]).any() else float("nan")
                                    for k in range(rel.shape[1])]
            out.append(row)
        return out

    def critical_path(self):
        """(steps from the last task back to the first, {grid: {"body", "dependency", "queue"}} in microseconds)."""
        plan = self.plan
        prev_on_worker = {}
        for q in plan.static_queues.values():
            for a, b in zip(q, q[1:]):
                prev_on_worker[b] = a
        steps, totals = [], {}
        cur = int(np.argmax(self.done)) if len(self.done) else -1
        while cur >= 0:
            t = plan.tasks[cur]
            cands = []
            for ev in plan.inst.task_in[(t.grid, t.coord)]:
                prods = [plan.task_index[p] for p in plan.inst.producers[ev]]
                if prods:
                    cands.append((max(prods, key=lambda i: self.done[i]), "dependency"))
            if cur in prev_on_worker:
                cands.append((prev_on_worker[cur], "queue"))
            body = float(self.done[cur] - self.ready[cur])
            if not cands:
                steps.append(Step(cur, t.grid, body, float(self.ready[cur] - self.t0), "start"))
                totals.setdefault(t.grid, {"body": 0.0, "dependency": 0.0, "queue": 0.0})["body"] += body
                break
            pred, via = max(cands, key=lambda c: self.done[c[0]])
            gap = float(self.ready[cur] - self.done[pred])
            steps.append(Step(cur, t.grid, body, gap, via))
            e = totals.setdefault(t.grid, {"body": 0.0, "dependency": 0.0, "queue": 0.0})
            e["body"] += body
            e[via] += gap
            cur = pred
        return steps, totals

    def raw_rows(self, tick_ns: float = 1.0) -> np.ndarray:
        n = len(self.plan.tasks)
        rows = np.zeros((n, 9), np.int64)
        for i, t in enumerate(self.plan.tasks):
            rows[i, 0] = self.plan.type_ids[t.grid]
            c = list(t.coord)[:4]
            rows[i, 1:1 + len(c)] = c
        for col, a in ((5, self.taken), (6, self.ready), (7, self.done)):
            rows[:, col] = np.round(a * 1e3 / tick_ns).astype(np.int64)
        rows[:, 8] = self.worker
        return rows

    def write_raw(self, path, tick_ns: float = 1.0) -> None:
        self.raw_rows(tick_ns).astype("<i8").tofile(str(path))

    def text(self, top: int = 12) -> str:
        lines = [f"span {self.span_us:.2f} us, {len(self.plan.tasks)} tasks on {len(self.plan.static_queues)} workers",
                 f"{'grid':14s} {'n':>4s} {'lastready':>9s} {'lastdone':>9s} {'phase':>7s} {'wait':>6s} {'body':>6s} {'max':>6s}  marks after ready (median us)"]
        for r in self.by_grid():
            m = "  ".join(f"{x:5.2f}" for x in r.get("marks", []))
            lines.append(f"{r['grid']:14s} {r['tasks']:4d} {r['last_ready']:9.2f} {r['last_done']:9.2f} {r['phase']:7.2f} {r['wait']:6.2f} "
                         f"{r['body']:6.2f} {r['body_max']:6.2f}  {m}")
        steps, totals = self.critical_path()
        b = sum(v["body"] for v in totals.values()); dgap = sum(v["dependency"] for v in totals.values())
        qgap = sum(v["queue"] for v in totals.values())
        lines.append(f"critical path: {len(steps)} tasks, bodies {b:.2f} us + dependency gaps {dgap:.2f} us + queue gaps {qgap:.2f} us")
        for g, v in sorted(totals.items(), key=lambda kv: -(kv[1]["body"] + kv[1]["dependency"] + kv[1]["queue"]))[:top]:
            lines.append(f"  {g:14s} body {v['body']:7.2f}  dependency gap {v['dependency']:6.2f}  queue gap {v['queue']:6.2f}")
        return "\n".join(lines)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", default="qwen3-30b-a3b")
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--maxlen", type=int, default=1072)
    ap.add_argument("--warm", type=int, default=64, help="untraced steps before the traced one")
    ap.add_argument("--batch", type=int, default=1, help="sequences per step (> 1: the batched step of models.batched)")
    ap.add_argument("--sim", action="store_true", help="simulate the schedule from the tile annotations instead of running on a GPU")
    ap.add_argument("--raw", help="also write the nine-int64-per-task rows to this file")
    a = ap.parse_args(argv)
    from ..models import qwen as Q
    if a.model == "deepseek-v2-lite":                                       # latent attention + shared-expert MoE: its own program
        import torch
        from ..models import dsv2 as M
        d = M.load_dims(a.model, layers=a.layers)
        dev = torch.device("cuda", 0)
        prog = M.MlaProgram(d, M.random_weights(d, a.maxlen, dev, seed=0), device=0, maxlen=a.maxlen)
        prog.buf["ckv"].normal_(0, 0.5)
        torch.cuda.synchronize(dev)
        for t in range(min(a.warm, 8)):
            prog.buf["token_in"][0] = 7
            prog.step(0, a.context + t, False)
        prog.session.set_option("trace", 1)
        prog.step(0, a.context + 9, False)
        print(Timeline.from_trace(prog.plan, prog.session.trace()).text())
        prog.close()
        return 0
    d = Q.load_dims(a.model, layers=a.layers)
    if a.sim:
        from ..passes import compile_graph
        from ..sim import simulate
        g, pool, _ = Q.build_graph(d, lambda name: 0, a.maxlen)
        plan = compile_graph(g, "b200", {"POOL": len(pool.bytes())})
        tl = Timeline.from_sim(plan, simulate(plan))
    else:
        import os
        import torch
        from ..models import decode as D
        from . import dist as RD
        rank, world, local = RD.rank_env(os.environ)
        dev = torch.device("cuda", local)
        torch.cuda.set_device(dev)
        w = D.random_packed_weights(d, a.maxlen, dev, seed=0)
        if a.batch > 1:
            from ..models import batched as BT
            prog = BT.BatchProgram(d, w, a.batch, device=local, maxlen=a.maxlen)
            prog.buf["kc"].normal_(0, 0.02); prog.buf["vc"].normal_(0, 0.02)
            prog.buf["token_in"].random_(0, 1000)
            torch.cuda.synchronize(dev)
            for t in range(min(a.warm, 8)):
                prog.step(0, a.context + t, False)
            prog.session.set_option("trace", 1)
            prog.step(1, a.context + 9, False)
            print(Timeline.from_trace(prog.plan, prog.session.trace()).text())
            prog.close()
            return 0
        if world > 1:
            # under torchrun: ONE request sharded over the ranks (the timeline of rank 0 is printed)
            import torch.distributed as dist
            dist.init_process_group("gloo")
            prog = D.DecodeProgram(Q.shard_dims(d, world), Q.shard_weights(w, d, world, rank), device=local, maxlen=a.maxlen, ranks=world, rank=rank)
            prog.session.set_option("timeout_ms", 10000)
            RD.connect_ranks(prog, dist)
        else:
            prog = D.DecodeProgram(d, w, device=local, maxlen=a.maxlen)
        prog.buf["kc"].normal_(0, 0.02); prog.buf["vc"].normal_(0, 0.02)
        for t in range(a.warm):
            prog.buf["token_in"][0] = 7
            prog.step(0, a.context + (t % 8), False, wait=(t % 32 == 31))
        prog.session.wait(60.0)
        prog.session.set_option("trace", 1)
        prog.step(0, a.context + 9, False)
        tl = Timeline.from_trace(prog.plan, prog.session.trace())
        if world > 1:
            RD.close_ranks(prog, dist)
            dist.destroy_process_group()
            if rank != 0:
                return 0
        else:
            prog.close()
    print(tl.text())
    if a.raw:
        tl.write_raw(a.raw)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
