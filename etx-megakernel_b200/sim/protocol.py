"""Host-side model of how the persistent kernel runs a plan (the role of etx/sim/protocol.py:62-210).

Every worker (persistent CTA) walks its static queue in order; a task starts when the worker is free AND every event
it waits on has received all its arrivals (plus the signalling latency of the machine model); it then runs for its
annotated duration and arrives on its out-events.  That is exactly the loop of `etxb_megakernel`, without the data.
Used before anything touches a GPU:

  * deadlock detection: which tasks could never start and which event they were waiting on (a task queued behind its
    own consumer, an event whose count can never be reached);
  * makespan, per-worker busy / wait time and a per-task schedule that `runtime.timeline` analyses like a measured trace.

It is a model: durations come from the tile annotations (`duration_us`, jittered by `duration_cv`), signalling from
the machine's cost table.  Scheduling is static only (the B200 runtime has no dynamic queues).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field

from ..ir.types import Scope
from ..passes.plan import Plan


@dataclass
class Segment:
    device: int
    worker: int
    start: float
    end: float
    kind: str           # "task" | "wait"
    task: int = -1


@dataclass
class SimResult:
    makespan_us: float
    segments: list
    deadlock: bool
    blocked: list
    busy_us: float
    wait_us: float
    sched_us: float
    n_workers: int
    per_grid_us: dict = field(default_factory=dict)
    taken: dict = field(default_factory=dict)     # task id -> time its worker reached it
    ready: dict = field(default_factory=dict)     # task id -> time it started
    done: dict = field(default_factory=dict)      # task id -> time it finished

    @property
    def utilisation(self) -> float:
        return self.busy_us / max(1e-9, self.makespan_us * self.n_workers)

    def summary(self) -> str:
        s = (f"makespan {self.makespan_us:.1f} us | busy {self.busy_us:.1f} wait {self.wait_us:.1f} sched {self.sched_us:.1f} "
             f"| utilisation {self.utilisation * 100:.1f}% over {self.n_workers} workers")
        if self.deadlock:
            s += "\nDEADLOCK: " + "; ".join(self.blocked[:8])
        return s


def simulate(plan: Plan, seed: int = 0, cv_scale: float = 1.0) -> SimResult:
    """Run the plan's static queues to completion (or until nothing can move)."""
    rng = random.Random(seed)
    inst, m = plan.inst, plan.machine
    t_sig = m.t_sync_us(Scope.DEVICE)
    grids = {g.name: g for g in plan.graph.grids}
    queues = {k: list(q) for k, q in plan.static_queues.items()}
    head = {k: 0 for k in queues}
    free = {k: 0.0 for k in queues}
    arrivals: dict = {}                       # event instance -> arrival times so far
    need = {ev: int(c) for ev, c in inst.wait_counts.items()}
    res = SimResult(0.0, [], False, [], 0.0, 0.0, 0.0, len(queues))

    complete: dict = {}                       # event instance -> time it was satisfied (cached once reached)

    def event_time(ev):
        """Time at which `ev` has all its arrivals, or None."""
        if ev in complete:
            return complete[ev]
        got = arrivals.get(ev, [])
        n = need.get(ev, len(inst.producers.get(ev, ())))
        if len(got) < n:
            return None
        complete[ev] = (sorted(got)[n - 1] if n else 0.0) + t_sig
        return complete[ev]

    progress = True
    while progress:
        progress = False
        # the worker whose head task can start earliest goes first, so arrivals are generated in time order
        best = None
        for k, q in queues.items():
            if head[k] >= len(q):
                continue
            t = plan.tasks[q[head[k]]]
            times = [event_time(ev) for ev in inst.task_in[(t.grid, t.coord)]]
            if any(x is None for x in times):
                continue
            start = max([free[k], *times])
            if best is None or start < best[0]:
                best = (start, k)
        if best is None:
            break
        start, k = best
        tid = queues[k][head[k]]
        t = plan.tasks[tid]
        g = grids[t.grid]
        dur = max(0.0, g.duration_us * (1.0 + cv_scale * g.duration_cv * rng.gauss(0.0, 1.0))) if g.duration_cv else g.duration_us
        end = start + dur
        if start > free[k]:
            res.segments.append(Segment(k[0], k[1], free[k], start, "wait", tid))
            res.wait_us += start - free[k]
        res.segments.append(Segment(k[0], k[1], start, end, "task", tid))
        res.busy_us += dur
        res.per_grid_us[t.grid] = res.per_grid_us.get(t.grid, 0.0) + dur
        res.taken[tid], res.ready[tid], res.done[tid] = free[k], start, end
        for ev in inst.task_out[(t.grid, t.coord)]:
            arrivals.setdefault(ev, []).append(end)
        free[k] = end
        head[k] += 1
        progress = True
    res.makespan_us = max(free.values(), default=0.0)
    for k, q in queues.items():
        if head[k] < len(q):
            res.deadlock = True
            t = plan.tasks[q[head[k]]]
            missing = [f"{ev[0]}{list(ev[1])} {len(arrivals.get(ev, []))}/{need.get(ev, '?')}"
                       for ev in inst.task_in[(t.grid, t.coord)] if event_time(ev) is None]
            res.blocked.append(f"worker {k}: task {q[head[k]]} ({t.grid}{list(t.coord)}) waits for {', '.join(missing)}")
    return res
