"""compile_graph: verify -> instantiate -> enumerate tasks -> lay out event counters -> static per-worker queues ->
verify_plan.  Same entry point and result type as the reference (etx/passes/pipeline.py:15-42); the passes that only
make sense on a multi-XCD part (P2 affinity, P3 recomputation, P4 modes, P5 relay, P6 placement) collapse into the
single static schedule below, with the decision recorded per grid as the reference does."""
from __future__ import annotations

import copy
from typing import Any, Mapping

from ..ir.dims import eval_expr
from ..ir.instantiate import instantiate
from ..ir.types import Graph, Scope
from ..ir.verify import verify
from ..machine.model import MachineModel, load_machine
from .plan import EventPlan, PassOptions, Plan, TaskInst, verify_plan


def compile_graph(graph: Graph, machine: MachineModel | str = "b200", bindings: Mapping[str, int] | None = None,
                  runtime: Mapping[str, Any] | None = None, options: PassOptions | None = None) -> Plan:
    m = load_machine(machine) if isinstance(machine, str) else machine
    options = options or PassOptions()
    bindings = dict(bindings or {})
    if options.force_mode not in (None, "static"):
        raise ValueError("only static scheduling is built for this backend")
    g = copy.deepcopy(graph)
    verify(g, bindings, runtime)
    if any(gr.device != 0 for gr in g.grids):
        raise ValueError("one plan covers one device; compile each rank's graph separately")
    inst = instantiate(g, bindings, runtime)
    plan = Plan(arch=m.name, graph=g, inst=inst, machine=m, bindings=bindings, options=options, runtime=runtime)
    W = options.workers or m.workers()
    if W > m.workers():
        raise ValueError(f"{W} workers requested but {m.name} keeps only {m.workers()} persistent CTAs co-resident")
    plan.workers_per_domain, plan.n_domains, plan.wg_per_cu = W, 1, 1
    # event counters: one word per coordinate, event tensors laid out in declaration order
    off = 0
    for e in g.events.values():
        shape = inst.event_shapes[e.name]
        n = 1
        for d in shape:
            n *= d
        ep = EventPlan(name=e.name, shape=shape, scope=m.effective_scope(e.scope or Scope.DEVICE), offset=off, numel=n)
        plan.events[e.name] = ep
        off += n
    plan.event_words = off
    for e in plan.events.values():
        e.counts = [0] * e.numel
    for (ev, c), prods in inst.producers.items():
        plan.events[ev].counts[plan.linear(ev, c)] = len(prods)
    for (ev, c), want in inst.wait_counts.items():
        have = plan.events[ev].counts[plan.linear(ev, c)]
        if want != have:
            raise RuntimeError(f"event {ev}{list(c)}: declared wait_count {want} but {have} tasks arrive")
    # tasks in program order; worker = by worker_map when given, else round-robin inside the grid
    for ti, gr in enumerate(g.grids):
        plan.type_ids[gr.name] = ti
        plan.modes[gr.name] = "static"
        plan.reasons[gr.name] = "static: single coherent L2, barrier-chain decode graph"
        for n, c in enumerate(inst.tasks[gr.name]):
            if gr.worker_map:
                lhs, rhs = gr.worker_map.replace(" ", "").split("->")
                w = eval_expr(rhs.strip("()"), {**bindings, **dict(zip(lhs, c))}) % W
            else:
                w = n % W
            t = TaskInst(id=len(plan.tasks), grid=gr.name, coord=c, type_id=ti, worker=w, duration_us=gr.duration_us)
            plan.task_index[(gr.name, c)] = t.id
            plan.tasks.append(t)
            plan.static_queues.setdefault((0, w), []).append(t.id)
    for w in range(W):
        plan.static_queues.setdefault((0, w), [])
    plan.task_in_words = [[plan.word(ev, c) for ev, c in inst.task_in[(t.grid, t.coord)]] for t in plan.tasks]
    plan.task_out_words = [[plan.word(ev, c) for ev, c in inst.task_out[(t.grid, t.coord)]] for t in plan.tasks]
    errors = verify_plan(plan)
    if errors:
        raise RuntimeError("plan verification failed:\n  " + "\n  ".join(errors))
    plan.say(f"{len(plan.tasks)} tasks on {W} workers, {plan.event_words} event counters, no per-step reset (monotonic counters)")
    return plan
