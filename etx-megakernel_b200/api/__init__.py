"""The public planning surface: `plan(PlanRequest) -> PlannedWorkload`, `simulate(planned, seed=)` (etx/api/__init__.py:211-218).

Two workload kinds plan here: "model" (a decode program of one of the bundled model configurations, or of an inline HF-style
config) and "graph" (a declarative graph: tensors, events and grids whose bodies name built-in tiles).  Planning needs no
GPU; the results are detached records (JSON values with a content identity).
"""
from __future__ import annotations

from collections.abc import Mapping
from dataclasses import fields

from .types import (SCHEMA_VERSION, Configuration, PlanRequest, PlannedWorkload, SimulationResult, WorkloadSpec)  # noqa: F401


def model(name: str, *, config: Mapping) -> WorkloadSpec:
    return WorkloadSpec(name=name, kind="model", config=Configuration(config))


def graph(name: str, *, config: Mapping) -> WorkloadSpec:
    return WorkloadSpec(name=name, kind="graph", config=Configuration(config))


def _compile(request: PlanRequest):
    from ..frontends import cuda_link
    from ..ir import Graph
    from ..machine import list_archs, load_machine
    from ..passes import PassOptions, compile_graph
    if not isinstance(request, PlanRequest):
        raise TypeError("plan requires PlanRequest")
    if request.target not in list_archs():
        raise ValueError(f"unknown packaged target {request.target!r}")
    opts = request.options.to_dict()
    unknown = set(opts) - {f.name for f in fields(PassOptions)}
    if unknown:
        raise ValueError(f"unknown planner options: {sorted(unknown)}")
    machine = load_machine(request.target)
    w = request.workload
    cfg = w.config.to_dict()
    if w.kind == "model":
        from ..models import qwen as Q
        unknown = set(cfg) - {"model", "hf_config", "layers", "maxlen", "fold_topk", "fused_attn"}
        if unknown:
            raise ValueError(f"unknown model configuration fields: {sorted(unknown)}")
        d = Q.load_dims(cfg.get("hf_config") or cfg.get("model", w.name), layers=cfg.get("layers"))
        g, pool, _ = Q.build_graph(d, lambda name: 0, int(cfg.get("maxlen", 1072)), machine, fold_topk=cfg.get("fold_topk", True),
                                   fused_attn=cfg.get("fused_attn", True))
        bindings = {"POOL": len(pool.bytes()), **request.bindings.to_dict()}
    elif w.kind == "graph":
        unknown = set(cfg) - {"tensors", "events", "grids"}
        if unknown:
            raise ValueError(f"unknown graph configuration fields: {sorted(unknown)}")
        g = Graph(w.name)
        for rec in cfg.get("tensors", []):
            g.tensor(**rec)
        for rec in cfg.get("events", []):
            g.etensor(**rec)
        for rec in cfg.get("grids", []):
            rec = dict(rec)
            body = rec.pop("body")
            g.call_device(rec.pop("name"), tuple(rec.pop("grid")), cuda_link(body.get("source", ""), body["symbol"]),
                          consts=tuple(rec.pop("consts", ())), **rec)
        if not g.grids:
            raise ValueError("graph requires at least one grid")
        bindings = request.bindings.to_dict()
    else:
        raise ValueError(f"no planning provider for workload kind {w.kind!r}")
    return compile_graph(g, machine, bindings, request.runtime.to_dict() or None, options=PassOptions(**opts)), machine


def plan(request: PlanRequest) -> PlannedWorkload:
    p, machine = _compile(request)
    from ..passes import verify_plan
    report = {"tasks": len(p.tasks), "workers": p.workers_per_device(), "event_words": p.event_words,
              "grids": {g.name: len(p.inst.tasks[g.name]) for g in p.graph.grids}, "modes": dict(p.modes),
              "verify": verify_plan(p)}
    return PlannedWorkload(request=request, machine={"name": machine.name, "workers": machine.workers()},
                           options=request.options.to_dict(), report=report, decisions=tuple(str(x) for x in p.log))


def simulate(planned: PlannedWorkload, *, seed: int = 0) -> SimulationResult:
    if not isinstance(planned, PlannedWorkload):
        raise TypeError("simulate requires PlannedWorkload")
    from ..sim import simulate as run
    p, _ = _compile(planned.request)
    r = run(p, seed=seed)
    return SimulationResult(plan_identity=planned.identity, seed=seed, deadlock=r.deadlock, blocked=tuple(r.blocked),
                            metrics={"makespan_us": r.makespan_us, "busy_us": r.busy_us, "wait_us": r.wait_us, "sched_us": r.sched_us,
                                     "utilisation": r.utilisation, "workers": r.n_workers, "per_grid_us": r.per_grid_us})
