"""Enumerate a symbolic graph for concrete bindings: every task, every event coordinate, who arrives / waits where.

Same result type as the reference (etx/ir/instantiate.py:22-83): the plan, the verifier and the simulator all read it.
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field
from typing import Any, Mapping

from .dims import eval_dim, eval_expr, eval_shape
from .types import Graph

TaskId = tuple
EvId = tuple


@dataclass
class Instance:
    bindings: dict
    grid_shapes: dict = field(default_factory=dict)
    event_shapes: dict = field(default_factory=dict)
    tasks: dict = field(default_factory=dict)
    producers: dict = field(default_factory=dict)
    consumers: dict = field(default_factory=dict)
    task_in: dict = field(default_factory=dict)
    task_out: dict = field(default_factory=dict)
    wait_counts: dict = field(default_factory=dict)

    def n_tasks(self) -> int:
        return sum(map(len, self.tasks.values()))

    def all_tasks(self) -> list:
        return [(g, c) for g, cs in self.tasks.items() for c in cs]


def _coords(shape):
    return list(itertools.product(*map(range, shape)))


def instantiate(graph: Graph, bindings: Mapping[str, int], runtime: Mapping[str, Any] | None = None) -> Instance:
    inst = Instance(bindings=dict(bindings))
    rt = runtime or {}
    for e in graph.events.values():
        shape = inst.event_shapes[e.name] = eval_shape(e.shape, bindings)
        for c in _coords(shape):
            inst.producers[(e.name, c)] = []
            inst.consumers[(e.name, c)] = []
    for g in graph.grids:
        shape = inst.grid_shapes[g.name] = eval_shape(g.grid, bindings)
        inst.tasks[g.name] = _coords(shape)
        for c in inst.tasks[g.name]:
            tid = (g.name, c)
            outs = inst.task_out[tid] = []
            ins = inst.task_in[tid] = []
            for ev, m in g.out_edges.items():
                for t in m.targets(c, inst.event_shapes[ev], rt, bindings):
                    outs.append((ev, t)); inst.producers[(ev, t)].append(tid)
            for ev, m in g.in_edges.items():
                for t in m.targets(c, inst.event_shapes[ev], rt, bindings):
                    ins.append((ev, t)); inst.consumers[(ev, t)].append(tid)
    for e in graph.events.values():
        for c in _coords(inst.event_shapes[e.name]):
            key = (e.name, c)
            if e.runtime_count is not None:
                inst.wait_counts[key] = eval_expr(e.runtime_count, {**bindings, **dict(zip("ijkl", c))}, rt)
            elif e.is_runtime_count:
                inst.wait_counts[key] = len(inst.producers[key])
            else:
                inst.wait_counts[key] = eval_dim(e.wait_count, bindings)
    return inst
