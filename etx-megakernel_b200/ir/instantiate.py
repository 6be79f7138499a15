"""Enumerate a symbolic graph for concrete bindings: every task, every event coordinate, who arrives / waits where.

The record type (`Instance`, its field names and key shapes) is the interface the plan, the verifier and the simulator
read, and matches the reference's (etx/ir/instantiate.py:22-83).  The enumeration here works edge by edge: for every
(grid, event, direction) it expands the edge map over the whole grid once and files each (task, event coordinate) pair
on both sides, then the expected arrival count of every coordinate is resolved from the event's declaration.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

import numpy as np

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
        return sum(len(v) for v in self.tasks.values())

    def all_tasks(self) -> list:
        out = []
        for grid, coords in self.tasks.items():
            out.extend((grid, c) for c in coords)
        return out


def _cells(shape) -> list:
    """Every coordinate of a box, in row-major order, as tuples of Python ints."""
    if not shape:
        return [()]
    return [tuple(int(v) for v in idx) for idx in np.ndindex(*shape)]


def _expected(event, coord, bindings, runtime, arrivals: int) -> int:
    if event.runtime_count is not None:                                   # an expression over the coordinate and runtime tensors
        scope = dict(bindings)
        scope.update(zip("ijkl", coord))
        return eval_expr(event.runtime_count, scope, runtime)
    if event.is_runtime_count:                                            # counted on the device: whatever the edges deliver
        return arrivals
    return eval_dim(event.wait_count, bindings)


def instantiate(graph: Graph, bindings: Mapping[str, int], runtime: Mapping[str, Any] | None = None) -> Instance:
    runtime = runtime or {}
    inst = Instance(bindings=dict(bindings))
    for name, ev in graph.events.items():
        inst.event_shapes[name] = eval_shape(ev.shape, bindings)
        for cell in _cells(inst.event_shapes[name]):
            inst.producers[(name, cell)], inst.consumers[(name, cell)] = [], []
    for grid in graph.grids:
        inst.grid_shapes[grid.name] = eval_shape(grid.grid, bindings)
        cells = inst.tasks[grid.name] = _cells(inst.grid_shapes[grid.name])
        for cell in cells:
            inst.task_out[(grid.name, cell)], inst.task_in[(grid.name, cell)] = [], []
        # arrivals first, then waits: the per-task lists keep the declaration order of the edges
        for edges, per_task, per_event in ((grid.out_edges, inst.task_out, inst.producers), (grid.in_edges, inst.task_in, inst.consumers)):
            for ev_name, emap in edges.items():
                box = inst.event_shapes[ev_name]
                for cell in cells:
                    task = (grid.name, cell)
                    for target in emap.targets(cell, box, runtime, bindings):
                        per_task[task].append((ev_name, target))
                        per_event[(ev_name, target)].append(task)
    for name, ev in graph.events.items():
        for cell in _cells(inst.event_shapes[name]):
            inst.wait_counts[(name, cell)] = _expected(ev, cell, bindings, runtime, len(inst.producers[(name, cell)]))
    return inst
