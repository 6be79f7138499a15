"""Graph verification: the four checks of the reference (etx/ir/verify.py:53-151).

1 acyclic      every waited event is produced by an EARLIER grid, no grid reaches itself
2 count        arrivals enumerated from the edge maps equal the declared wait_count at every event coordinate
3 runtime      a runtime tensor used by an edge map / runtime count is written by an earlier grid on a dependency path
4 coverage     one writer grid per tensor
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .instantiate import instantiate
from .types import Graph


@dataclass
class Issue:
    check: str
    message: str
    severity: str = "error"

    def __str__(self):
        return f"[{self.check}] {self.message}"


class VerifyError(Exception):
    def __init__(self, issues):
        self.issues = list(issues)
        super().__init__("\n".join(map(str, self.issues)))


def _reachable(graph: Graph) -> dict:
    succ = {g.name: set() for g in graph.grids}
    for g in graph.grids:
        for ev in g.out_edges:
            succ[g.name].update(c.name for c in graph.consumers_of(ev))
    reach = {}
    for name in succ:
        seen, todo = set(), list(succ[name])
        while todo:
            n = todo.pop()
            if n not in seen:
                seen.add(n)
                todo.extend(succ[n])
        reach[name] = seen
    return reach


def verify(graph: Graph, bindings: Mapping[str, int], runtime: Mapping[str, Any] | None = None, strict: bool = True) -> list:
    issues: list[Issue] = []
    order = {g.name: i for i, g in enumerate(graph.grids)}

    def done():
        if strict and any(i.severity == "error" for i in issues):
            raise VerifyError(issues)
        return issues

    for g in graph.grids:
        for ev in g.in_edges:
            if ev not in graph.events:
                issues.append(Issue("exists", f"grid {g.name!r} waits on unknown event {ev!r}"))
                continue
            producers = graph.producers_of(ev)
            if not producers:
                issues.append(Issue("acyclic", f"event {ev!r} consumed by {g.name!r} has no producer"))
            for p in producers:
                if order[p.name] >= order[g.name]:
                    issues.append(Issue("acyclic", f"grid {g.name!r} waits on {ev!r} produced by later grid {p.name!r} (cycle or forward reference)"))
        for ev in g.out_edges:
            if ev not in graph.events:
                issues.append(Issue("exists", f"grid {g.name!r} notifies unknown event {ev!r}"))
    reach = _reachable(graph)
    issues += [Issue("acyclic", f"grid {n!r} reaches itself") for n, r in reach.items() if n in r]
    if issues:
        return done()
    try:
        inst = instantiate(graph, bindings, runtime)
    except KeyError as e:
        issues.append(Issue("instantiate", str(e)))
        return done()

    for name, e in graph.events.items():
        coords = [k for k in inst.producers if k[0] == name]
        if e.is_runtime_count:
            if e.runtime_init_by is None:
                issues.append(Issue("count", f"event {name!r} has runtime wait_count but no runtime_init_by grid"))
            elif e.runtime_init_by not in order:
                issues.append(Issue("count", f"event {name!r} runtime_init_by unknown grid {e.runtime_init_by!r}"))
            else:
                for c in graph.consumers_of(name):
                    if order[e.runtime_init_by] >= order[c.name]:
                        issues.append(Issue("count", f"event {name!r} counts written by {e.runtime_init_by!r} after consumer {c.name!r}"))
            if e.runtime_count is not None:
                bad = [k for k in coords if len(inst.producers[k]) != inst.wait_counts[k]]
                if bad:
                    k = bad[0]
                    issues.append(Issue("count", f"event {name}{list(k[1])}: runtime_count gives {inst.wait_counts[k]} but "
                                                 f"{len(inst.producers[k])} producers notify it ({len(bad)} coords)"))
            continue
        bad = [k for k in coords if len(inst.producers[k]) != inst.wait_counts[k]]
        for k in bad[:3]:
            issues.append(Issue("count", f"event {name}{list(k[1])}: wait_count={inst.wait_counts[k]} but {len(inst.producers[k])} producers notify it"))
        if len(bad) > 3:
            issues.append(Issue("count", f"event {name!r}: {len(bad)} coordinates with mismatched counts (first 3 shown)"))

    for g in graph.grids:
        for m in (*g.in_edges.values(), *g.out_edges.values()):
            for rt in m.runtime:
                writers = [w for w in graph.grids if rt in w.writes]
                if not writers:
                    issues.append(Issue("runtime-first", f"runtime tensor {rt!r} used by {g.name!r} is written by no grid"))
                for w in writers:
                    if order[w.name] >= order[g.name]:
                        issues.append(Issue("runtime-first", f"runtime tensor {rt!r} is written by {w.name!r} after it is used by {g.name!r}"))
                    elif g.name not in reach[w.name]:
                        issues.append(Issue("runtime-first", f"{g.name!r} reads runtime tensor {rt!r} but no event path orders it after writer {w.name!r}"))
    for name, e in graph.events.items():
        if e.is_runtime_count and e.runtime_init_by in order:
            for c in graph.consumers_of(name):
                if c.name != e.runtime_init_by and c.name not in reach[e.runtime_init_by]:
                    issues.append(Issue("runtime-first", f"event {name!r} counts are initialised by {e.runtime_init_by!r} but consumer {c.name!r} is not ordered after it"))

    by_tensor: dict = {}
    for g in graph.grids:
        for t in g.writes:
            by_tensor.setdefault(t, []).append(g.name)
    issues += [Issue("coverage", f"tensor {t!r} written by {ws}; each output must have exactly one writer grid")
               for t, ws in by_tensor.items() if len(ws) > 1]
    return done()
