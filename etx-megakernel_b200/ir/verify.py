"""Graph verification before anything is planned.

The check names, the `Issue` record and `VerifyError` are the interface (the reference's verifier, etx/ir/verify.py:
53-151, reports under the same names so that callers can filter on them):

  exists         an edge names an event the graph declares
  acyclic        every waited event has a producer, producers come earlier in launch order, no grid reaches itself
  count          the arrivals the edge maps deliver to an event coordinate equal its declared wait count
  runtime-first  whatever is only known at run time (a tensor an edge map reads, an event's counts) is written by a grid
                 that both precedes its user and is ordered before it by a chain of events
  coverage       a tensor has one writer grid

Structure here: a launch-order table and a transitive closure over the event edges are built once; each check is a
generator of issues over those two tables, run in sequence (the count check needs the enumeration, so it is skipped
when the structural checks already failed).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Iterator, Mapping

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
        super().__init__("\n".join(str(i) for i in self.issues))


class _Order:
    """Launch positions and event-path reachability between grids."""

    def __init__(self, graph: Graph):
        self.pos = {g.name: n for n, g in enumerate(graph.grids)}
        direct = {g.name: {c.name for ev in g.out_edges for c in graph.consumers_of(ev)} for g in graph.grids}
        # transitive closure by repeated squaring of the successor sets (graphs here have tens to hundreds of grids)
        reach = {n: set(s) for n, s in direct.items()}
        grew = True
        while grew:
            grew = False
            for n, s in reach.items():
                more = set().union(*(reach[m] for m in s)) - s if s else set()
                if more:
                    s |= more
                    grew = True
        self.after = reach

    def before(self, a: str, b: str) -> bool:
        return self.pos[a] < self.pos[b]

    def ordered(self, a: str, b: str) -> bool:
        """b is reached from a through events."""
        return b in self.after[a]


def _structure(graph: Graph, order: _Order) -> Iterator[Issue]:
    for g in graph.grids:
        for ev in g.out_edges:
            if ev not in graph.events:
                yield Issue("exists", f"grid {g.name!r} notifies unknown event {ev!r}")
        for ev in g.in_edges:
            if ev not in graph.events:
                yield Issue("exists", f"grid {g.name!r} waits on unknown event {ev!r}")
                continue
            sources = graph.producers_of(ev)
            if not sources:
                yield Issue("acyclic", f"event {ev!r} consumed by {g.name!r} has no producer")
            for src in sources:
                if not order.before(src.name, g.name):
                    yield Issue("acyclic", f"grid {g.name!r} waits on {ev!r} produced by later grid {src.name!r} (cycle or forward reference)")
    for name in order.pos:
        if order.ordered(name, name):
            yield Issue("acyclic", f"grid {name!r} reaches itself")


def _counts(graph: Graph, order: _Order, inst) -> Iterator[Issue]:
    for name, ev in graph.events.items():
        off = [key for key, who in inst.producers.items() if key[0] == name and len(who) != inst.wait_counts[key]]
        if not ev.is_runtime_count:
            for key in off[:3]:
                yield Issue("count", f"event {name}{list(key[1])}: wait_count={inst.wait_counts[key]} but {len(inst.producers[key])} producers notify it")
            if len(off) > 3:
                yield Issue("count", f"event {name!r}: {len(off)} coordinates with mismatched counts (first 3 shown)")
            continue
        init = ev.runtime_init_by
        if init is None:
            yield Issue("count", f"event {name!r}: its wait count is only known at run time, so it must name the grid that writes the counts (runtime_init_by)")
        elif init not in order.pos:
            yield Issue("count", f"event {name!r}: runtime_init_by names {init!r}, which is not a grid of this graph")
        else:
            for user in graph.consumers_of(name):
                if not order.before(init, user.name):
                    yield Issue("count", f"event {name!r}: {init!r} writes the counts, but its consumer {user.name!r} is launched no later")
        if ev.runtime_count is not None and off:
            key = off[0]
            yield Issue("count", f"event {name}{list(key[1])}: the runtime_count expression says {inst.wait_counts[key]} arrivals, the edge maps "
                                 f"deliver {len(inst.producers[key])} ({len(off)} coordinates disagree)")


def _runtime_first(graph: Graph, order: _Order) -> Iterator[Issue]:
    writers: dict = {}
    for g in graph.grids:
        for t in g.writes:
            writers.setdefault(t, []).append(g.name)
    for g in graph.grids:
        needed = {t for emap in (*g.in_edges.values(), *g.out_edges.values()) for t in emap.runtime}
        for t in sorted(needed):
            if t not in writers:
                yield Issue("runtime-first", f"runtime tensor {t!r} used by {g.name!r} is written by no grid")
            for w in writers.get(t, ()):
                if not order.before(w, g.name):
                    yield Issue("runtime-first", f"runtime tensor {t!r}: its writer {w!r} is launched no earlier than its user {g.name!r}")
                elif not order.ordered(w, g.name):
                    yield Issue("runtime-first", f"runtime tensor {t!r}: no chain of events orders its user {g.name!r} after its writer {w!r}")
    for name, ev in graph.events.items():
        init = ev.runtime_init_by
        if ev.is_runtime_count and init in order.pos:
            for user in graph.consumers_of(name):
                if user.name != init and not order.ordered(init, user.name):
                    yield Issue("runtime-first", f"event {name!r}: no chain of events orders its consumer {user.name!r} after {init!r}, which writes its counts")


def _coverage(graph: Graph) -> Iterator[Issue]:
    owners: dict = {}
    for g in graph.grids:
        for t in g.writes:
            owners.setdefault(t, []).append(g.name)
    for t, names in owners.items():
        if len(names) > 1:
            yield Issue("coverage", f"tensor {t!r} written by {names}; each output must have exactly one writer grid")


def verify(graph: Graph, bindings: Mapping[str, int], runtime: Mapping[str, Any] | None = None, strict: bool = True) -> list:
    """All issues found (strict: raise VerifyError when any is an error)."""
    order = _Order(graph)
    issues = list(_structure(graph, order))
    if not issues:
        try:
            inst = instantiate(graph, bindings, runtime)
        except KeyError as e:
            issues.append(Issue("instantiate", str(e)))
        else:
            issues += _counts(graph, order, inst)
            issues += _runtime_first(graph, order)
            issues += _coverage(graph)
    if strict and any(i.severity == "error" for i in issues):
        raise VerifyError(issues)
    return issues
