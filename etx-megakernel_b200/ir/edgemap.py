"""Edge maps: task coordinate -> event coordinate(s).

The grammar is the reference's (etx/ir/edgemap.py:1-17):
  "ij->i"  "h->bh"                      letters; a letter only on the right broadcasts over that event axis
  "ij->(i/2)j"                          parenthesised integer expressions over the left letters and graph symbols
  "i->range(indptr[i], indptr[i+1])"    runtime range over a rank-1 event
  "i->topk[i,:]"                        runtime gather (one row of a runtime tensor)
  "*"                                   every coordinate of the event
There is no code emission here: the plan enumerates `targets()` per task and ships the resulting event lists, and a
runtime map is evaluated from the sample the caller gives (the device-side evaluation of runtime maps is not built).
"""
from __future__ import annotations

import itertools
import re
from dataclasses import dataclass
from typing import Any, Mapping, Sequence

from .dims import eval_expr

_RANGE = re.compile(r"^range\((.+),(.+)\)$")
_GATHER = re.compile(r"^(\w+)\[(.+),\s*:\s*\]$")


def _split_rhs(rhs: str, lhs: tuple[str, ...], text: str):
    items, i = [], 0
    while i < len(rhs):
        ch = rhs[i]
        if ch == "(":
            depth, j = 1, i + 1
            while j < len(rhs) and depth:
                depth += (rhs[j] == "(") - (rhs[j] == ")")
                j += 1
            if depth:
                raise ValueError(f"unbalanced parentheses in {text!r}")
            expr = rhs[i + 1:j - 1]
            for name in re.findall(r"[A-Za-z_]\w*", expr):
                if len(name) == 1 and name.islower() and name not in lhs:
                    raise ValueError(f"expression letter {name!r} not in lhs of {text!r}")
            items.append(("expr", expr))
            i = j
        elif ch.isalpha():
            items.append(("idx" if ch in lhs else "bcast", ch))
            i += 1
        else:
            raise ValueError(f"unexpected {ch!r} in edge map {text!r}")
    return tuple(items)


@dataclass(frozen=True)
class EdgeMap:
    text: str
    kind: str                                   # affine | range | gather | all
    lhs: tuple[str, ...] = ()
    items: tuple[tuple[str, str], ...] = ()
    runtime: tuple[str, ...] = ()
    range_lo: str = ""
    range_hi: str = ""
    gather_tensor: str = ""
    gather_row: str = ""

    @staticmethod
    def parse(text: str) -> "EdgeMap":
        t = text.replace(" ", "")
        if t == "*":
            return EdgeMap(text=text, kind="all")
        if "->" not in t:
            raise ValueError(f"edge map {text!r} must contain '->'")
        left, rhs = t.split("->", 1)
        lhs = tuple(left)
        if not all(c.isalpha() for c in lhs):
            raise ValueError(f"edge map lhs must be single letters: {text!r}")
        m = _RANGE.match(rhs)
        if m:
            lo, hi = m.groups()
            names = tuple(sorted(set(re.findall(r"(\w+)\[", lo + " " + hi))))
            return EdgeMap(text=text, kind="range", lhs=lhs, runtime=names, range_lo=lo, range_hi=hi)
        m = _GATHER.match(rhs)
        if m:
            return EdgeMap(text=text, kind="gather", lhs=lhs, runtime=(m.group(1),), gather_tensor=m.group(1), gather_row=m.group(2))
        if rhs == "()":
            return EdgeMap(text=text, kind="affine", lhs=lhs)
        return EdgeMap(text=text, kind="affine", lhs=lhs, items=_split_rhs(rhs, lhs, text))

    @property
    def is_runtime(self) -> bool:
        return self.kind in ("range", "gather")

    def event_rank(self) -> int | None:
        return {"affine": len(self.items), "range": 1, "gather": 1}.get(self.kind)

    def targets(self, coord: Sequence[int], event_shape: Sequence[int], runtime: Mapping[str, Any] | None = None,
                bindings: Mapping[str, int] | None = None) -> list[tuple[int, ...]]:
        env = dict(bindings or {})
        env.update(zip(self.lhs, map(int, coord)))                # coordinates shadow symbols
        if self.kind == "all":
            return list(itertools.product(*map(range, event_shape)))
        if self.kind == "affine":
            if len(self.items) != len(event_shape):
                raise ValueError(f"{self.text!r} produces rank {len(self.items)} but event has rank {len(event_shape)}")
            axes = []
            for (kind, payload), n in zip(self.items, event_shape):
                axes.append([env[payload]] if kind == "idx" else [eval_expr(payload, env)] if kind == "expr" else list(range(n)))
            return list(itertools.product(*axes))
        if self.kind == "range":
            return [(t,) for t in range(eval_expr(self.range_lo, env, runtime), eval_expr(self.range_hi, env, runtime))]
        if runtime is None or self.gather_tensor not in runtime:
            raise KeyError(f"runtime tensor {self.gather_tensor!r} required by {self.text!r}")
        return [(int(v),) for v in runtime[self.gather_tensor][eval_expr(self.gather_row, env)]]
