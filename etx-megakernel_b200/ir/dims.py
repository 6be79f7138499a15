"""Symbolic dimensions: a dimension is an int or an integer expression over symbol names ("B*H", "cdiv(S, 128)").

Same grammar and helper set as the reference (etx/ir/dims.py:1-102): + - * / // % **, unary minus, cdiv / max / min /
ceil / floor, and subscripts of runtime tensors ("indptr[i+1]") when a runtime mapping is supplied.  Evaluation walks
the Python AST and refuses everything else.
"""
from __future__ import annotations

import ast
import math
import operator
from typing import Any, Mapping

Dim = int | str

HELPERS = {"cdiv": lambda a, b: -(-a // b), "max": max, "min": min, "ceil": math.ceil, "floor": math.floor}
_OPS = {ast.Add: operator.add, ast.Sub: operator.sub, ast.Mult: operator.mul, ast.FloorDiv: operator.floordiv,
        ast.Div: operator.floordiv, ast.Mod: operator.mod, ast.Pow: operator.pow}


def eval_expr(src, env: Mapping[str, int], runtime: Mapping[str, Any] | None = None) -> int:
    text = str(src).strip()
    rt = runtime or {}

    def walk(n):
        if isinstance(n, ast.Expression):
            return walk(n.body)
        if isinstance(n, ast.Constant):
            if isinstance(n.value, bool) or not isinstance(n.value, int):
                raise ValueError(f"only integer constants are allowed in {text!r}")
            return n.value
        if isinstance(n, ast.Name):
            if n.id not in env:
                raise KeyError(f"unbound symbol {n.id!r} in {text!r}")
            return int(env[n.id])
        if isinstance(n, ast.UnaryOp) and isinstance(n.op, ast.USub):
            return -walk(n.operand)
        if isinstance(n, ast.BinOp):
            fn = _OPS.get(type(n.op))
            if fn is None:
                raise ValueError(f"unsupported operator {type(n.op).__name__} in {text!r}")
            return fn(walk(n.left), walk(n.right))
        if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id in HELPERS and not n.keywords:
            return int(HELPERS[n.func.id](*map(walk, n.args)))
        if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name):
            if n.value.id not in rt:
                raise KeyError(f"runtime tensor {n.value.id!r} not provided for {text!r}")
            sl = n.slice
            val = rt[n.value.id]
            for i in ([walk(e) for e in sl.elts] if isinstance(sl, ast.Tuple) else [walk(sl)]):
                val = val[i]
            return int(val)
        raise ValueError(f"unsupported expression node {type(n).__name__} in {text!r}")

    return walk(ast.parse(text, mode="eval"))


def eval_dim(d: Dim, bindings: Mapping[str, int]) -> int:
    if isinstance(d, bool):
        raise TypeError("bool is not a dimension")
    if isinstance(d, int):
        return d
    v = eval_expr(d, bindings)
    if v < 0:
        raise ValueError(f"dimension {d!r} evaluated to {v} < 0")
    return v


def eval_shape(shape, bindings: Mapping[str, int]) -> tuple[int, ...]:
    return tuple(eval_dim(d, bindings) for d in shape)


def free_symbols(d: Dim) -> set[str]:
    if isinstance(d, int):
        return set()
    names, tensors = set(), set()
    for n in ast.walk(ast.parse(str(d), mode="eval")):
        if isinstance(n, ast.Subscript) and isinstance(n.value, ast.Name):
            tensors.add(n.value.id)
        elif isinstance(n, ast.Name) and n.id not in HELPERS:
            names.add(n.id)
    return names - tensors
