"""The router's softmax + top-k as an ETX op (export dsl_topk): the reference's 64-byte block, grid words at 48
(etx/ops/topk.py:16-23).  mode: 0 softmax top-k, 1 renormalised over the selected k; | 0x100 round the weights to bf16
(the numerics of the reference's CPU path, examples/llm/ref_numpy.py:136-141).  One warp per activation column,
E <= 256, K <= 16; ties go to the lower expert index."""
from __future__ import annotations

from ._layout import entry

ARG_BYTES, GRID_OFF = 64, 48
PARAMS = [("logits", "ptr addrspace(1)", 0, 8), ("wts", "ptr addrspace(1)", 8, 8), ("ids", "ptr addrspace(1)", 16, 8),
          ("tei", "ptr addrspace(1)", 24, 8), ("E", "i32", 32, 4), ("K", "i32", 36, 4), ("mode", "i32", 40, 4),
          ("nbsv", "i32", 44, 4)]
MAX_E, MAX_K = 256, 16


def import_entries(threads: int = 512) -> dict:
    return {"dsl_topk": entry("dsl_topk", "topk", PARAMS, ARG_BYTES, GRID_OFF, threads, "ETX DSL softmax top-k")}


def check_shape(E: int, K: int) -> None:
    if not 1 <= E <= MAX_E or not 1 <= K <= min(E, MAX_K):
        raise ValueError(f"dsl_topk: E={E}, K={K} outside 1 <= K <= min(E, {MAX_K}), E <= {MAX_E}")
