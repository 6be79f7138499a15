"""Attention preparation of one kv head as an ETX op (export dsl_attnprep): the reference's 112-byte block, grid
words at 96 (etx/ops/attnprep.py:11-15).  One task per kv head: q/k RMSNorm (skipped when the norm weight pointer is
null) + neox rotary in place on qkv, k and v rows into the paged cache (key [blocks][NKV][HD/X][BS][X], value
[blocks][NKV][HD][BS], slot = slot_mapping[0])."""
from __future__ import annotations

from ._layout import entry

ARG_BYTES, GRID_OFF = 112, 96
PARAMS = [("qkv", "ptr addrspace(1)", 0, 8), ("qw", "ptr addrspace(1)", 8, 8), ("kw", "ptr addrspace(1)", 16, 8),
          ("cos_sin", "ptr addrspace(1)", 24, 8), ("positions", "ptr addrspace(1)", 32, 8), ("kc", "ptr addrspace(1)", 40, 8),
          ("vc", "ptr addrspace(1)", 48, 8), ("slot_mapping", "ptr addrspace(1)", 56, 8),
          ("NH", "i32", 64, 4), ("NKV", "i32", 68, 4), ("HD", "i32", 72, 4), ("eps", "float", 76, 4), ("BS", "i32", 80, 4), ("X", "i32", 84, 4)]


def import_entries(threads: int = 512) -> dict:
    return {"dsl_attnprep": entry("dsl_attnprep", "attnprep", PARAMS, ARG_BYTES, GRID_OFF, threads,
                                  "ETX DSL attention prep (q/k norm + rope + cache write of one kv head)")}


def check_shape(NH: int, NKV: int, HD: int, BS: int, X: int) -> None:
    if NH % NKV or NH // NKV + 2 > 16:
        raise ValueError(f"dsl_attnprep: needs G + 2 <= 16 warps, got NH={NH}, NKV={NKV}")
    if HD % 32 or HD > 256 or X != 8 or HD % X:
        raise ValueError(f"dsl_attnprep: head_dim {HD} must be a multiple of 32, at most 256, with X = 8")
    if BS not in (16, 32):
        raise ValueError(f"dsl_attnprep: block size {BS} not in (16, 32)")
