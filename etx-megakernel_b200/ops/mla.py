"""Absorbed multi-head latent attention (DeepSeek-V2 family) as an ETX op: one task per (head, partition of 128 positions).

It stands where the reference's DeepSeek-V2-Lite graph runs q_absorb, the chunked attention and merge_uv
(examples/dsv2lite/graph.py:98-209).  The 128-byte block (grid words at 112):

  qkv       bf16 [NH * (DN + DR) + C + DR]   the q heads (nope | rope part each), then the kv_a row (latent | k_pe)
  kvln      bf16 [C]                         weight of the latent's RMSNorm
  cos_sin   fp32 [maxlen][2 * DR]            rotary table rows: cos | sin (YaRN scaling already applied)
  wkvb      bf16 [NH * (DN + DV)][C]         kv_b_proj: per head DN rows of W_UK, then DV rows of W_UV
  cache     bf16 [maxlen][C + DR]            the layer's latent cache (row `pos` is written by head 0's task)
  positions int64 [1],  out bf16 [NH * DV]
  tmp       (value, flag) pairs [NH][max_parts][C + 8] (8 bytes each): the partitions' partial results; the task of the
            four finishing tasks per head merge them and apply a quarter of W_UV each.  max_parts * 128 >= maxlen; grid =
            (max_parts + 4) * NH tasks (task = partition * NH + head, then the finishing tasks); tag = a number that differs between the grids sharing tmp (the layer)
"""
from __future__ import annotations

from ._layout import entry

ARG_BYTES, GRID_OFF = 128, 112
PART = 128
FINISHERS = 4            # finishing tasks per head, after the partition tasks in the grid
MAX_CTX = 8192
PARAMS = [("qkv", "ptr addrspace(1)", 0, 8), ("kvln", "ptr addrspace(1)", 8, 8), ("cos_sin", "ptr addrspace(1)", 16, 8),
          ("wkvb", "ptr addrspace(1)", 24, 8), ("cache", "ptr addrspace(1)", 32, 8), ("positions", "ptr addrspace(1)", 40, 8),
          ("out", "ptr addrspace(1)", 48, 8), ("NH", "i32", 56, 4), ("C", "i32", 60, 4), ("DN", "i32", 64, 4), ("DR", "i32", 68, 4),
          ("DV", "i32", 72, 4), ("maxlen", "i32", 76, 4), ("scale", "float", 80, 4), ("eps", "float", 84, 4),
          ("tmp", "ptr addrspace(1)", 88, 8), ("max_parts", "i32", 96, 4), ("tag", "i32", 100, 4)]


def import_entries(threads: int = 544) -> dict:
    return {"mla_attn": entry("mla_attn", "mla_attn", PARAMS, ARG_BYTES, GRID_OFF, threads, "absorbed multi-head latent attention, one (head, 128 positions) per task, merged by the last partition's task")}


def partitions(maxlen: int) -> int:
    return -(-maxlen // PART)


def tmp_pairs(NH: int, C: int, maxlen: int) -> int:
    """8-byte pairs of the partial-result buffer."""
    return NH * partitions(maxlen) * (C + 8)


def check_shape(NH: int, C: int, DN: int, DR: int, DV: int, maxlen: int) -> None:
    """The limits of the tile's shared-memory layout (csrc/etxb_mla.cuh)."""
    if not (1 <= NH and 8 <= C <= 512 and C % 8 == 0 and 1 <= DN and DN + DR <= 256 and 8 <= DR <= 64 and DR % 8 == 0 and C + DR <= 640 and DV >= 1):
        raise ValueError(f"mla_attn: needs C <= 512 and DR <= 64 (multiples of 8), DN + DR <= 256 (NH={NH}, C={C}, DN={DN}, DR={DR}, DV={DV})")
    if not 1 <= maxlen <= MAX_CTX:
        raise ValueError(f"mla_attn: context {maxlen} outside 1..{MAX_CTX}")
