"""Split-KV paged GQA decode attention and its merge as ETX ops (exports attn_decode, attn_reduce).

The reference imports vLLM's paged_attention kernels for this phase (call recipe etx/importer/spec.py:243-244, grid
(1, parts, NKV) + reduce grid NH, examples/vllm_llm/model.py:78-84, 358-362); these tiles are this library's own, so
the block layout is too: 128 bytes, grid words at 112.  attn_decode task blk = part * NKV + h covers 32 positions;
partials are fp32 (max logit, exp sum, unnormalised output per q head and partition); attn_reduce task = q head."""
from __future__ import annotations

from ._layout import entry

ARG_BYTES, GRID_OFF = 128, 112
PART = 32
PARAMS = [("q", "ptr addrspace(1)", 0, 8), ("kc", "ptr addrspace(1)", 8, 8), ("vc", "ptr addrspace(1)", 16, 8),
          ("block_tables", "ptr addrspace(1)", 24, 8), ("seq_lens", "ptr addrspace(1)", 32, 8),
          ("exp_sums", "ptr addrspace(1)", 40, 8), ("max_logits", "ptr addrspace(1)", 48, 8), ("tmp_out", "ptr addrspace(1)", 56, 8),
          ("out", "ptr addrspace(1)", 64, 8), ("scale", "float", 72, 4), ("NH", "i32", 76, 4), ("NKV", "i32", 80, 4),
          ("HD", "i32", 84, 4), ("BS", "i32", 88, 4), ("X", "i32", 92, 4), ("max_parts", "i32", 96, 4), ("max_blocks", "i32", 100, 4)]


def import_entries(threads: int = 512) -> dict:
    return {e: entry(e, e, PARAMS, ARG_BYTES, GRID_OFF, threads, spec)
            for e, spec in (("attn_decode", "paged GQA decode attention, 32 positions x one kv head per task"),
                            ("attn_reduce", "merge of the attention partitions of one q head"))}


def check_shape(NH: int, NKV: int, HD: int, BS: int, X: int, max_parts: int) -> None:
    if NH % NKV or NH // NKV > 16:
        raise ValueError(f"attn_decode: G = NH / NKV must be an integer <= 16, got {NH}/{NKV}")
    if HD % 16 or HD > 256 or X != 8:
        raise ValueError(f"attn_decode: head_dim {HD} must be a multiple of 16, at most 256, with X = 8")
    if BS not in (16, 32):
        raise ValueError(f"attn_decode: block size {BS} not in (16, 32)")
    if not 1 <= max_parts <= 4096:
        raise ValueError(f"attn_decode: max_parts {max_parts} outside 1..4096 (context <= 131072)")
