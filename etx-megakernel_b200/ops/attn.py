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


# the fused phase (export attn_fused): q/k norm + rope + cache write of the new position, attention over the partition,
# and the merge.  General form: by the last task of each kv head to finish (counters: one int32 per kv head, monotonic,
# never reset).  Grouped form: by the task of the context's last partition, which polls the partials the others publish
# as flagged (value, step flag) pairs in `tmp_out` -- [NH][max_parts][GQ_PARTIAL_FLOATS] floats, zeroed once by the
# caller; exp_sums, max_logits and counters are not used by it
F_ARG_BYTES, F_GRID_OFF = 176, 160
F_PARAMS = [("qkv", "ptr addrspace(1)", 0, 8), ("qw", "ptr addrspace(1)", 8, 8), ("kw", "ptr addrspace(1)", 16, 8),
            ("cos_sin", "ptr addrspace(1)", 24, 8), ("kc", "ptr addrspace(1)", 32, 8), ("vc", "ptr addrspace(1)", 40, 8),
            ("block_tables", "ptr addrspace(1)", 48, 8), ("seq_lens", "ptr addrspace(1)", 56, 8), ("positions", "ptr addrspace(1)", 64, 8),
            ("slot_mapping", "ptr addrspace(1)", 72, 8), ("exp_sums", "ptr addrspace(1)", 80, 8), ("max_logits", "ptr addrspace(1)", 88, 8),
            ("tmp_out", "ptr addrspace(1)", 96, 8), ("out", "ptr addrspace(1)", 104, 8), ("counters", "ptr addrspace(1)", 112, 8),
            ("scale", "float", 120, 4), ("eps", "float", 124, 4), ("NH", "i32", 128, 4), ("NKV", "i32", 132, 4), ("HD", "i32", 136, 4),
            ("BS", "i32", 140, 4), ("X", "i32", 144, 4), ("max_parts", "i32", 148, 4),
            # gq > 0: the grouped form -- a task is gq q heads of one kv head x part_len (128) positions, task index
            # part * (NH / gq) + group, one counter per group; gq = 0: the general form (32 positions x one kv head)
            ("gq", "i32", 152, 4), ("part_len", "i32", 156, 4)]
GQ_PART = 128
GQ_WHOLE = 1 << 24
RING_BYTES = 6 * 24576     # shared memory of the weight ring, where the whole-sequence form keeps its partials


def tagged_part_len(tag: int, whole: bool = False) -> int:
    """part_len word of a grouped attention block: 128 positions per task, and in bits 16..23 a tag that differs between the
    grids of a step that share the partial buffers (the layer index): a merger only accepts partials carrying its own.
    whole: bit 24, the form with one task per (sequence, q group) that walks all partitions itself -- for plans without
    streamed tiles (the batched step), whose idle weight ring holds the partials."""
    return GQ_PART | ((tag & 0xff) << 16) | (GQ_WHOLE if whole else 0)


def whole_sequence_fits(gq: int, max_parts: int) -> bool:
    return 65536 + max_parts * gq * 130 * 4 <= RING_BYTES      # a partition of K / V pieces + the partials


GQ_PARTIAL_FLOATS = 272   # grouped form: floats of `tmp_out` per (q head, partition) -- 136 (value, flag) pairs: 128 outputs, max, sum, padding


def import_entries(threads: int = 544) -> dict:
    out = {e: entry(e, e, PARAMS, ARG_BYTES, GRID_OFF, threads, spec)
           for e, spec in (("attn_decode", "paged GQA decode attention, 32 positions x one kv head per task"),
                           ("attn_reduce", "merge of the attention partitions of one q head"))}
    out["attn_fused"] = entry("attn_fused", "attn_fused", F_PARAMS, F_ARG_BYTES, F_GRID_OFF, threads,
                              "q/k norm + rope + cache write + paged GQA decode attention + merge, one phase")
    return out


def check_fused(NH: int, NKV: int, HD: int, BS: int, X: int, max_parts: int, gq: int = 0, part_len: int = 0) -> None:
    check_shape(NH, NKV, HD, BS, X, max_parts)
    G = NH // NKV
    if gq:
        if gq not in (1, 2, 4, 8) or G % gq or HD != 128 or BS != 16 or (part_len & 0xffff) != GQ_PART or part_len >> 25:
            raise ValueError(f"attn_fused grouped form: needs gq in (1, 2, 4, 8) dividing G={G}, head_dim 128, block size 16 and "
                             f"part_len {GQ_PART} (gq={gq}, HD={HD}, BS={BS}, part_len={part_len})")
        if gq * max_parts > 4096:
            raise ValueError(f"attn_fused grouped form: gq * max_parts = {gq * max_parts} exceeds 4096")
        return
    if G + 2 > 16 or G * HD > 2048 or HD % 32:
        raise ValueError(f"attn_fused: needs G + 2 <= 16 warps, G * HD <= 2048 and HD % 32 == 0 (G={G}, HD={HD})")
    if G * max_parts > 8192:
        raise ValueError(f"attn_fused: G * max_parts = {G * max_parts} exceeds 8192 (context too long for the in-tile merge)")


def check_shape(NH: int, NKV: int, HD: int, BS: int, X: int, max_parts: int) -> None:
    if NH % NKV or NH // NKV > 16:
        raise ValueError(f"attn_decode: G = NH / NKV must be an integer <= 16, got {NH}/{NKV}")
    if HD % 16 or HD > 256 or X != 8:
        raise ValueError(f"attn_decode: head_dim {HD} must be a multiple of 16, at most 256, with X = 8")
    if BS not in (16, 32):
        raise ValueError(f"attn_decode: block size {BS} not in (16, 32)")
    if not 1 <= max_parts <= 4096:
        raise ValueError(f"attn_decode: max_parts {max_parts} outside 1..4096 (context <= 131072)")
