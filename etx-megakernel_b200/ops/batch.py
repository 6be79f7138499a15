"""The tiles of a batched decode step (several sequences per step) as ETX ops: argument-block layouts and exports.

Column-batched dense GEMV and the per-column norm keep the reference's 160-byte GEMV block with its column strides
(etx/ops/gemv.py:40-73, 80-94: nb, sx, sout, srows, srin, srout -- element counts); the expert-grouped tiles read the
same block with `rows` = the per-expert token lists and `resid_in` = their lengths; the routing tile and the per-column
prologue / argmax have small blocks of their own.

  norm_col      task b: z = bf16(resid_in[b] + the R rows of column b added in bf16 in ascending id order),
                x[b] = rmsnorm(z) * ln, resid_out[b] = z                     (R = 0: no rows; ids = null: rows in order)
  gemv_nb       out[b][r] = bf16(W[r,:] . x[b] (+ bias)), rows [blk * rpt, ...), all nb columns per weight read
  route         softmax top-k of every column; elist[e][0 .. ecount[e]) = (column << 8 | slot) pairs that selected expert e;
                *active += the number of experts with a non-empty list (what the byte ledger of a batched step needs).
                elist = 0: one task per column that only writes the column's ids / wts
  moe_up_g      task (expert e, row chunk): act[b][slot][r] for every (b, slot) of e's list
  moe_down_g    task (expert e, row chunk): y[b][slot][r] = bf16(bf16(W2_e[r,:] . act[b][slot]) * wts[b][slot])
  gemv_tc       the dense grid on tcgen05.mma (K % 64 == 0); `ln` is filled by the library with the address of the grid's TMA
                tensor map.  tpe = S > 1 splits K: task blk = (row block blk // S, K-slice blk % S), fp32 partials in `rows`
                ([S][M][nb]), arrival counters in `resid_in`; the S-th arrival of a row block sums the slices in order
  moe_up_tc, moe_down_tc   the expert grids on tcgen05.mma, scheduled by share: nblocks = workers, task blk takes an equal
                share of (active experts x row tiles); ids = the step's routing ids [nb][R] (the tiles build the
                per-expert lists themselves), E set; moe_up_tc's resid_out = optional counter += active experts
  prologue_nb   task b: residual <- embedding row of column b's token, positions / slot of column b
  argmax_nb     task b: greedy token of column b
"""
from __future__ import annotations

from . import gemv as _gemv
from ._layout import entry

NB_MAX = 64                 # columns of a batched step
ROUTE_BYTES, ROUTE_GRID = 88, 72
ROUTE_PARAMS = [("logits", "ptr addrspace(1)", 0, 8), ("wts", "ptr addrspace(1)", 8, 8), ("ids", "ptr addrspace(1)", 16, 8),
                ("ecount", "ptr addrspace(1)", 24, 8), ("elist", "ptr addrspace(1)", 32, 8), ("active", "ptr addrspace(1)", 40, 8),
                ("E", "i32", 48, 4), ("K", "i32", 52, 4), ("mode", "i32", 56, 4), ("nb", "i32", 60, 4), ("cap", "i32", 64, 4)]
COLS_BYTES, COLS_GRID = 32, 16
COLS_PARAMS = [("nb", "i32", 0, 4), ("slot_span", "i32", 4, 4), ("zero", "ptr addrspace(1)", 8, 8)]
SPLITK_COUNTERS = 768       # int32 arrival counters `zero` names (cleared by column 0's prologue task every step)
TC_ROWS = 256               # weight rows one tcgen05 instruction takes (two TMA boxes of 128)
XBYTES = 40960              # shared memory for the token vectors of a pass: min(8, XBYTES // (2 K + 64)) columns per pass
GROUP_ROWS = 128            # weight rows a block of the tensor-core loop covers


def import_entries(threads: int = 544) -> dict:
    out = {e: entry(e, e, _gemv.PARAMS, _gemv.ARG_BYTES, _gemv.GRID_OFF, threads, spec)
           for e, spec in (("norm_col", "residual add + expert combine + RMSNorm of one column"),
                           ("gemv_nb", "bf16 GEMV, nb activation columns per weight read (mma.sync)"),
                           ("moe_up_g", "expert-grouped gate+up with SiLU*mul"), ("moe_down_g", "expert-grouped down, scaled"),
                           ("gemv_tc", "bf16 GEMV, up to 32 columns per weight read (tcgen05.mma, TMA, tensor memory)"),
                           ("moe_up_tc", "expert-grouped gate+up on tcgen05"), ("moe_down_tc", "expert-grouped down on tcgen05"))}
    out["route"] = entry("route", "route", ROUTE_PARAMS, ROUTE_BYTES, ROUTE_GRID, threads, "softmax top-k per column + per-expert token lists")
    out["cols"] = entry("cols", "cols", COLS_PARAMS, COLS_BYTES, COLS_GRID, threads, "per-column prologue / argmax of a batched step")
    return out


def check_batch(nb: int, K: int) -> None:
    if not 1 <= nb <= NB_MAX:
        raise ValueError(f"batched step: {nb} columns outside 1..{NB_MAX}")
    if K % 8 or XBYTES // (2 * K + 64) < 1:
        raise ValueError(f"batched GEMV: K={K} must be a multiple of 8 and one token vector must fit {XBYTES} bytes")


def split_k(M: int, K: int, workers: int) -> tuple:
    """(tasks, rows per task, K-split) of a dense tcgen05 grid: row blocks of TC_ROWS (128 for a matrix of at most 128 rows),
    and the largest power-of-two split of K up to 8 (slices of at least 256 columns: the task that arrives last adds
    the slices' partial sums, which it reads from L2) that keeps the grid within one wave of the workers.  A matrix with a wave of row blocks of its own is not split."""
    rpt = TC_ROWS if M > 128 else 128
    blocks = -(-M // rpt)
    if blocks >= workers:
        rpt = -(-(-(-M // workers)) // 128) * 128
        return -(-M // rpt), rpt, 1
    S = 1
    while S < 8 and blocks * S * 2 <= workers and K % (64 * S * 2) == 0 and K // (S * 2) >= 256:
        S *= 2
    return blocks * S, rpt, S
