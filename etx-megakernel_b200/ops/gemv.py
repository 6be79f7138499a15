"""The streaming bf16 GEMV family as an ETX op: argument-block layout and export table.

The layout is the reference's, byte for byte (etx/ops/gemv.py:80-94: 25 parameters, 160 bytes, grid words at 144, type
string "pppppliiiippppifiipiiiiii"), so a host that fills blocks for the reference's dsl_gemv / dsl_moe_up / dsl_moe_down
tiles fills them for the sm_100a tiles unchanged.  The tile bodies are CUDA (csrc/etxb_gemv.cuh), not generated text.

Forms:
  dsl_gemv[_fold]       out[r] = bf16(W[r,:] . x)  rows [blk*rpt, ...) of W [M, K]; fold: x = rmsnorm(bf16(resid + rows))
  dsl_moe_up[_fold]     act[s, r] = bf16(bf16(silu(bf16 g)) * bf16 u), expert e = ids[s]; fold: top-k recomputed in-tile
  dsl_moe_down[_fold]   out[s, r] = bf16(bf16(W_e[r,:] . act_s) * wts[s])
mode: 0 plain, 1 norm fold, 2 / 3 top-k fold without / with renormalisation; | 0x100 bf16 routing weights (the numerics
of the reference's CPU path), | 0x200 bf16 bias row passed in `wts` (plain form), | 0x400 MoE down: the task covers
every slot and writes out[r] = the slots' results added in bf16 in ascending expert id (the expert combine), bits
16..23 expert slots per task (task blk -> slots [blk / tpe * spt, ...), row chunk blk % tpe); | 0x1000 sharded model:
`rows` names a [ranks][.] block of flagged 4-byte words (bf16 value | step flag << 16) -- an exchanged plain / down grid
publishes the rows it wrote into row `rank` of it on every rank, a norm fold reads its R = ranks rows from it.
"""
from __future__ import annotations

from ._layout import entry

ARG_BYTES, GRID_OFF = 160, 144
PARAMS = [("W", "ptr addrspace(1)", 0, 8), ("x", "ptr addrspace(1)", 8, 8), ("out", "ptr addrspace(1)", 16, 8),
          ("ids", "ptr addrspace(1)", 24, 8), ("wts", "ptr addrspace(1)", 32, 8), ("estride", "i64", 40, 8),
          ("M", "i32", 48, 4), ("K", "i32", 52, 4), ("rpt", "i32", 56, 4), ("tpe", "i32", 60, 4),
          ("rows", "ptr addrspace(1)", 64, 8), ("resid_in", "ptr addrspace(1)", 72, 8), ("resid_out", "ptr addrspace(1)", 80, 8),
          ("ln", "ptr addrspace(1)", 88, 8), ("R", "i32", 96, 4), ("eps", "float", 100, 4), ("mode", "i32", 104, 4),
          ("E", "i32", 108, 4), ("logits", "ptr addrspace(1)", 112, 8),
          ("nb", "i32", 120, 4), ("sx", "i32", 124, 4), ("sout", "i32", 128, 4), ("srows", "i32", 132, 4),
          ("srin", "i32", 136, 4), ("srout", "i32", 140, 4)]
FORMS = {"dsl_gemv": "plain", "dsl_moe_up": "silu_mul", "dsl_moe_down": "scale",
         "dsl_gemv_fold": "plain", "dsl_moe_up_fold": "silu_mul", "dsl_moe_down_fold": "scale"}
MODE_NORM, MODE_TOPK, MODE_TOPK_RENORM, MODE_BF16_WTS, MODE_BIAS, MODE_SUM_SLOTS, MODE_ROUTE_READY = 1, 2, 3, 0x100, 0x200, 0x400, 0x800
MODE_FLAGGED = 0x1000      # sharded model: `rows` is a [ranks][M or K] block of flagged words (see build_graph(ranks=...))


def mode_shared(ns: int) -> int:
    """Always-on experts of a top-k fold, carried in mode bits 24..27: ns experts stored after the E routed ones take the last
    ns of the R slots with weight 1 (DeepSeek's shared experts); the fold picks the other R - ns from the logits."""
    if not 0 <= ns <= 15:
        raise ValueError("0 <= shared experts <= 15")
    return ns << 24


def mode_spt(spt: int) -> int:
    """Expert slots per task of the MoE forms, carried in mode bits 16..23 (0 and 1 both mean one slot per task)."""
    return (spt & 0xff) << 16
THREADS = 544              # 16 consumer warps + the producer warp of the persistent CTA
MAX_K = 12288              # a streamed row (and its bf16 activation vector in shared memory)
MAX_K_NORM = 8192          # the norm fold works on fp32 in shared memory
MAX_RESULTS = 2048         # row results one MoE task holds in shared memory (ranges x rows per range)
NB_ALLOWED = (1, 2, 4, 8)
NB_STAGE_BYTES = 200 * 1024 - 32768   # stand-alone batched GEMV (nb > 1): nb token rows of K bf16 (+ 64 bytes each) staged in shared memory


def type_string() -> str:
    return "".join({"ptr addrspace(1)": "p", "i64": "l", "i32": "i", "float": "f"}[ty] for _, ty, _, _ in PARAMS)


def import_entries(threads: int = THREADS) -> dict:
    return {e: entry(e, form, PARAMS, ARG_BYTES, GRID_OFF, threads, f"ETX DSL GEMV ({form})") for e, form in FORMS.items()}


def check_shape(export: str, *, M: int, K: int, rpt: int, nb: int = 1, mode: int = 0) -> None:
    """Host-side guard of what the CUDA tiles support; raises before anything is packed."""
    nb = max(nb, 1)
    if K % 8:
        raise ValueError(f"{export}: K={K} must be a multiple of 8 (16-byte weight vectors)")
    if nb not in NB_ALLOWED:
        raise ValueError(f"{export}: nb={nb} activation columns; supported {NB_ALLOWED}")
    if nb > 1:
        if FORMS[export] != "plain" or (mode & 0xff):
            raise ValueError(f"{export}: nb > 1 is built for the plain stand-alone GEMV only")
        if nb > 8 or nb * (2 * K + 64) > NB_STAGE_BYTES or rpt > 1024:
            raise ValueError(f"{export}: batched form takes nb <= 8, nb * (2 K + 64) <= {NB_STAGE_BYTES} bytes of staged activations and "
                             f"at most 1024 rows per task (nb={nb}, K={K}, rpt={rpt})")
    elif K > MAX_K:
        raise ValueError(f"{export}: K={K} exceeds {MAX_K} (one row must fit a 24 KB ring stage)")
    if (mode & 0xff) == MODE_NORM and K > MAX_K_NORM:
        raise ValueError(f"{export}: norm fold over K={K} > {MAX_K_NORM}")
    spt = ((mode >> 16) & 0xff) or 1
    if FORMS[export] == "silu_mul" and 2 * spt * rpt > MAX_RESULTS:
        raise ValueError(f"{export}: 2 * {spt} slots * rpt={rpt} row results exceed {MAX_RESULTS}")
    if FORMS[export] == "scale" and (spt * rpt > MAX_RESULTS or spt * K > MAX_K):
        raise ValueError(f"{export}: {spt} slots per task: results {spt * rpt} > {MAX_RESULTS} or activations {spt * K} > {MAX_K}")
    if FORMS[export] == "plain" and (mode & (MODE_SUM_SLOTS | 0xff0000)):
        raise ValueError(f"{export}: slot bits are for the MoE forms only")
    if rpt < 1 or M < 1:
        raise ValueError(f"{export}: M and rpt must be positive")
