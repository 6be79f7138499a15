"""Batched decode: B sequences per step through ONE persistent launch (softmax top-k MoE models of the Qwen family).

What this takes over from the reference: request batching inside the megakernel (examples/vllm_llm/model.py:194-211 --
dense nodes emitted once for all requests with NB activation columns per weight read, attention per sequence, top-k one
column per wave, buffers / KV caches / argument blocks per request, weights shared) and the column-batched GEMV
(etx/ops/gemv.py:40-73).  The reference keeps one expert task per (request, slot), so an expert chosen by several
requests is streamed once per request; here the expert phases are grouped by EXPERT: a routing tile lists, per expert,
the (sequence, slot) pairs that selected it, and the gate+up / down tiles read an expert's rows once for all of them.

Phases per layer (one event after each):
  norm1 (B tasks: residual add + expert combine of the previous layer in ascending expert id + input RMSNorm)
  -> qkv (column-batched GEMV) -> attention (per sequence: the one-phase tile, grid (tasks, B), one argument block per
  sequence) -> o_proj (batched) -> norm2 (B tasks) -> router (batched) -> route (1 task: top-k per column + token lists)
  -> moe_up (expert-grouped) -> moe_down (expert-grouped)
then final norm (B tasks) -> lm_head (batched) -> argmax (B tasks).  All sequences of a step are at the same position
(prompts of one length, as the benchmark's); every sequence has its own KV blocks in a shared block pool.
"""
from __future__ import annotations

import numpy as np
import torch

from ..frontends import cuda_link
from ..importer import argblock
from ..ir import Graph, Resource
from ..machine import MachineModel, load_machine
from ..ops import attn as op_attn
from ..ops import batch as op_batch
from ..ops import gemv as op_gemv
from ..passes import PassOptions, compile_graph
from ..runtime import Session
from . import qwen as Q
from .qwen import BS, SRC, X, ArgPool

_DT = {"bf16": torch.bfloat16, "f32": torch.float32, "i32": torch.int32, "i64": torch.int64}
UP_ROWS, DOWN_ROWS = 256, 512      # mma.sync engine: rows of one expert a gate+up / down task covers (blocks of 128 inside the tile)
SKP_FLOATS = 4 << 20               # fp32 partial sums of a split-K dense grid ([split][rows][B])


def buffer_shapes(d: Q.Dims, B: int, maxlen: int, steps: int, parts: int) -> dict:
    """name -> (shape, dtype) of the activation / runtime buffers of B sequences (column b of every [B, ...] buffer
    belongs to sequence b; the KV block pool gives sequence b the blocks [b * nblk, (b + 1) * nblk))."""
    nblk = -(-maxlen // BS)
    return {"resid": ((B, d.H), "bf16"), "resid2": ((B, d.H), "bf16"), "hn": ((B, d.H), "bf16"), "qkv": ((B, d.NQKV), "bf16"),
            "attn_out": ((B, d.NH * d.HD), "bf16"), "o": ((B, d.H), "bf16"), "o_norm": ((B, d.H), "bf16"), "logits": ((B, d.V), "bf16"),
            "positions": ((B,), "i64"), "seq_lens": ((B,), "i32"), "slot_mapping": ((B,), "i64"), "block_tables": ((B, nblk), "i32"),
            "token_in": ((steps + 2, B), "i32"), "token_out": ((steps + 1, B), "i32"), "token_time": ((2 * (steps + 1),), "i64"),
            "exp_sums": ((B, d.NH, parts), "f32"), "max_logits": ((B, d.NH, parts), "f32"),
            "tmp_out": ((B, d.NH, parts, op_attn.GQ_PARTIAL_FLOATS), "f32"),
            "kc": ((d.L, B * nblk, d.NKV, d.HD // X, BS, X), "bf16"), "vc": ((d.L, B * nblk, d.NKV, d.HD, BS), "bf16"),
            "attn_counters": ((d.L, B, d.NH), "i32"), "rlog": ((B, d.E), "bf16"), "tw": ((B, d.TOPK), "f32"), "ti": ((B, d.TOPK), "i32"),
            "mc2": ((B, d.TOPK, d.MI), "bf16"), "mc3": ((B, d.TOPK, d.H), "bf16"), "ecount": ((d.E,), "i32"), "elist": ((d.E, B), "i32"), "active": ((d.L,), "i32"),
            "skp": ((SKP_FLOATS,), "f32"), "skc": ((op_batch.SPLITK_COUNTERS,), "i32")}


def build_graph(d: Q.Dims, ptr, B: int, maxlen: int = 1072, machine: MachineModel | str = "b200", engine: str = "tc"):
    """The batched decode step of `d` for B sequences as a Graph plus its argument pool.  ptr(name) -> device address of
    a buffer (buffer_shapes) or packed weight (models.qwen.weight_shapes).  Returns (graph, pool, info).

    engine: what multiplies the batched grids (dense projections, expert gate+up / down) -- "tc": tcgen05.mma with TMA tensor
    copies and accumulators in tensor memory (needs every K a multiple of 64); "mma": the mma.sync tiles that read their
    weights straight from global memory.  Same grids, same argument blocks, same results up to fp32 summation order."""
    if engine not in ("tc", "mma"):
        raise ValueError("engine is 'tc' or 'mma'")
    if engine == "tc" and any(k % 64 for k in (d.H, d.NH * d.HD, d.MI)):
        engine = "mma"
    if not d.moe:
        raise ValueError("the batched step is built for the softmax top-k MoE models")
    if d.HD != 128 or d.G not in (1, 2, 4, 8):
        raise ValueError("the batched step uses the grouped attention tile: head_dim 128 and 1, 2, 4 or 8 q heads per kv head")
    op_batch.check_batch(B, max(d.H, d.NH * d.HD))
    m = load_machine(machine) if isinstance(machine, str) else machine
    ent = {}
    for mod in (op_gemv, op_attn, op_batch):
        ent.update(mod.import_entries())
    g = Graph(f"vlb{B}_{d.name}")
    g.codegen.update(nb=B, requests=B)
    g.tensor("impargs", ("POOL",), role="weight", bytes_per_elem=1)
    pool = ArgPool()
    res = Resource(threads=op_gemv.THREADS, vgpr=128, lds_bytes=0)
    nblk = -(-maxlen // BS)
    kv_layer_bytes = B * nblk * d.NKV * d.HD * BS * 2
    W = m.workers()
    gq, plen, gparts = d.G, op_attn.GQ_PART, -(-maxlen // op_attn.GQ_PART)      # one task per (128 positions, kv head): K / V read once
    # enough sequences to fill the workers: one task per (sequence, kv head) walks the whole context; else one per partition
    whole = B * (d.NH // gq) >= W // 2 and op_attn.whole_sequence_fits(gq, gparts)
    ntask = (d.NH // gq) if whole else gparts * (d.NH // gq)
    op_attn.check_fused(d.NH, d.NKV, d.HD, BS, X, gparts, gq, plen)
    scale = float(np.float32(1.0 / np.sqrt(d.HD)))
    state = {"prev": None}

    def add(name, symbol, blob, grid, n_out, two_d=False, stride=0):
        off = pool.add(blob)
        pool.rows.append((name, symbol, "", 0, off, n_out, 0, 0))
        ev = "E_" + name
        g.etensor(ev, (1,), wait_count=n_out)
        imap = "ij->(0)" if two_d else "i->(0)"
        g.call_device(name, grid, cuda_link(SRC, symbol), resource=res, args=["impargs"], consts=(off, stride),
                      in_edges={state["prev"]: imap} if state["prev"] else {}, out_edges={ev: imap})
        state["prev"] = ev

    def gb(export, tasks, **f):
        return argblock.pack_named(ent[export], (tasks, 1, 1), **f)

    def norm(name, rows, R, ids, srows, rin, rout, x, ln):
        add(name, "etx_tile_norm_col", gb("norm_col", B, x=ptr(x), rows=ptr(rows) if rows else 0, resid_in=ptr(rin), resid_out=ptr(rout) if rout else 0,
                                          ln=ln, ids=ptr(ids) if ids else 0, R=R, K=d.H, M=d.H, rpt=1, tpe=1, eps=d.eps, nb=B, sx=d.H, srows=srows,
                                          srin=d.H, srout=d.H), (B,), B)

    skc = {"n": 0}                                                     # arrival counters handed out so far; grids of one shape share theirs

    def dense(name, Wp, x, out, M, K, bias=0):
        mode = op_gemv.MODE_BIAS if bias else 0
        if engine == "tc":
            # row blocks of 256 (one instruction's worth); narrow matrices are also cut along K to fill the workers
            t, rpt, S = op_batch.split_k(M, K, W)
            blocks = t // S
            if S > 1 and ((M, K, S) not in skc and skc["n"] + blocks > op_batch.SPLITK_COUNTERS or S * B * M > SKP_FLOATS):
                t, rpt, S = blocks, rpt, 1
            extra = {}
            if S > 1:
                if (M, K, S) not in skc:
                    skc[(M, K, S)] = skc["n"]
                    skc["n"] += blocks
                extra = dict(rows=ptr("skp"), resid_in=ptr("skc") + 4 * skc[(M, K, S)])
            add(name, "etx_tile_gemv_tc", gb("gemv_tc", t, W=Wp, x=ptr(x), out=ptr(out), M=M, K=K, rpt=rpt, tpe=S, nb=B, sx=K, sout=M, wts=bias, mode=mode, **extra), (t,), t)
            return
        t, rpt = m.gemv_tasks(M)
        add(name, "etx_tile_gemv_nb", gb("gemv_nb", t, W=Wp, x=ptr(x), out=ptr(out), M=M, K=K, rpt=rpt, tpe=1, nb=B, sx=K, sout=M, wts=bias, mode=mode), (t,), t)

    cols = argblock.pack_named(ent["cols"], (B, 1, 1), nb=B, slot_span=nblk * BS, zero=ptr("skc"))
    add("prologue", "vl_prologue_nb", cols, (B,), B)
    for L in range(d.L):
        Wl = lambda n, L=L: ptr(f"{L}.{n}")                                  # noqa: E731
        if L == 0:
            norm("norm1_0", None, 0, None, 0, "resid", None, "hn", Wl("ln1"))
        else:
            norm(f"norm1_{L}", "mc3", d.TOPK, "ti", d.TOPK * d.H, "resid2", "resid", "hn", Wl("ln1"))
        dense(f"qkv_{L}", Wl("wqkv"), "hn", "qkv", d.NQKV, d.H, bias=Wl("bqkv") if d.bias else 0)
        blobs = b""
        for b in range(B):
            blobs += argblock.pack_named(
                ent["attn_fused"], (ntask, 1, 1), qkv=ptr("qkv") + b * d.NQKV * 2, qw=Wl("qn") if d.qk_norm else 0, kw=Wl("kn") if d.qk_norm else 0,
                cos_sin=ptr("cos_sin"), kc=ptr("kc") + L * kv_layer_bytes, vc=ptr("vc") + L * kv_layer_bytes,
                block_tables=ptr("block_tables") + b * nblk * 4, seq_lens=ptr("seq_lens") + 4 * b, positions=ptr("positions") + 8 * b,
                slot_mapping=ptr("slot_mapping") + 8 * b, exp_sums=ptr("exp_sums") + b * d.NH * gparts * 4, max_logits=ptr("max_logits") + b * d.NH * gparts * 4,
                tmp_out=ptr("tmp_out") + b * d.NH * gparts * op_attn.GQ_PARTIAL_FLOATS * 4, out=ptr("attn_out") + b * d.NH * d.HD * 2,
                counters=ptr("attn_counters") + 4 * (L * B + b) * d.NH, scale=scale, eps=d.eps, NH=d.NH, NKV=d.NKV, HD=d.HD, BS=BS, X=X,
                max_parts=gparts, gq=gq, part_len=op_attn.tagged_part_len(L, whole))
        add(f"attn_{L}", "etx_tile_attn_fused", blobs, (ntask, B), ntask * B, two_d=True, stride=op_attn.F_ARG_BYTES)
        dense(f"o_proj_{L}", Wl("wo"), "attn_out", "o", d.H, d.NH * d.HD)
        norm(f"norm2_{L}", "o", 1, None, d.H, "resid", "resid2", "o_norm", Wl("ln2"))
        dense(f"router_{L}", Wl("wr"), "o_norm", "rlog", d.E, d.H)
        rmode = (1 if d.norm_topk else 0) | op_gemv.MODE_BF16_WTS
        if engine == "tc":
            # one routing task per column; the expert grids have one task per worker, which takes an equal share of the
            # active experts' tiles and derives the token lists from the routing ids itself
            add(f"route_{L}", "etx_tile_route", argblock.pack_named(ent["route"], (B, 1, 1), logits=ptr("rlog"), wts=ptr("tw"), ids=ptr("ti"), ecount=0, elist=0,
                                                                    active=0, E=d.E, K=d.TOPK, mode=rmode, nb=B, cap=B), (B,), B)
            add(f"moe_up_{L}", "etx_tile_moe_up_tc", gb("moe_up_tc", W, E=d.E, W=Wl("w13"), x=ptr("o_norm"), out=ptr("mc2"), estride=2 * d.MI * d.H, M=d.MI, K=d.H,
                                                        rpt=128, tpe=-(-d.MI // 128), ids=ptr("ti"), resid_out=ptr("active") + 4 * L, nb=B, R=d.TOPK, sx=d.H, eps=d.eps), (W,), W)
            add(f"moe_down_{L}", "etx_tile_moe_down_tc", gb("moe_down_tc", W, E=d.E, W=Wl("w2"), x=ptr("mc2"), out=ptr("mc3"), wts=ptr("tw"), estride=d.H * d.MI,
                                                            M=d.H, K=d.MI, rpt=256, tpe=-(-d.H // 256), ids=ptr("ti"), nb=B, R=d.TOPK, eps=d.eps), (W,), W)
            continue
        add(f"route_{L}", "etx_tile_route", argblock.pack_named(ent["route"], (1, 1, 1), logits=ptr("rlog"), wts=ptr("tw"), ids=ptr("ti"), ecount=ptr("ecount"),
                                                                elist=ptr("elist"), active=ptr("active") + 4 * L, E=d.E, K=d.TOPK, mode=rmode, nb=B, cap=B), (1,), 1)
        tpe = -(-d.MI // UP_ROWS)
        add(f"moe_up_{L}", "etx_tile_moe_up_g", gb("moe_up_g", d.E * tpe, E=d.E, W=Wl("w13"), x=ptr("o_norm"), out=ptr("mc2"), estride=2 * d.MI * d.H, M=d.MI, K=d.H,
                                                   rpt=UP_ROWS, tpe=tpe, rows=ptr("elist"), resid_in=ptr("ecount"), nb=B, R=d.TOPK, sx=d.H, eps=d.eps),
            (d.E * tpe,), d.E * tpe)
        tpe = -(-d.H // DOWN_ROWS)
        add(f"moe_down_{L}", "etx_tile_moe_down_g", gb("moe_down_g", d.E * tpe, E=d.E, W=Wl("w2"), x=ptr("mc2"), out=ptr("mc3"), wts=ptr("tw"), estride=d.H * d.MI,
                                                       M=d.H, K=d.MI, rpt=DOWN_ROWS, tpe=tpe, rows=ptr("elist"), resid_in=ptr("ecount"), nb=B, R=d.TOPK, eps=d.eps),
            (d.E * tpe,), d.E * tpe)
    norm("norm_f", "mc3", d.TOPK, "ti", d.TOPK * d.H, "resid2", "resid", "hn", ptr("final_norm"))
    dense("lm_head", ptr("embed") if d.tie else ptr("lm_head"), "hn", "logits", d.V, d.H)
    add("argmax", "vl_argmax_nb", cols, (B,), B)
    return g, pool, {"workers": W, "attn": (gq, plen, gparts), "attn_tasks": ntask, "attn_whole": whole, "engine": engine}


class BatchProgram:
    """B sequences decoded in lock step on one GPU: weights, per-sequence buffers and KV blocks, plan, session."""

    def __init__(self, dims: Q.Dims, weights: dict, batch: int, device: int = 0, maxlen: int = 1072, steps: int | None = None, machine="b200",
                 engine: str = "tc"):
        self.d, self.B, self.maxlen = dims, int(batch), maxlen
        self.dev = torch.device("cuda", device)
        self.machine = load_machine(machine) if isinstance(machine, str) else machine
        self.steps = steps or maxlen
        self.w = weights
        for k, shp in Q.weight_shapes(dims, maxlen).items():
            if k not in weights or tuple(weights[k].shape) != tuple(shp):
                raise ValueError(f"weight {k}: expected shape {shp}, got {tuple(weights[k].shape) if k in weights else None}")
        parts = -(-maxlen // op_attn.GQ_PART)
        self.buf = {n: torch.zeros(shape, dtype=_DT[dt], device=self.dev) for n, (shape, dt) in buffer_shapes(dims, self.B, maxlen, self.steps, parts).items()}
        nblk = self.buf["block_tables"].shape[1]
        self.buf["block_tables"].copy_(torch.arange(self.B * nblk, dtype=torch.int32).view(self.B, nblk))

        def ptr(name):
            t = self.buf.get(name)
            if t is None:
                t = self.w[name]
            return t.data_ptr()
        self.graph, self.pool, self.info = build_graph(dims, ptr, self.B, maxlen, self.machine, engine=engine)
        pool = self.pool.bytes()
        self.plan = compile_graph(self.graph, self.machine, {"POOL": len(pool)}, options=PassOptions())
        self.session = Session(self.plan, {}, pool, device)
        b = self.buf
        self.session.set_step(tok=0, pos=0, write_next=0, H=dims.H, V=dims.V, nrep=self.B, embed=self.w["embed"], resid=b["resid"],
                              positions=b["positions"], seq_lens=b["seq_lens"], slot_mapping=b["slot_mapping"], logits=b["logits"],
                              token_in=b["token_in"], token_out=b["token_out"], token_time=b["token_time"])

    def step(self, t: int, pos: int, write_next: bool, wait: bool = True):
        self.session.set_step(tok=t, pos=pos, write_next=int(write_next))
        if wait:
            self.session.run(120.0)
        else:
            self.session.launch()

    def generate(self, prompts, n_gen: int, sync_every: int = 32):
        """prompts: [B][P] token ids (one length).  Feeds them position by position, then n_gen greedy tokens per sequence
        (the next tokens never leave the device).  Returns [B][n_gen]."""
        prompts = np.asarray(prompts, np.int64)
        if prompts.shape[0] != self.B:
            raise ValueError(f"{prompts.shape[0]} prompts for a batch of {self.B}")
        P = prompts.shape[1]
        n = P + n_gen - 1
        if n + 2 > self.buf["token_in"].shape[0] or n > self.maxlen:
            raise ValueError("sequence longer than the session was sized for")
        tin = torch.zeros_like(self.buf["token_in"])
        tin[:P] = torch.from_numpy(prompts.T.copy()).to(torch.int32)
        self.buf["token_in"].copy_(tin)
        torch.cuda.synchronize(self.dev)
        for t in range(n):
            self.step(t, t, write_next=t + 1 >= P, wait=(t % sync_every == sync_every - 1) or t == n - 1)
        return self.buf["token_out"][P - 1:n].cpu().numpy().T

    def load_kv(self, layer: int, seq: int, K: np.ndarray, V: np.ndarray):
        """Pre-fill positions 0..ctx-1 of one layer of sequence `seq` from contiguous float32 (bf16-exact) [ctx][NKV][HD] arrays."""
        ctx, nkv, hd = K.shape
        nblk = self.buf["block_tables"].shape[1]
        kc, vc = self.buf["kc"][layer], self.buf["vc"][layer]
        Kt = torch.from_numpy(np.ascontiguousarray(K)).to(self.dev).to(torch.bfloat16)
        Vt = torch.from_numpy(np.ascontiguousarray(V)).to(self.dev).to(torch.bfloat16)
        pad = (-ctx) % BS
        if pad:
            Kt = torch.cat([Kt, torch.zeros(pad, nkv, hd, dtype=Kt.dtype, device=self.dev)])
            Vt = torch.cat([Vt, torch.zeros(pad, nkv, hd, dtype=Vt.dtype, device=self.dev)])
        nb = Kt.shape[0] // BS
        kc[seq * nblk:seq * nblk + nb] = Kt.view(nb, BS, nkv, hd // X, X).permute(0, 2, 3, 1, 4)
        vc[seq * nblk:seq * nblk + nb] = Vt.view(nb, BS, nkv, hd).permute(0, 2, 3, 1)

    def read(self, name: str) -> np.ndarray:
        t = self.buf[name]
        return (t.float() if t.dtype == torch.bfloat16 else t).cpu().numpy()

    def active_experts(self, reset: bool = True) -> np.ndarray:
        """Per layer: experts with at least one token, summed over the steps since the last reset (the routing tile counts
        them; divide by the number of steps for the average a byte ledger wants)."""
        out = self.read("active").copy()
        if reset:
            self.buf["active"].zero_()
            torch.cuda.synchronize(self.dev)
        return out

    def close(self):
        self.session.close()
