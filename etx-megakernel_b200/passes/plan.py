"""The Plan: everything decided before launch, as data.

Keeps the reference's Plan vocabulary (etx/passes/plan.py:18-193: PassOptions, TaskInst, EventPlan, Plan, verify_plan,
summary) for the subset the B200 backend needs: task enumeration in program order, one event counter per event
coordinate with its per-step arrival count, static per-worker queues.  XCD affinity, relay words, coherence modes and
dynamic / hybrid queues of the reference have no counterpart on a single coherent L2 and are not modelled.

`Plan.to_blob()` serialises the tables into the layout csrc/etxb_abi.h documents; the C library validates it again
(arrivals == declared counts, indices in range) before anything is uploaded.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field
from typing import Any

import numpy as np

from ..ir.instantiate import Instance
from ..ir.types import Graph, Scope
from ..machine.model import MachineModel

MAGIC = 0x3030324258544555
BLOB_VERSION = 1
EV_STRIDE = 32
MAX_ARGS = 4

# tile symbol -> ETXB_BODY_* (include/etxb200.h).  Both the reference's export names and short names are accepted.
TILE_SYMBOLS = {
    "etx_builtin_nop": 0, "nop": 0,
    "vl_prologue": 1, "vl_argmax": 2,
    "etx_tile_dsl_gemv": 3, "etx_tile_dsl_gemv_fold": 3,
    "etx_tile_dsl_moe_up": 4, "etx_tile_dsl_moe_up_fold": 4,
    "etx_tile_dsl_moe_down": 5, "etx_tile_dsl_moe_down_fold": 5,
    "etx_tile_dsl_topk": 6, "etx_tile_dsl_attnprep": 7,
    "etx_tile_attn_decode": 8, "etx_tile_attn_reduce": 9, "etx_tile_attn_fused": 12,
    "etx_tile_partial_sum": 10, "etx_tile_final_sum": 11,
    "etx_tile_norm_col": 13, "etx_tile_gemv_nb": 14, "etx_tile_route": 15, "etx_tile_moe_up_g": 16, "etx_tile_moe_down_g": 17,
    "vl_prologue_nb": 18, "vl_argmax_nb": 19, "etx_tile_gemv_tc": 20, "etx_tile_moe_up_tc": 21, "etx_tile_moe_down_tc": 22,
    "etx_tile_mla_attn": 23,
}


@dataclass
class PassOptions:
    workers: int | None = None             # persistent CTAs; default: one per SM of the machine model
    event_elimination: bool = True         # accepted for source compatibility; no recomputation pass here
    prefetch: bool = True
    force_mode: str | None = None          # only "static" exists
    coherence: str = "declared"
    relay: str = "off"


@dataclass
class TaskInst:
    id: int
    grid: str
    coord: tuple
    type_id: int
    device: int = 0
    domain: int = 0
    worker: int | None = None
    mode: str = "static"
    duration_us: float = 1.0


@dataclass
class EventPlan:
    name: str
    shape: tuple
    scope: Scope = Scope.DEVICE
    memory: str = "device"
    offset: int = 0
    numel: int = 0
    counts: list = field(default_factory=list)


@dataclass
class Plan:
    arch: str
    graph: Graph
    inst: Instance
    machine: MachineModel
    bindings: dict
    options: PassOptions
    runtime: Any = None
    tasks: list = field(default_factory=list)
    task_index: dict = field(default_factory=dict)
    type_ids: dict = field(default_factory=dict)
    events: dict = field(default_factory=dict)
    modes: dict = field(default_factory=dict)
    reasons: dict = field(default_factory=dict)
    n_devices: int = 1
    n_domains: int = 1
    workers_per_domain: int = 1
    wg_per_cu: int = 1
    static_queues: dict = field(default_factory=dict)      # (device, worker) -> task ids
    task_in_words: list = field(default_factory=list)      # per task id: event word indices waited on
    task_out_words: list = field(default_factory=list)
    event_words: int = 0
    log: list = field(default_factory=list)

    def say(self, msg: str) -> None:
        self.log.append(msg)

    def workers_per_device(self) -> int:
        return self.n_domains * self.workers_per_domain

    def task(self, tid) -> TaskInst:
        return self.tasks[self.task_index[tid]]

    def linear(self, event: str, coord) -> int:
        idx = 0
        for d, c in zip(self.events[event].shape, coord):
            idx = idx * d + c
        return idx

    def word(self, event: str, coord) -> int:
        return self.events[event].offset + self.linear(event, coord)

    def summary(self) -> str:
        out = [f"plan: graph={self.graph.name} arch={self.arch} bindings={self.bindings}",
               f"  devices={self.n_devices} workers={self.workers_per_domain} tasks={len(self.tasks)} events={len(self.events)} words={self.event_words}"]
        out += [f"  {g:24s} {m:8s} {self.reasons.get(g, '')}" for g, m in self.modes.items()]
        out += [f"  event {e.name:16s} scope={e.scope.name:7s} mem={e.memory:8s} numel={e.numel}" for e in self.events.values()]
        return "\n".join(out)

    # ---- plan.json (keys of the reference's emit_plan_json, etx/codegen/kernel.py:684-723)
    def to_json(self) -> dict:
        return {"graph": self.graph.name, "arch": self.arch, "bindings": self.bindings,
                "types": [{"id": i, "grid": g} for g, i in self.type_ids.items()],
                "events": {e.name: {"offset": e.offset, "shape": list(e.shape), "scope": e.scope.name, "counts": list(e.counts)}
                           for e in self.events.values()},
                "descs": [{"id": t.id, "type": t.type_id, "coord": list(t.coord), "device": t.device, "domain": t.domain,
                           "worker": t.worker, "mode": t.mode} for t in self.tasks],
                "static_queues": {f"{d}:{w}": q for (d, w), q in self.static_queues.items()},
                "task_in": {str(t.id): list(self.task_in_words[t.id]) for t in self.tasks}}

    # ---- binary plan for the C library
    def to_blob(self, tensors: list, pool: bytes, type_args: dict | None = None) -> bytes:
        """tensors: [(name, bytes)], tensors[0] must be the argument pool ("impargs"); pool: its contents.
        type_args: grid name -> list of tensor names (defaults to the grid's call_device args)."""
        names = [n for n, _ in tensors]
        if not names or len(pool) != tensors[0][1]:
            raise ValueError("tensor 0 must be the argument pool and match its declared size")
        grids = {g.name: g for g in self.graph.grids}
        types = bytearray()
        for gname, tid in sorted(self.type_ids.items(), key=lambda kv: kv[1]):
            g = grids[gname]
            if g.body.symbol not in TILE_SYMBOLS:
                raise ValueError(f"grid {gname!r}: no built-in tile for symbol {g.body.symbol!r} (known: {sorted(TILE_SYMBOLS)})")
            cst = list(g.consts) + [0] * (4 - len(g.consts))
            argn = list((type_args or {}).get(gname, g.args))[:MAX_ARGS]
            for a in argn:
                if a not in names:
                    raise ValueError(f"grid {gname!r} names tensor {a!r} which the session does not bind")
            idx = [names.index(a) for a in argn] + [-1] * (MAX_ARGS - len(argn))
            body = TILE_SYMBOLS[g.body.symbol]
            after = g.body.stream_after
            if after is None:
                sword = -2
            elif after == "":
                sword = -1
            else:
                if after not in self.events or self.events[after].numel != 1:
                    raise ValueError(f"grid {gname!r}: stream_after={after!r} must name an event with a single counter")
                if not any(after in self.graph.grid(p.grid).out_edges for p in self.tasks if p.id < self.task_index[(gname, self.inst.tasks[gname][0])]):
                    raise ValueError(f"grid {gname!r}: stream_after={after!r} is not produced before it")
                sword = self.events[after].offset
            types += struct.pack("<i4i4iiii", body, *cst, *idx, 1 if 3 <= body <= 5 else 0, sword, 1 if g.body.exchange else 0)
        W = self.workers_per_device()
        qbegin, rows, inw, outw = [0], [], [], []
        for w in range(W):
            for tid in self.static_queues.get((0, w), []):
                t = self.tasks[tid]
                c = list(t.coord)[:4] + [0] * (4 - min(4, len(t.coord)))
                i_w, o_w = self.task_in_words[tid], self.task_out_words[tid]
                rows.append((t.type_id, *c, len(inw), len(i_w), len(outw), len(o_w), tid))
                inw += i_w; outw += o_w
            qbegin.append(len(rows))
        counts = [0] * self.event_words
        for e in self.events.values():
            counts[e.offset:e.offset + e.numel] = e.counts

        def sect(b: bytes) -> bytes:
            return b + b"\0" * (-len(b) % 8)
        head = struct.pack("<Q10I4I", MAGIC, BLOB_VERSION, W, len(rows), len(self.type_ids), self.event_words, len(inw), len(outw),
                           len(tensors), len(pool), 0, 0, 0, 0, 0)
        tens = b"".join(struct.pack("<56sQ", n.encode()[:55], b) for n, b in tensors)
        body = [tens, bytes(types), np.asarray(qbegin, "<i4").tobytes(), np.asarray(rows, "<i4").reshape(-1, 10).tobytes() if rows else b"",
                np.asarray(counts, "<i4").tobytes(), np.asarray(inw, "<i4").tobytes(), np.asarray(outw, "<i4").tobytes(), bytes(pool)]
        return sect(head) + b"".join(sect(b) for b in body)


def verify_plan(plan: Plan) -> list:
    """Co-residency and static-queue order safety (checks 6 and the queue check of etx/passes/plan.py:155-193):
    a task must never sit behind one of its own producers on the same worker, or the worker deadlocks on itself."""
    errors = []
    cap = plan.machine.workers()
    if plan.workers_per_device() > cap:
        errors.append(f"{plan.workers_per_device()} workers exceed co-resident capacity {cap}")
    where = {tid: (key, i) for key, q in plan.static_queues.items() for i, tid in enumerate(q)}
    if sorted(where) != list(range(len(plan.tasks))):
        errors.append("static queues do not hold every task exactly once")
    for key, q in plan.static_queues.items():
        for i, tid in enumerate(q):
            t = plan.tasks[tid]
            for ev in plan.inst.task_in[(t.grid, t.coord)]:
                for p in plan.inst.producers[ev]:
                    pid = plan.task_index[p]
                    if pid in where and where[pid][0] == key and where[pid][1] > i:
                        errors.append(f"worker {key}: task {tid} ({t.grid}{list(t.coord)}) queued before its producer {pid} -> deadlock")
    for e in plan.events.values():
        if any(c < 0 for c in e.counts):
            errors.append(f"event {e.name}: negative count")
    return errors
