"""Session host: plan -> device session -> steps.  The Python face of the C ABI, shaped after the reference's
etx_host lifecycle (etx/runtime/include/etx/host.h:518-531: setup once, then run = reset + launch + wait per step;
here a step is launch + wait, nothing is reset).

Buffers are torch tensors owned by the caller; only raw device pointers cross the boundary.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import lib as L


class Session:
    def __init__(self, plan, tensors: dict, pool: bytes, device: int = 0, pool_name: str = "impargs"):
        """plan: passes.Plan.  tensors: name -> torch tensor (device memory) for every tensor the graph's grids name in
        args=[...] except the argument pool, whose bytes are `pool` (uploaded by the library)."""
        self.plan, self.device = plan, device
        self.lib = L.load()
        named = [(pool_name, len(pool))] + [(n, t.numel() * t.element_size()) for n, t in tensors.items()]
        blob = plan.to_blob(named, pool)
        self._h = C.c_void_p()
        L.check(self.lib.etxb_create(blob, len(blob), device, C.byref(self._h)))
        self._keep = dict(tensors)
        for n, t in tensors.items():
            L.check(self.lib.etxb_bind(self._h, n.encode(), C.c_void_p(t.data_ptr()), t.numel() * t.element_size()))
        self.step_params = L.StepParams()

    # -- lifecycle
    def close(self):
        if getattr(self, "_h", None):
            self.lib.etxb_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_option(self, key: str, value: int):
        L.check(self.lib.etxb_set_option(self._h, key.encode(), int(value)))

    def set_step(self, **fields):
        for k, v in fields.items():
            if hasattr(v, "data_ptr"):
                v = v.data_ptr()
            setattr(self.step_params, k, v)
        L.check(self.lib.etxb_set_step(self._h, C.byref(self.step_params)))

    def set_exchange(self, rank: int, n_ranks: int, region: "ExchangeRegion"):
        """Make this session rank `rank` of a model sharded over `n_ranks` processes: the grids the graph marks
        `exchange=True` publish the rows they write, as flagged words, into `region` and into every peer's region
        (region.connect first); the norm folds that follow poll them there.  n_ranks = 1: the same hand-off on one GPU."""
        bases = (C.c_void_p * max(n_ranks, 1))(*[region.peers.get(r, 0) or None for r in range(n_ranks)])
        L.check(self.lib.etxb_set_exchange(self._h, rank, n_ranks, C.c_void_p(region.ptr), region.nbytes, bases))
        self._keep["__exchange__"] = region

    def launch(self, stream: int | None = None):
        L.check(self.lib.etxb_launch(self._h, C.c_void_p(stream or 0)))

    def launch_unfused(self, stream: int | None = None):
        """The same step as one launch per grid (the unfused baseline); wait() as after launch()."""
        L.check(self.lib.etxb_launch_unfused(self._h, C.c_void_p(stream or 0)))

    def wait(self, timeout_s: float = 60.0):
        L.check(self.lib.etxb_wait(self._h, float(timeout_s)))

    def run(self, timeout_s: float = 60.0, stream: int | None = None) -> bool:
        """One step: launch + bounded wait.  Raises EtxbError on a failed step (the reference returns False and prints)."""
        L.check(self.lib.etxb_step(self._h, C.c_void_p(stream or 0), float(timeout_s)))
        return True

    def status(self) -> L.Status:
        st = L.Status()
        L.check(self.lib.etxb_status(self._h, C.byref(st)))
        return st

    def trace(self) -> np.ndarray:
        """[n_tasks][8] uint64: taken, deps ready, body done (globaltimer ns), worker, then four in-body marks (0 when a
        tile did not set one); rows in program order."""
        out = np.zeros((len(self.plan.tasks), 8), np.uint64)
        L.check(self.lib.etxb_trace(self._h, out.ctypes.data_as(C.c_void_p), out.nbytes))
        return out

    def exec_counts(self) -> np.ndarray:
        out = np.zeros(len(self.plan.tasks), np.int32)
        L.check(self.lib.etxb_exec_counts(self._h, out.ctypes.data_as(C.c_void_p), out.size))
        return out

    def decode_host(self, tokens_in, n_total: int, start_pos: int = 0):
        """Greedy decode through host buffers (tokens in and out of host memory every step).  Returns (tokens, ms per step)."""
        tin = np.ascontiguousarray(tokens_in, np.int32)
        out = np.zeros(n_total, np.int32)
        ms = np.zeros(n_total, np.float32)
        L.check(self.lib.etxb_decode_host(self._h, tin.ctypes.data_as(C.c_void_p), len(tin), n_total, start_pos,
                                          out.ctypes.data_as(C.c_void_p), ms.ctypes.data_as(C.c_void_p)))
        return out, ms


def op_launch(body: str | int, argblock: bytes, ntasks: int, device: int = 0, step: L.StepParams | None = None, stream: int | None = None):
    """Run `ntasks` tasks of one built-in tile on the persistent grid (asynchronous on `stream`)."""
    b = L.BODY[body] if isinstance(body, str) else int(body)
    L.check(L.load().etxb_op_launch(device, b, argblock, len(argblock), ntasks, C.byref(step) if step is not None else None,
                                    C.c_void_p(stream or 0)))


def attn_fused_static(argblock: bytes, device: int = 0, stream: int | None = None):
    """The fused attention phase through the entry point that allocates nothing (scratch in a static device array of the
    library: NH <= 64, max_parts <= 64, HD <= 128).  `argblock`: an attn_fused block; its scratch pointers are ignored."""
    L.check(L.load().etxb_attn_fused_static(device, argblock, len(argblock), C.c_void_p(stream or 0)))


class ExchangeRegion:
    """One rank's exchange region of a sharded model: a device allocation of the library's ([event counters][rows]) with
    its 64-byte inter-process handle, and the mappings of the peers' regions once `connect` opened their handles."""

    def __init__(self, nbytes: int, device: int = 0):
        self.device, self.nbytes = device, int(nbytes)
        p, h = C.c_void_p(), (C.c_ubyte * L.IPC_HANDLE_BYTES)()
        L.check(L.load().etxb_exchange_alloc(device, self.nbytes, C.byref(p), C.cast(h, C.c_void_p)))
        self.ptr, self.handle = int(p.value), bytes(h)
        self.peers = {}

    def connect(self, rank: int, handles: list):
        """handles[r]: rank r's handle (entry `rank` is this region's own and is not opened)."""
        for r, h in enumerate(handles):
            if r == rank or r in self.peers:
                continue
            if len(h) != L.IPC_HANDLE_BYTES:
                raise ValueError(f"rank {r}: a handle is {L.IPC_HANDLE_BYTES} bytes")
            p = C.c_void_p()
            L.check(L.load().etxb_exchange_open(self.device, h, C.byref(p)))
            self.peers[r] = int(p.value)

    def close(self):
        lib = L.load()
        for p in self.peers.values():
            lib.etxb_exchange_close(self.device, C.c_void_p(p))
        self.peers = {}
        if self.ptr:
            lib.etxb_exchange_free(self.device, C.c_void_p(self.ptr))
            self.ptr = 0
