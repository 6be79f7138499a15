"""Graph builder types of the program surface: tensors, event tensors, tile handles, task grids.

Field names, defaults and the builder methods follow the reference (etx/ir/types.py:15-207) so that a graph-building
module written for it constructs the same objects here; what the B200 backend does not use (scopes per XCD, coherence
modes of tiles, per-XCD domain maps) is kept as data and ignored by the plan.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import IntEnum

from .dims import Dim, free_symbols
from .edgemap import EdgeMap


class Scope(IntEnum):
    WORKGROUP = 0
    CLUSTER = 1
    DOMAIN = 2
    DEVICE = 3
    SYSTEM = 4


class InitKind(IntEnum):
    STATIC = 0
    PER_STEP = 1
    RUNTIME = 2


@dataclass
class Tensor:
    name: str
    shape: tuple
    dtype: str = "bf16"
    role: str = "activation"        # activation | weight | runtime | scratch
    bytes_per_elem: int = 2

    def nbytes(self, bindings) -> int:
        from .dims import eval_shape
        n = self.bytes_per_elem
        for d in eval_shape(self.shape, bindings):
            n *= d
        return n


@dataclass
class ETensor:
    name: str
    shape: tuple
    wait_count: Dim | str = 1
    init_kind: InitKind = InitKind.STATIC
    runtime_init_by: str | None = None
    runtime_count: str | None = None
    scope: Scope | None = None
    domain_id: int | None = None
    memory: str | None = None
    epoch: bool = False

    @property
    def is_runtime_count(self) -> bool:
        return self.wait_count == "runtime" or self.init_kind == InitKind.RUNTIME


@dataclass
class Resource:
    threads: int = 256
    lds_bytes: int = 0
    vgpr: int = 128
    agpr: int = 0
    tensor_core: bool = False
    prefetch_bytes: int = 0


@dataclass
class TileBody:
    kind: str                       # hip_link | cuda_link | triton | builtin
    symbol: str
    source: str | None = None
    prefetch: str | None = None
    pre_wait: str | None = None
    touch: str | None = None
    coherence: str = "imported"
    arg_bytes: int = 0
    coherence_caps: tuple = ()
    stream_after: str | None = None    # B200 backend: what the tile's WEIGHT ADDRESSES depend on -- "" nothing (static weights:
                                       # the producer warp streams them ahead of the task's events), an event name (a
                                       # single-counter event, e.g. the router's for expert weights), None = the task's in-events
    exchange: bool = False             # B200 backend, sharded model: a row-parallel grid whose partial rows and arrivals also go
                                       # to the other ranks (see runtime.Session.set_exchange)


@dataclass
class TaskGrid:
    name: str
    grid: tuple
    body: TileBody
    resource: Resource = field(default_factory=Resource)
    args: list = field(default_factory=list)
    reads: list = field(default_factory=list)
    writes: list = field(default_factory=list)
    in_edges: dict = field(default_factory=dict)
    out_edges: dict = field(default_factory=dict)
    pure: bool = False
    out_to_in: str | None = None
    weight_args: list = field(default_factory=list)
    domain_map: str | None = None
    worker_map: str | None = None
    bytes_per_tile: Dim = 0
    duration_us: float = 1.0
    duration_cv: float = 0.0
    device: int = 0
    consts: tuple = ()
    prologue: list = field(default_factory=list)

    def __post_init__(self):
        if len(self.consts) > 4 or not all(isinstance(c, int) and not isinstance(c, bool) for c in self.consts):
            raise ValueError(f"{self.name}: consts must be at most 4 ints, got {self.consts!r}")
        both = sorted(set(self.reads) & set(self.writes))
        if self.pure and both:
            raise ValueError(f"{self.name}: pure=True but writes {both} it also reads (in-place tiles are not idempotent)")

    @property
    def has_runtime_edges(self) -> bool:
        return any(m.is_runtime for m in (*self.in_edges.values(), *self.out_edges.values()))


@dataclass
class Graph:
    name: str
    tensors: dict = field(default_factory=dict)
    events: dict = field(default_factory=dict)
    grids: list = field(default_factory=list)          # program order == topological order
    symbols: list = field(default_factory=list)
    codegen: dict = field(default_factory=dict)

    def _note(self, dims) -> None:
        for d in dims:
            for s in sorted(free_symbols(d)):
                if s not in self.symbols:
                    self.symbols.append(s)

    def tensor(self, name: str, shape, **kw) -> Tensor:
        t = Tensor(name, tuple(shape), **kw)
        self.tensors[name] = t
        self._note(shape)
        return t

    def etensor(self, name: str, shape, wait_count: Dim | str = 1, **kw) -> ETensor:
        e = ETensor(name, tuple(shape), wait_count, **kw)
        if wait_count == "runtime" or e.runtime_count is not None:
            e.init_kind, e.wait_count = InitKind.RUNTIME, "runtime"
        self.events[name] = e
        self._note(shape)
        if wait_count != "runtime":
            self._note((wait_count,))
        return e

    def call_device(self, name: str, grid, body: TileBody, *, in_edges=None, out_edges=None, **kw) -> TaskGrid:
        if any(g.name == name for g in self.grids):
            raise ValueError(f"duplicate task grid {name!r}")
        g = TaskGrid(name=name, grid=tuple(grid), body=body,
                     in_edges={k: EdgeMap.parse(v) for k, v in (in_edges or {}).items()},
                     out_edges={k: EdgeMap.parse(v) for k, v in (out_edges or {}).items()}, **kw)
        self.grids.append(g)
        self._note(grid)
        return g

    def grid(self, name: str) -> TaskGrid:
        for g in self.grids:
            if g.name == name:
                return g
        raise KeyError(name)

    def producers_of(self, event: str) -> list:
        return [g for g in self.grids if event in g.out_edges]

    def consumers_of(self, event: str) -> list:
        return [g for g in self.grids if event in g.in_edges]

    def readers_of(self, tensor: str) -> list:
        return [g for g in self.grids if tensor in g.reads or tensor in g.args]
