"""Machine model: the data passes and model builders read (never the arch name).

Same accessor surface as the reference's MachineModel (etx/machine/model.py:43-165: load_machine, effective_scope,
vis, total_cus, cost accessors); the B200 entry adds what sizes the decode tiles: persistent CTA shape, the GEMV task
split and the attention partition.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import yaml

from ..ir.types import Scope

ARCH_DIR = Path(__file__).parent / "arch"


@dataclass
class ExecDomain:
    name: str
    count: int
    cus: int
    l2_mb: float = 0.0


@dataclass
class Visibility:
    release: list
    acquire: list
    poll: str
    arrive: str
    memory: str = "any"
    acquire_relaxed: list | None = None


@dataclass
class MachineModel:
    name: str
    family: str
    vendor: str
    wave_size: int
    devices_per_package: int
    exec_domains: list
    shared_cache: dict
    resources: dict
    bandwidth: dict
    visibility: dict
    capabilities: dict
    costs: dict
    lowering: dict = field(default_factory=dict)
    primitives: dict = field(default_factory=dict)
    notes: list = field(default_factory=list)
    extra: dict = field(default_factory=dict)

    # ---- topology: the exec-domain tree is a list from the outermost level to the leaf that holds the compute units
    @property
    def leaf_domain(self) -> ExecDomain:
        return self.exec_domains[-1]

    @property
    def num_domains(self) -> int:
        return math.prod(level.count for level in self.exec_domains)

    @property
    def has_domain_level(self) -> bool:
        return self.num_domains > 1

    def cus_per_domain(self) -> int:
        return self.leaf_domain.cus

    def total_cus(self) -> int:
        return self.cus_per_domain() * self.num_domains

    # ---- scopes: an event's declared scope is lowered to the nearest level this machine really has.  A cluster scope
    # needs cluster launch; without it, and for anything narrower than a domain, the event lives at domain level --
    # or, on a machine that is a single domain (B200: one L2 serves every SM), at device level.
    def effective_scope(self, scope: Scope) -> Scope:
        if scope == Scope.CLUSTER and self.capabilities.get("cluster_launch", False):
            return scope
        if scope in (Scope.CLUSTER, Scope.DOMAIN, Scope.WORKGROUP):
            return Scope.DOMAIN if self.has_domain_level else Scope.DEVICE
        return scope

    def vis(self, scope: Scope) -> Visibility:
        lowered = self.effective_scope(scope)
        try:
            return self.visibility[lowered]
        except KeyError:
            raise KeyError(f"{self.name}: no visibility entry for scope {lowered.name}") from None

    def memory_for(self, scope: Scope) -> str:
        kind = self.vis(scope).memory
        return kind if kind != "any" else "device"

    # ---- costs (the arch file gives nanoseconds, callers get microseconds)
    SYNC_COST_KEY = {Scope.DOMAIN: "t_local_ns", Scope.DEVICE: "t_cross_ns", Scope.SYSTEM: "t_dev_ns"}
    SYNC_COST_GUESS_NS = {"t_local_ns": 200, "t_cross_ns": 800, "t_dev_ns": 10000}     # used (and noted) when the arch file has no figure

    def _cost_ns(self, key: str, guess: float) -> float:
        if self.costs.get(key) is None:
            self.costs[key] = guess
            self.notes.append(f"{self.name}: no calibrated {key}; assuming {guess} ns")
        return float(self.costs[key])

    def t_sync_us(self, scope: Scope) -> float:
        """One hand-off through an event of `scope`."""
        lowered = self.effective_scope(scope)
        key = self.SYNC_COST_KEY.get(lowered, "t_cross_ns")
        if lowered == Scope.DEVICE and not self.has_domain_level:
            key = "t_local_ns"                                             # a single-domain device pays no cross-domain hop
        return self._cost_ns(key, self.SYNC_COST_GUESS_NS[key]) / 1e3

    def t_pop_us(self) -> float:
        return float(self.costs.get("t_pop_ns", 300)) / 1e3

    def t_push_us(self, cross_domain: bool) -> float:
        push = float(self.costs.get("t_push_ns", 300)) / 1e3
        return push + self.t_sync_us(Scope.DEVICE) if cross_domain else push

    def cache_bw_bytes_per_us(self) -> float:
        return 1e6 * float(self.bandwidth.get("cache_bw_tbs", self.bandwidth["hbm_tbs"]))

    def hbm_bw_bytes_per_us(self) -> float:
        return 1e6 * float(self.bandwidth["hbm_tbs"])

    def supports(self, cap: str) -> Any:
        return self.capabilities.get(cap, False)

    # ---- tile sizing for the persistent decode kernel
    def workers(self) -> int:
        """Persistent CTAs: one per SM (the whole shared memory and register file of the SM belong to one CTA)."""
        return self.total_cus()

    def gemv_tasks(self, rows: int, waves: int = 1, min_rows: int = 1) -> tuple[int, int]:
        """(tasks, rows per task) of a row-split GEMV: `waves` tasks per worker, rows spread as evenly as the
        reference's blk * rpt mapping allows (etx/ops/gemv.py BODIES: r0 = blk * rpt)."""
        want = max(1, self.workers() * waves)
        rpt = max(min_rows, -(-rows // want))
        return -(-rows // rpt), rpt

    # measured on B200 (per-task device stamps of the decode kernel): what one persistent CTA streams and multiplies
    # per microsecond once its weights flow, and what a tile costs before / after that (event poll, activation
    # staging with or without the norm fold, routing, release)
    STREAM_BYTES_PER_US = 40e3
    TILE_OVERHEAD_US = {"qkv": 3.4, "o_proj": 1.6, "router": 4.6, "moe_up": 5.5, "moe_down": 6.5, "lm_head": 3.0, "gate_up": 3.4,
                        "down": 2.5, "attn_fused": 8.0, "prep": 3.0, "attn": 6.0, "reduce": 3.0, "topk": 3.0}

    def tile_duration_us(self, role: str, task_bytes: float) -> float:
        """Annotation for the schedule simulator: fixed cost of the tile kind + its weight bytes at the per-CTA stream rate."""
        return self.TILE_OVERHEAD_US.get(role, 2.0) + task_bytes / self.STREAM_BYTES_PER_US

    def attention_part(self) -> int:
        """KV positions per attention task.  32 positions x 4 kv heads fills the SMs at a 1K context and keeps one
        task's K and V (2 x 8 KB at head_dim 128) a single round trip."""
        return 32

    def attention_groups(self, NH: int, NKV: int, HD: int, BS: int, maxlen: int) -> tuple:
        """(q heads per task, positions per task, partitions) of the grouped attention tile, or (0, 0, 0) when the
        shape needs the general tile.  The fewest q heads per task that still gives every task its own SM: the merge
        a group's last task runs reads gq * partitions partial rows, and the groups of a kv head share its K / V in L2."""
        G = NH // NKV
        if HD != 128 or BS != 16 or G not in (1, 2, 4, 8):
            return (0, 0, 0)
        parts = -(-maxlen // 128)
        fits = [gq for gq in (1, 2, 4, 8) if G % gq == 0 and (NH // gq) * parts <= self.workers()]
        return (fits[0] if fits else G, 128, parts)


def _visibility(raw: dict) -> dict:
    return {Scope[k.upper()]: Visibility(release=list(v.get("release", [])), acquire=list(v.get("acquire", [])), poll=v["poll"],
                                         arrive=v["arrive"], memory=v.get("memory", "any"),
                                         acquire_relaxed=list(v["acquire_relaxed"]) if "acquire_relaxed" in v else None)
            for k, v in raw.items()}


def list_archs() -> list:
    return sorted(p.stem for p in ARCH_DIR.glob("*.yaml"))


def load_machine(name_or_path) -> MachineModel:
    p = Path(name_or_path)
    if not p.exists():
        p = ARCH_DIR / f"{name_or_path}.yaml"
    if not p.exists():
        raise FileNotFoundError(f"no machine model {name_or_path!r}; known: {list_archs()}")
    raw = yaml.safe_load(p.read_text(encoding="utf-8"))
    known = {"name", "family", "vendor", "wave_size", "devices_per_package", "exec_domains", "shared_cache", "resources",
             "bandwidth", "visibility", "capabilities", "costs", "lowering", "primitives", "notes"}
    return MachineModel(name=raw["name"], family=raw["family"], vendor=raw["vendor"], wave_size=int(raw["wave_size"]),
                        devices_per_package=int(raw.get("devices_per_package", 1)),
                        exec_domains=[ExecDomain(**d) for d in raw["exec_domains"]], shared_cache=raw.get("shared_cache", {}),
                        resources=raw["resources"], bandwidth=raw["bandwidth"], visibility=_visibility(raw["visibility"]),
                        capabilities=raw.get("capabilities", {}), costs=dict(raw.get("costs", {})), lowering=raw.get("lowering", {}),
                        primitives=dict(raw.get("primitives", {})), notes=list(raw.get("notes", [])),
                        extra={k: v for k, v in raw.items() if k not in known})
