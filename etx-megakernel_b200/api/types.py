"""Declarations of the public planning surface (the role of etx/api/types.py:1-186): immutable, JSON-valued records
with a content identity.  No compiler, file or GPU dependency."""
from __future__ import annotations

import hashlib
import json
import math
from collections.abc import Iterator, Mapping
from dataclasses import dataclass, field

SCHEMA_VERSION = 1


def _json_value(v):
    if v is None or type(v) in (str, bool, int):
        return v
    if type(v) is float and math.isfinite(v):
        return v
    if isinstance(v, Mapping):
        if any(type(k) is not str for k in v):
            raise ValueError("configuration keys must be strings")
        return {k: _json_value(x) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [_json_value(x) for x in v]
    raise ValueError(f"configuration requires finite JSON values, got {type(v).__name__}")


class Configuration(Mapping):
    """Immutable JSON value store; what it returns are detached copies."""

    def __init__(self, values: Mapping):
        if not isinstance(values, Mapping):
            raise ValueError("configuration must be a mapping")
        self._json = json.dumps(_json_value(values), sort_keys=True, separators=(",", ":"), allow_nan=False)

    def to_dict(self) -> dict:
        return json.loads(self._json)

    def __getitem__(self, key):
        return self.to_dict()[key]

    def __iter__(self) -> Iterator:
        return iter(self.to_dict())

    def __len__(self) -> int:
        return len(self.to_dict())

    def __eq__(self, other):
        return isinstance(other, Configuration) and other._json == self._json

    def __hash__(self):
        return hash(self._json)


def _name(v):
    if type(v) is not str or not v or v != v.strip():
        raise ValueError("name must be a nonempty string without surrounding whitespace")


def _digest(d: dict) -> str:
    return hashlib.sha256(json.dumps(d, sort_keys=True, separators=(",", ":"), allow_nan=False).encode()).hexdigest()


@dataclass(frozen=True)
class WorkloadSpec:
    name: str
    kind: str                      # "model" | "graph"
    config: Configuration
    schema_version: int = SCHEMA_VERSION

    def __post_init__(self):
        _name(self.name)
        if self.kind not in ("model", "graph", "imported", "native"):
            raise ValueError("unknown workload kind")
        if type(self.schema_version) is not int or self.schema_version != SCHEMA_VERSION:
            raise ValueError("unsupported workload schema")
        object.__setattr__(self, "config", Configuration(self.config))

    def to_dict(self) -> dict:
        return dict(schema_version=self.schema_version, name=self.name, kind=self.kind, config=self.config.to_dict())

    @classmethod
    def from_dict(cls, v: Mapping) -> "WorkloadSpec":
        if not isinstance(v, Mapping) or set(v) != {"schema_version", "name", "kind", "config"}:
            raise ValueError("workload record requires exactly schema_version/name/kind/config")
        return cls(**v)

    @property
    def identity(self) -> str:
        return _digest(self.to_dict())


@dataclass(frozen=True)
class PlanRequest:
    workload: WorkloadSpec
    target: str = "b200"
    bindings: Configuration = field(default_factory=lambda: Configuration({}))
    runtime: Configuration = field(default_factory=lambda: Configuration({}))
    options: Configuration = field(default_factory=lambda: Configuration({}))

    def __post_init__(self):
        if not isinstance(self.workload, WorkloadSpec):
            raise TypeError("plan request requires WorkloadSpec")
        _name(self.target)
        for n in ("bindings", "runtime", "options"):
            object.__setattr__(self, n, Configuration(getattr(self, n)))
        if any(type(x) is not int or x < 0 for x in self.bindings.values()):
            raise ValueError("bindings require nonnegative integers")

    def to_dict(self) -> dict:
        return dict(workload=self.workload.to_dict(), target=self.target, bindings=self.bindings.to_dict(),
                    runtime=self.runtime.to_dict(), options=self.options.to_dict())


@dataclass(frozen=True)
class PlannedWorkload:
    """Detached planner output: a report, not an executable and not a correctness certificate."""
    request: PlanRequest
    machine: Configuration
    options: Configuration
    report: Configuration
    decisions: tuple
    schema_version: int = SCHEMA_VERSION

    def __post_init__(self):
        if not isinstance(self.request, PlanRequest):
            raise TypeError("planned workload requires PlanRequest")
        if type(self.schema_version) is not int or self.schema_version != SCHEMA_VERSION:
            raise ValueError("unsupported plan schema")
        for n in ("machine", "options", "report"):
            object.__setattr__(self, n, Configuration(getattr(self, n)))
        if any(type(x) is not str for x in self.decisions):
            raise ValueError("decisions require strings")
        object.__setattr__(self, "decisions", tuple(self.decisions))

    def to_dict(self) -> dict:
        return dict(schema_version=self.schema_version, request=self.request.to_dict(), machine=self.machine.to_dict(),
                    options=self.options.to_dict(), report=self.report.to_dict(), decisions=list(self.decisions))

    @classmethod
    def from_dict(cls, v: Mapping) -> "PlannedWorkload":
        if not isinstance(v, Mapping) or set(v) != {"schema_version", "request", "machine", "options", "report", "decisions"}:
            raise ValueError("invalid planned workload record")
        req = dict(v["request"])
        req["workload"] = WorkloadSpec.from_dict(req["workload"])
        return cls(**{**v, "request": PlanRequest(**req)})

    @property
    def identity(self) -> str:
        return _digest(self.to_dict())


@dataclass(frozen=True)
class SimulationResult:
    plan_identity: str
    seed: int
    metrics: Configuration
    deadlock: bool
    blocked: tuple
    backend: str = "simulation"

    def __post_init__(self):
        if self.backend != "simulation":
            raise ValueError("simulation results cannot claim a device backend")
        if type(self.seed) is not int or type(self.deadlock) is not bool:
            raise ValueError("invalid simulation result")
        object.__setattr__(self, "metrics", Configuration(self.metrics))
        object.__setattr__(self, "blocked", tuple(self.blocked))
