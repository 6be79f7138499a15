"""Declarations of the public planning surface (the role of etx/api/types.py:1-186): immutable, JSON-valued records
with a content identity.  No compiler, file or GPU dependency."""
from __future__ import annotations

import hashlib
import json
import math
from collections.abc import Iterator, Mapping
from dataclasses import dataclass, field

SCHEMA_VERSION = 1


_SCALARS = (str, bool, int)


def canonical(value, where: str = "configuration"):
    """`value` rebuilt from plain JSON types only (dict with string keys, list, str, bool, int, finite float, None);
    anything else is refused.  Exact types are required for the scalars: a subclass could carry state JSON would drop."""
    stack_free = value is None or type(value) in _SCALARS or (type(value) is float and math.isfinite(value))
    if stack_free:
        return value
    if isinstance(value, Mapping):
        out = {}
        for key, item in value.items():
            if type(key) is not str:
                raise ValueError(f"{where} keys must be strings")
            out[key] = canonical(item, where)
        return out
    if isinstance(value, (list, tuple)):
        return [canonical(item, where) for item in value]
    raise ValueError(f"{where} requires finite JSON values, got {type(value).__name__}")


def _dumps(value) -> str:
    """The canonical text of a JSON value: sorted keys, no blanks, no NaN -- equal values give equal text."""
    return json.dumps(value, sort_keys=True, separators=(",", ":"), allow_nan=False)


class Configuration(Mapping):
    """An immutable JSON value: stored as its canonical text, handed out as detached copies."""

    __slots__ = ("_text",)

    def __init__(self, values: Mapping):
        if not isinstance(values, Mapping):
            raise ValueError("configuration must be a mapping")
        self._text = _dumps(canonical(values))

    def to_dict(self) -> dict:
        return json.loads(self._text)

    def __getitem__(self, key):
        return self.to_dict()[key]

    def __iter__(self) -> Iterator:
        return iter(self.to_dict())

    def __len__(self) -> int:
        return len(self.to_dict())

    def __eq__(self, other):
        return isinstance(other, Configuration) and self._text == other._text

    def __hash__(self):
        return hash(self._text)


def _require_name(value, what: str = "name"):
    ok = type(value) is str and value != "" and value == value.strip()
    if not ok:
        raise ValueError(f"{what} must be a nonempty string without surrounding whitespace")


def _require_schema(value, what: str):
    if type(value) is not int or value != SCHEMA_VERSION:
        raise ValueError(f"unsupported {what} schema")


def _freeze(record, *names):
    """Replace the named fields of a frozen record by Configuration copies."""
    for n in names:
        object.__setattr__(record, n, Configuration(getattr(record, n)))


def _digest(d: dict) -> str:
    return hashlib.sha256(_dumps(d).encode()).hexdigest()


@dataclass(frozen=True)
class WorkloadSpec:
    name: str
    kind: str                      # "model" | "graph"
    config: Configuration
    schema_version: int = SCHEMA_VERSION

    KINDS = ("model", "graph", "imported", "native")

    def __post_init__(self):
        _require_name(self.name)
        _require_schema(self.schema_version, "workload")
        if self.kind not in self.KINDS:
            raise ValueError("unknown workload kind")
        _freeze(self, "config")

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
        _require_name(self.target)
        _freeze(self, "bindings", "runtime", "options")
        for value in self.bindings.values():
            if type(value) is not int or value < 0:
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
        _require_schema(self.schema_version, "plan")
        _freeze(self, "machine", "options", "report")
        decisions = tuple(self.decisions)
        if not all(type(x) is str for x in decisions):
            raise ValueError("decisions require strings")
        object.__setattr__(self, "decisions", decisions)

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
        _freeze(self, "metrics")
        object.__setattr__(self, "blocked", tuple(self.blocked))
