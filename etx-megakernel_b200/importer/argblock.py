"""Host-side argument blocks (etx/importer/argblock.py:16-29 of the reference): every parameter at its natural
alignment in declaration order, then u32 grid[3] and u32 nblocks at `grid_offset`.  `pack(info, values, grid)` returns
the bytes of one launch; values come in parameter order (ints, floats, device pointers as ints)."""
from __future__ import annotations

import struct

_FMT = {"i8": "b", "i16": "h", "i32": "i", "i64": "q", "float": "f", "double": "d", "half": "e"}


def pack(info: dict, values: list, grid: tuple) -> bytes:
    params = info["params"]
    if len(values) != len(params):
        raise ValueError(f"{info['export']}: {len(values)} values for {len(params)} parameters")
    from .spec import validate_values
    validate_values(info["export"], values, grid)
    buf = bytearray(info["arg_bytes"])
    for p, v in zip(params, values):
        ptr = p["ty"].startswith("ptr")
        if ptr and not isinstance(v, int):
            raise TypeError(f"{info['export']}: parameter {p['name']} is a pointer, got {type(v).__name__}")
        struct.pack_into("<" + ("Q" if ptr else _FMT[p["ty"]]), buf, p["offset"], v)
    gx, gy, gz = grid
    struct.pack_into("<IIII", buf, info["grid_offset"], gx, gy, gz, gx * gy * gz)
    return bytes(buf)


def pack_named(info: dict, grid: tuple, **fields) -> bytes:
    """pack() with values given by field name (unset parameters are zero / null)."""
    names = [p["field"] for p in info["params"]]
    unknown = set(fields) - set(names)
    if unknown:
        raise KeyError(f"{info['export']}: unknown parameters {sorted(unknown)}")
    return pack(info, [fields.get(n, 0.0 if p["ty"] == "float" else 0) for n, p in zip(names, info["params"])], grid)
