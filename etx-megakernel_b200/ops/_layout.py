"""Shared helper: the imports.json-style entry of a built-in tile (what the reference's `import_entries()` return,
etx/ops/gemv.py:107-116), so argblock.pack and the operator table treat built-in tiles like any other export."""
from __future__ import annotations


def entry(export: str, form: str, params, arg_bytes: int, grid_off: int, threads: int, spec: str) -> dict:
    ps = [{"ty": ty, "name": f"%{n}", "field": name, "size": size, "align": min(size, 8), "offset": off}
          for n, (name, ty, off, size) in enumerate(params)]
    return {"dsl": form, "export": f"etx_tile_{export}", "kernel": export, "block": [threads, 1, 1], "threads": threads, "slots": 1,
            "slot_threads": threads, "params": ps, "grid_offset": grid_off, "arg_bytes": arg_bytes, "lds_bytes_per_slot": 0,
            "lds_bytes": 0, "barriers": 0, "slot_barrier": False, "spec": spec}
