"""Tile handles (etx/frontends/tileop.py:14-33 of the reference).

`cuda_link(source, symbol)` is the working path here: `symbol` names one of the built-in sm_100a tiles of the
megakernel (passes/plan.py: TILE_SYMBOLS); `source` is informational.  `hip_link` accepts the reference's keyword set
so that graph modules written for it import unchanged; a hip_link handle whose symbol is one of the reference's tile
names (etx_tile_dsl_gemv, vl_prologue, ...) is mapped to the same built-in tile.
"""
from __future__ import annotations

from ..ir.types import TileBody


def hip_link(source, symbol, prefetch=None, pre_wait=None, touch=None, coherence="imported", arg_bytes=0, coherence_caps=()):
    return TileBody(kind="hip_link", symbol=symbol, source=source, prefetch=prefetch, pre_wait=pre_wait, touch=touch,
                    coherence=coherence, arg_bytes=arg_bytes, coherence_caps=tuple(coherence_caps))


def cuda_link(source, symbol, prefetch=None, stream_after=None, exchange=False):
    """`stream_after`: see TileBody.stream_after ("" = static weights, an event name, or None = the task's in-events);
    `exchange`: TileBody.exchange (a row-parallel grid of a sharded model)."""
    return TileBody(kind="cuda_link", symbol=symbol, source=source, prefetch=prefetch, stream_after=stream_after, exchange=bool(exchange))


def triton_fn(module, name):
    return TileBody(kind="triton", symbol=name, source=module)


def builtin(name):
    return TileBody(kind="builtin", symbol=f"etx_builtin_{name}", source=None)
