"""Split-K row sum: the smallest graph with a real event (etx/operators/splitk_sum.py:10-33 of the reference).

  partial_sum (n, chunks) --"ij->i"--> E(n, wait chunks) --"i->i"--> final_sum (n,)

partial_sum task (i, j) adds chunk j of row i of A into parts[i][j]; final_sum task i waits for the row's `chunks`
partials and adds them into out[i].  The reference's tiles receive the tensors A / B / C directly; the built-in sm_100a
tiles of this library take an argument block like every other built-in tile, so both grids name the argument pool and
share one 56-byte block {in, parts, out, rows, cols, chunks} (csrc/etxb_abi.h: etxb_splitk_args).
"""
from __future__ import annotations

import struct

from ..frontends import cuda_link
from ..ir import Graph, Resource

ARG_BYTES = 56


def pack_block(a_ptr: int, parts_ptr: int, out_ptr: int, rows: int, cols: int, chunks: int) -> bytes:
    if cols % chunks:
        raise ValueError(f"{cols} columns do not split into {chunks} equal chunks")
    return struct.pack("<QQQiiii4I", a_ptr, parts_ptr, out_ptr, rows, cols, chunks, 0, rows, chunks, 1, rows * chunks)


def build_program(n: int = 64, cols: int = 128, chunks: int = 4, a_ptr: int = 0, parts_ptr: int = 0, out_ptr: int = 0):
    """The graph and the bytes of its argument pool (one block) for an [n, cols] float32 input."""
    pool = pack_block(a_ptr, parts_ptr, out_ptr, n, cols, chunks)
    pool += b"\0" * (-len(pool) % 16)
    g = Graph("splitk_sum")
    g.tensor("impargs", (len(pool),), role="weight", bytes_per_elem=1)
    g.etensor("E", (n,), wait_count=chunks)
    g.call_device("partial_sum", (n, chunks), cuda_link("etx-megakernel_b200/csrc", "etx_tile_partial_sum"),
                  resource=Resource(threads=544, lds_bytes=0, vgpr=64), args=["impargs"], consts=(0,), out_edges={"E": "ij->i"}, duration_us=2.0)
    g.call_device("final_sum", (n,), cuda_link("etx-megakernel_b200/csrc", "etx_tile_final_sum"),
                  resource=Resource(threads=544, lds_bytes=0, vgpr=32), args=["impargs"], consts=(0,), in_edges={"E": "i->i"}, duration_us=0.8)
    return g, pool


def build() -> Graph:
    return build_program()[0]


def bindings(**overrides) -> dict:
    b = {"n": 64}
    b.update(overrides)
    return b


def runtime(bindings, rng=None):
    return {}
