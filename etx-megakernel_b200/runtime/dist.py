"""Multi-GPU plumbing of the decode bench: one process per GPU, each rank a full replica of the session (the reference
has no multi-device decode path: its only cross-device program is the two-GPU GEMM + reduce-scatter demo,
etx/operators/gemm_rs.py).  No data-path collective: ranks only agree on the slowest step time."""
from __future__ import annotations


def rank_env(environ) -> tuple[int, int, int]:
    """(rank, world size, local rank) as torchrun exports them; (0, 1, 0) for a plain launch."""
    return int(environ.get("RANK", 0)), int(environ.get("WORLD_SIZE", 1)), int(environ.get("LOCAL_RANK", 0))


def slowest(values, dist=None, device=None):
    """Element-wise maximum over the ranks of a list of per-rank timings (a no-op without a process group)."""
    import torch
    t = torch.tensor([float(v) for v in values], dtype=torch.float64, device=device)
    if dist is not None and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.cpu()]


def replica_metric(step_ms: float, world: int) -> dict:
    """Whole-job figures of `world` replicas that each decode one sequence: every step yields `world` tokens."""
    return {"ms_per_token": step_ms / world, "tokens_per_s": 1000.0 * world / step_ms}


def gather_handles(handle: bytes, dist) -> list:
    """Every rank's exchange-region handle, in rank order (the handles are plain bytes: any transport will do; this one
    is the process group the ranks already share)."""
    out = [None] * dist.get_world_size()
    dist.all_gather_object(out, bytes(handle))
    return out


def connect_ranks(program, dist):
    """Sharded DecodeProgram: exchange the region handles, map the peers, and hold every rank until all are connected
    (no rank may step before its peers' counters are in place)."""
    program.connect(gather_handles(program.region.handle, dist))
    dist.barrier()


def close_ranks(program, dist):
    """Close a sharded program: wait for this rank's last kernel, then for every rank's, and only then unmap and free
    (a peer that is still running stores into this rank's region)."""
    import torch
    torch.cuda.synchronize(program.dev)
    dist.barrier()
    program.close()
    dist.barrier()
