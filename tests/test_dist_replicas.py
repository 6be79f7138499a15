"""The N > 1 path of the bench on CPU: two gloo ranks agree on the slowest step time and on the aggregate metric."""
import os

import pytest

torch = pytest.importorskip("torch")
import torch.distributed as dist  # noqa: E402
import torch.multiprocessing as mp  # noqa: E402

import etx_megakernel_b200  # noqa: E402,F401
from etx_megakernel_b200.runtime import dist as D  # noqa: E402


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    r, w, lr = D.rank_env(os.environ)
    dist.init_process_group("gloo", rank=r, world_size=w)
    mine = [4.0 + rank, 5.0 - rank]                       # rank 1 is slower on the first timing, rank 0 on the second
    got = D.slowest(mine, dist)
    dist.barrier()
    q.put((rank, got, D.replica_metric(got[0], w)))
    dist.destroy_process_group()


def test_two_ranks_take_the_slowest_time_and_aggregate_tokens():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29611, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    for rank, got, metric in out:
        assert got == [5.0, 5.0]                           # max over ranks, identical on every rank
        assert metric == {"ms_per_token": 2.5, "tokens_per_s": 400.0}


def test_single_process_is_a_no_op():
    assert D.rank_env({}) == (0, 1, 0)
    assert D.slowest([1.5, 2.5]) == [1.5, 2.5]
    assert D.replica_metric(4.0, 1) == {"ms_per_token": 4.0, "tokens_per_s": 250.0}
