"""Multi-replica bookkeeping on CPU: two gloo ranks, each pretending to be one GPU's replica.
Checks the request split, the max-over-ranks time and the aggregate throughput, and that a rank
that fails before the barrier is reported on the host instead of hanging the others."""
import os
import socket

import pytest

torch = pytest.importorskip("torch")
import torch.multiprocessing as mp  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q, fail_rank):
    import datetime

    import torch.distributed as dist
    from rvllm_b200 import replicas
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    try:
        if rank == fail_rank:
            raise RuntimeError("replica failed before the timed region")
        mine = replicas.split_requests(1024 + 3, world, rank)
        dist.barrier()
        seconds = 0.5 + 0.25 * rank          # rank 1 is the slow replica
        tokens = len(mine) * 8               # 8 steps each
        q.put((rank, list(mine)[:1] + list(mine)[-1:], len(mine), replicas.job_seconds(dist, seconds),
               replicas.job_throughput(dist, tokens, seconds)))
    except Exception as e:  # report on the host; never leave the peer waiting forever
        q.put((rank, "error", str(e)))
    finally:
        dist.destroy_process_group()


def _run(world, fail_rank=-1):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, fail_rank)) for r in range(world)]
    for p in procs:
        p.start()
    out = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    return sorted(out, key=lambda x: x[0])


def test_two_replicas_split_and_aggregate():
    a, b = _run(2)
    assert a[2] + b[2] == 1027 and a[1][0] == 0 and a[1][1] + 1 == b[1][0] and b[1][1] == 1026
    assert a[3] == b[3] == 0.75                       # slowest rank defines the job time
    assert abs(a[4] - 1027 * 8 / 0.75) < 1e-6 and a[4] == b[4]


def test_split_edge_cases():
    from rvllm_b200 import replicas
    assert [len(replicas.split_requests(5, 8, r)) for r in range(8)] == [1, 1, 1, 1, 1, 0, 0, 0]
    assert list(replicas.split_requests(0, 2, 1)) == []
    covered = [i for r in range(3) for i in replicas.split_requests(10, 3, r)]
    assert covered == list(range(10))
    with pytest.raises(ValueError):
        replicas.split_requests(4, 2, 2)
    assert replicas.job_throughput(None, 64, 2.0) == 32.0


def test_failed_replica_is_reported_not_hung():
    res = _run(2, fail_rank=1)
    kinds = {r[0]: r[1] for r in res}
    assert kinds[1] == "error"
    # rank 0 either finished nothing (barrier timed out -> error) or was told; it must have returned
    assert 0 in kinds
