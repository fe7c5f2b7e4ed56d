"""The N > 1 path on CPU: two gloo ranks agree on the job's time (the slowest rank's) and split the slots."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from qwenny_b200 import replicas


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ms = replicas.slowest_ms(5.0 + 2.0 * rank)
    dist.barrier()
    q.put((rank, ms, list(replicas.rank_slots(5, rank, world))))
    dist.destroy_process_group()


def test_two_ranks_take_the_slowest_time():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    ps = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    got = sorted(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [g[1] for g in got] == [7.0, 7.0]
    assert got[0][2] == [0, 1, 2] and got[1][2] == [3, 4]
    assert replicas.job_throughput(5, 7.0, 2) == 2 * 5 / 7.0 * 1e3


def test_single_rank():
    assert replicas.slowest_ms(3.5) == 3.5
    assert list(replicas.rank_slots(3, 0, 1)) == [0, 1, 2]
