"""The N > 1 plumbing of the benchmark on CPU: two gloo ranks, each with its own observation, slowest rank reported."""
import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pi05_megakernel_b200 import dp as DP
from pi05_megakernel_b200 import fixture as FX


def _worker(rank: int, world: int, port: int, out) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    geo = FX.Geometry(prefix=8, layers=1, hidden=32, intermediate=64, q_heads=2, head_dim=16, horizon=4, action_dim=4)
    obs = FX.make_observation(geo, DP.observation_seed(7301, rank))
    fake_ms = [5.0 + rank, 6.0 - rank]                      # rank 1 is slower on the first, rank 0 on the second
    worst = DP.max_over_ranks(fake_ms)
    gathered = [None] * world
    dist.all_gather_object(gathered, float(obs["noise"].sum()))
    out.put((rank, worst, gathered))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_get_different_observations_and_the_slowest_time():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29000 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, worst, gathered in results:
        assert worst == [6.0, 6.0]
        assert gathered[0] != gathered[1]                    # no shared observation: nothing to exchange
    assert DP.chunks_per_second(2, 6.0) == 2 * 1e3 / 6.0
    assert DP.max_over_ranks([1.0, 2.0]) == [1.0, 2.0]       # no process group: identity
    assert DP.observation_seed(7301, 3, 2) == 7301 + 3000 + 2
