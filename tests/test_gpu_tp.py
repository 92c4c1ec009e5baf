"""Tensor parallel on GPUs: one observation shared by several engines, one per GPU.

* ``test_peer_that_never_arrives_is_reported`` needs one GPU: an engine created as rank 0 of 2 whose "peer" is a
  buffer nobody writes.  Its pushes land in that buffer, its own arrival counters never move, the bounded wait inside
  the first exchange runs out after ~20 ms and the engine reports it; the GPU is never stalled or faulted.
* ``test_two_ranks_match_the_oracle`` needs two GPUs (skipped otherwise): two child processes, one engine each, the
  export blobs exchanged over gloo, plain peer stores between the GPUs (no NCCL, no multicast).  Both ranks must
  produce actions inside the oracle's band (reference fixture.py:105-120: error to the FP32 result <= 2x the BF16
  eager path's own error + 0.003) and agree with each other (they add the partial sums in the same order).
"""
import os

import pytest
import torch
import torch.multiprocessing as mp

from oracle import pi05_oracle as O
from pi05_megakernel_b200 import _lib
from pi05_megakernel_b200 import fixture as FX

pytestmark = pytest.mark.gpu


def test_peer_that_never_arrives_is_reported():
    from pi05_megakernel_b200.arm import Pi05Arm
    geo = FX.Geometry(prefix=128)
    dev = {k: v.cuda() for k, v in FX.make_inputs(geo, FX.SEEDS[0], "cpu").items()}
    arm = Pi05Arm(geo, "b200-s1-l2", "cuda", tp=(0, 2))
    assert (arm.config["tp_rank"], arm.config["tp_size"]) == (0, 2)
    arm.bind(dev)
    with pytest.raises(_lib.EngineError) as info:
        arm.launch()                                    # no peer attached yet
    assert info.value.code == _lib.ERR_NOT_BOUND
    nobody = torch.zeros(arm.ws.numel(), dtype=torch.uint8, device="cuda")
    _lib.check(arm.lib, arm.handle, arm.lib.pi05_tp_attach_pointer(arm.handle, 1, nobody.data_ptr()))
    assert arm.lib.pi05_tp_attach_pointer(arm.handle, 0, nobody.data_ptr()) == _lib.ERR_ARGUMENT    # itself
    arm.debug(-1, 40_000_000, -1)                       # every device-side wait gives up after ~20 ms
    arm.launch()
    with pytest.raises(_lib.EngineError) as info:
        arm.status()
    assert info.value.code == _lib.ERR_DEVICE_TIMEOUT
    assert bool(torch.isnan(arm.outputs()["actions"]).all())
    assert int(nobody.view(torch.int32).ne(0).sum()) > 0             # the pushes went where the peer's buffers would be
    arm.close()
    # the GPU is fine: a one-GPU engine runs right after
    one = Pi05Arm(geo, "b200-s1-l2", "cuda")
    one.bind(dev)
    one.launch()
    one.status()
    assert bool(torch.isfinite(one.outputs()["actions"]).all())
    one.close()


def _rank(rank: int, world: int, port: int, variant: str, out) -> None:
    import torch.distributed as dist
    from pi05_megakernel_b200.arm import Pi05Arm
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    geo = FX.Geometry(prefix=128)
    cpu = FX.make_inputs(geo, FX.SEEDS[1], "cpu", "scatter")        # every rank binds the same observation
    arm = Pi05Arm(geo, variant, f"cuda:{rank}", tp=(rank, world))
    arm.bind({k: v.cuda(rank) for k, v in cpu.items()})
    arm.tp_attach_all()
    results = []
    for _ in range(2):                                              # twice: the arrival counters carry on
        dist.barrier()
        arm.launch()
        arm.status()
        results.append(arm.outputs()["actions"].cpu())
    out.put((rank, results, arm.config))
    dist.barrier()
    arm.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("variant", ["b200-s2-l3", "b200"])
def test_two_ranks_match_the_oracle(variant):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 33000 + os.getpid() % 2000
    procs = [ctx.Process(target=_rank, args=(r, 2, port, variant, out)) for r in range(2)]
    for p in procs:
        p.start()
    got = dict()
    for _ in procs:
        rank, results, config = out.get(timeout=600)
        got[rank] = results
        assert config["tp_size"] == 2 and config["units"]["gate_up"] == 32
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    geo, ogeo = FX.Geometry(prefix=128), O.Geo(prefix=128)
    cpu = FX.make_inputs(geo, FX.SEEDS[1], "cpu", "scatter")
    steps, layers = (2, 3) if variant != "b200" else (None, None)
    want, exact = O.chunk(cpu, ogeo, False, steps, layers), O.chunk(cpu, ogeo, True, steps, layers)
    for launch in range(2):
        # the ranks add the partial sums of every exchange in rank order; what differs between them is only the order
        # in which their own split-K atomics landed, and those sums are the same numbers on both
        assert float((got[0][launch] - got[1][launch]).abs().max()) <= 2 * (O.ATOL + O.RTOL * float(want.abs().max()))
        for rank in range(2):
            d = O.band(want, got[rank][launch], exact)
            assert d["pass"], (rank, launch, d)
