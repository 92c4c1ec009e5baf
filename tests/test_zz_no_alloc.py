"""The entry point that works out of the library's own fixed device array (pi05_chunk_static).

It exists for callers that cannot allocate device memory where they call the engine (a frozen or foreign
allocator, a plugin step inside another framework).  This test drives it through the C ABI only - no handle,
no workspace tensor - twice in a row on the same GPU, and checks each result against what the regular
handle-based entry points produce for the same inputs, and against the CPU oracle's band.  It is collected last
on purpose: a run that stops at the first failure has then already run every other test.  It does not depend on
state left by other tests, so it also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

from oracle import pi05_oracle as O
from pi05_megakernel_b200 import _lib
from pi05_megakernel_b200 import fixture as FX

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_regular_entry_twice():
    from pi05_megakernel_b200.arm import Pi05Arm
    geo, ogeo = FX.Geometry(prefix=128), O.Geo(prefix=128)
    cpu = FX.make_inputs(geo, FX.SEEDS[2], "cpu")
    dev = {k: v.cuda() for k, v in cpu.items()}
    want, exact = O.chunk(cpu, ogeo, False), O.chunk(cpu, ogeo, True)

    arm = Pi05Arm(geo, "b200", "cuda")          # the existing path: caller-allocated workspace
    arm.bind(dev)
    arm.launch()
    arm.status()
    regular = arm.outputs()["actions"].cpu()
    assert O.band(want, regular, exact)["pass"]
    arm.close()

    lib = _lib.load()
    ptrs = (ctypes.c_void_p * _lib.NUM_INPUTS)(*[dev[k].data_ptr() for k in FX.ORDER])
    actions = torch.empty(50, 32, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    # the same slack the band grants around the oracle: atol + rtol * max|value| (fixture tolerances 0.003 / 0.003),
    # doubled because both results carry their own split-K summation order
    slack = 2 * (O.ATOL + O.RTOL * float(regular.abs().max()))
    for call in range(2):
        actions.fill_(float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = lib.pi05_chunk_static(0, ptrs, geo.prefix, actions.data_ptr(), geo.steps, geo.layers, stream)
        assert rc == _lib.OK, lib.pi05_error_string(rc)
        torch.cuda.synchronize()
        if call == 1:
            # the defining property: nothing on this path takes device memory (the first call's set-up creates an event
            # and a stream, which may cost the driver a little; the second call must cost nothing at all)
            assert torch.cuda.mem_get_info()[0] == free_before
        got = actions.cpu()
        assert bool(torch.isfinite(got).all())
        assert float((got - regular).abs().max()) <= slack, call
        d = O.band(want, got, exact)
        assert d["pass"], (call, d)

    # sizes beyond the stated maximum are refused on the host, before anything is enqueued
    assert lib.pi05_chunk_static(0, ptrs, _lib.STATIC_MAX_PREFIX + 1, actions.data_ptr(), 10, 18, stream) \
        == _lib.ERR_UNSUPPORTED
    assert lib.pi05_chunk_static(0, ptrs, 0, actions.data_ptr(), 10, 18, stream) == _lib.ERR_ARGUMENT
    assert lib.pi05_chunk_static(0, None, 128, actions.data_ptr(), 10, 18, stream) == _lib.ERR_ARGUMENT


def test_static_scratch_entry_rebinds_behind_a_running_call():
    """Two calls back to back on a non-blocking stream with different output buffers and prefix lengths: the second one
    has to re-describe and clear the shared array, and must wait for the first one's kernel before it does.  Both
    results are checked against the handle-based entry points."""
    from pi05_megakernel_b200.arm import Pi05Arm
    lib = _lib.load()
    cases = []
    for prefix, seed in ((128, FX.SEEDS[0]), (192, FX.SEEDS[1])):
        geo = FX.Geometry(prefix=prefix)
        cpu = FX.make_inputs(geo, seed, "cpu", "pad")
        dev = {k: v.cuda() for k, v in cpu.items()}
        arm = Pi05Arm(geo, "b200-s2-l4", "cuda")
        arm.bind(dev)
        arm.launch()
        arm.status()
        cases.append((geo, dev, arm.outputs()["actions"].clone()))
        arm.close()
    side = torch.cuda.Stream()
    outs = [torch.full((50, 32), float("nan"), dtype=torch.float32, device="cuda") for _ in cases]
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        for (geo, dev, _), out in zip(cases, outs):
            ptrs = (ctypes.c_void_p * _lib.NUM_INPUTS)(*[dev[k].data_ptr() for k in FX.ORDER])
            rc = lib.pi05_chunk_static(0, ptrs, geo.prefix, out.data_ptr(), 2, 4, side.cuda_stream)
            assert rc == _lib.OK, lib.pi05_error_string(rc)
    side.synchronize()
    for (geo, dev, regular), out in zip(cases, outs):
        slack = 2 * (O.ATOL + O.RTOL * float(regular.abs().max()))
        assert bool(torch.isfinite(out).all())
        assert float((out - regular).abs().max()) <= slack, geo.prefix
