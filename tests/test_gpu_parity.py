"""Parity of the CUDA engine with the oracle, through the arm / C ABI.  Every test needs a B200.

Tolerances: the engine's result must sit inside the reference harness's band (fixture.py:105-120): error
against the FP32 oracle <= 2x the BF16 reference's own error + rtol 0.003 (relative L2), and max-abs <=
2x reference max-abs + atol 0.003 + 0.003 * max|exact|.  Stage checks compare single stages computed from
the engine's own inputs to that stage, where only summation order differs: BF16 buffers within 1e-3 relative L2
(a BF16 ulp is 2^-8 relative), FP32 accumulators within 1e-4 relative L2.  Split-K partial sums meet in FP32
atomics, so two launches may differ in the last bit of an accumulator; values derived from an accumulator of an
earlier launch are therefore compared to one BF16 ulp, not bit for bit.
"""
import ctypes
import json
import os

import pytest
import torch
import torch.nn.functional as F

from oracle import pi05_oracle as O
from pi05_megakernel_b200 import _lib
from pi05_megakernel_b200 import fixture as FX
from tests.helpers import fingerprints_match, load_full

pytestmark = pytest.mark.gpu

WAIT_DEFAULT = 4_000_000_000


def _arm(geo, variant="b200"):
    from pi05_megakernel_b200.arm import Pi05Arm
    return Pi05Arm(geo, variant, "cuda")


@pytest.fixture(scope="module")
def case128():
    geo = FX.Geometry(prefix=128)
    cpu = FX.make_inputs(geo, FX.SEEDS[0], "cpu", "full")
    dev = {k: v.cuda() for k, v in cpu.items()}
    return geo, O.Geo(prefix=128), cpu, dev


def _run(arm):
    arm.launch()
    arm.status()
    return arm.outputs()["actions"].cpu()


def _rel(got, want):
    got, want = got.float(), want.float()
    return float((got - want).norm() / want.norm().clamp_min(1e-30))


def _rope_tables(arm):
    """cos / sin [50, 128] BF16 from the engine's table (one 32-bit word per entry: cos | sin << 16)."""
    raw = arm.region("rope", torch.bfloat16, (50, 128, 2)).clone()
    return raw[:, :, 0], raw[:, :, 1]


def _assert_one_ulp(got, want):
    """BF16 values that may differ by one unit in the last place of the largest operand (the sum h + delta can
    cancel, so the unit is taken from the tensor's scale) and differ in at most 1 % of the places."""
    diff = (got - want).abs()
    assert float(diff.max()) <= 2 ** -7 * float(want.abs().max())
    assert float((diff > 0).float().mean()) < 0.01


def test_prologue_tables(case128):
    """Time embedding, time MLP, all 370 modulation vectors, RoPE table, first action_in and norm."""
    geo, ogeo, cpu, dev = case128
    arm = _arm(geo)
    arm.bind(dev)
    arm.debug(0, 0, -1)
    _run(arm)
    dt = -1.0 / 10
    times = [torch.full((1,), 1.0 + s * dt, dtype=torch.float32) for s in range(10)]
    temb = torch.stack([O.time_embedding(t, 1024)[0] for t in times])
    cond = torch.stack([O.time_condition(cpu, t, 1024)[0] for t in times])
    assert torch.equal(arm.region("temb", torch.float32, (10, 1024)).cpu(), temb)
    assert _rel(arm.region("cond", torch.float32, (10, 1024)).cpu(), cond) < 2e-6
    nw = torch.cat([torch.stack([dev["attn_norm_weight"], dev["ffn_norm_weight"]], 1).reshape(36, 3072, 1024),
                    dev["final_norm_weight"][None]])
    nb = torch.cat([torch.stack([dev["attn_norm_bias"], dev["ffn_norm_bias"]], 1).reshape(36, 3072),
                    dev["final_norm_bias"][None]])
    torch.backends.cuda.matmul.allow_tf32 = False
    mod_want = torch.einsum("sk,njk->snj", cond.cuda(), nw) + nb[None]
    mod = arm.region("mod", torch.float32, (10, 37, 3072))
    assert _rel(mod, mod_want) < 5e-6
    pos, _ = O.suffix_layout(cpu["prefix_mask"], 50)
    inv = 1.0 / (O.ROPE_THETA ** (torch.arange(0, 256, 2, dtype=torch.int64).float() / 256))
    ph = pos.float()[:, None] * inv[None]
    rcos, rsin = _rope_tables(arm)
    rcos, rsin = rcos.cpu(), rsin.cpu()
    # cos/sin of phases up to ~180 rad: allow a last-bit difference of the FP32 phase on a few entries
    assert float((rcos.float() - ph.cos().to(torch.bfloat16).float()).abs().max()) <= 2 ** -7
    assert float((rsin.float() - ph.sin().to(torch.bfloat16).float()).abs().max()) <= 2 ** -7
    h0 = F.linear(cpu["noise"], cpu["action_in_weight"], cpu["action_in_bias"]).to(torch.bfloat16)
    got_h0 = arm.region("h", torch.bfloat16, (50, 1024)).cpu()
    assert float((got_h0.float() - h0.float()).abs().max()) <= 2 ** -8 * float(h0.abs().max())
    an, _ = O.ada_rms(got_h0, mod[0, 0].cpu(), O._cast(False))
    assert _rel(arm.region("an_attn", torch.bfloat16, (50, 1024)).cpu(), an) < 1e-3
    arm.close()


def test_one_layer_stage_by_stage(case128):
    """Each of the seven stages of layer 0, checked from the engine's own inputs to that stage."""
    geo, ogeo, cpu, dev = case128
    arm = _arm(geo)
    arm.bind(dev)
    f = lambda x: x.float()
    _, allowed = O.suffix_layout(cpu["prefix_mask"], 50)
    keep = {}
    for stage in range(1, 8):
        arm.debug(stage, 0, -1)
        _run(arm)
        reg = lambda n, d, s: arm.region(n, d, s).clone()
        if stage == 1:
            # QKV GEMM: q as FP32 split-K sums (rounded and rotated later, by attention); k (with RoPE) and v as BF16
            an = f(reg("an_attn", torch.bfloat16, (50, 1024)))
            keep["q_acc"] = reg("qkv_acc", torch.float32, (50, 2560))[:, :2048].clone()
            assert _rel(keep["q_acc"], an @ f(dev["wq"][0]).T) < 1e-4
            cos, sin = _rope_tables(arm)
            cos, sin = torch.cat((cos, cos), -1)[:, None].float(), torch.cat((sin, sin), -1)[:, None].float()
            keep["rot"] = lambda x: O.rb(O.rb(x * cos) + O.rb(torch.cat((-x[..., 128:], x[..., :128]), -1) * sin))
            k = keep["rot"](O.rb(an @ f(dev["wk"][0]).T).view(50, 1, 256)).reshape(50, 256)
            assert _rel(reg("k", torch.bfloat16, (50, 256)), k) < 1e-3
            assert _rel(reg("v", torch.bfloat16, (50, 256)), O.rb(an @ f(dev["wv"][0]).T)) < 1e-3
        elif stage == 2:
            # attention from the engine's own q sums (round, RoPE with BF16 products and sum) and its k / v
            q = keep["rot"](O.rb(keep["q_acc"]).view(50, 8, 256))
            keys = torch.cat((f(dev["prefix_k"][0][:, 0]), f(reg("k", torch.bfloat16, (50, 256)))))
            vals = torch.cat((f(dev["prefix_v"][0][:, 0]), f(reg("v", torch.bfloat16, (50, 256)))))
            s = O.rb(O.rb(torch.einsum("thd,kd->thk", q, keys)) * (1 / 16))
            s = torch.where(allowed.cuda()[:, None, :], s, torch.full_like(s, float("-inf")))
            e = torch.exp(s - s.max(-1, keepdim=True).values)
            o = torch.einsum("thk,kd->thd", O.rb(e), vals) / e.sum(-1, keepdim=True)
            assert _rel(reg("attn", torch.bfloat16, (50, 2048)), O.rb(o).reshape(50, 2048)) < 4e-3
        elif stage == 3:
            keep["o_acc"] = reg("o_acc", torch.float32, (50, 1024))
            want = f(reg("attn", torch.bfloat16, (50, 2048))) @ f(dev["wo"][0]).T
            assert _rel(keep["o_acc"], want) < 1e-4
            keep["h"] = f(reg("h", torch.bfloat16, (50, 1024)))
        elif stage == 4:
            mod = reg("mod", torch.float32, (10, 37, 3072))
            hn = O.rb(keep["h"] + O.rb(O.rb(keep["o_acc"]) * O.rb(mod[0, 0, 2048:])))
            got_h = reg("h", torch.bfloat16, (50, 1024))
            _assert_one_ulp(f(got_h), hn)
            an, _ = O.ada_rms(got_h.cpu(), mod[0, 1].cpu(), O._cast(False))
            assert _rel(reg("an_ffn", torch.bfloat16, (50, 1024)).cpu(), an) < 1e-3
            assert float(reg("o_acc", torch.float32, (50, 1024)).abs().max()) == 0.0
            assert float(reg("qkv_acc", torch.float32, (50, 2560)).abs().max()) == 0.0   # cleared for the next layer
        elif stage == 5:
            an = f(reg("an_ffn", torch.bfloat16, (50, 1024)))
            g, u = O.rb(an @ f(dev["wg"][0]).T), O.rb(an @ f(dev["wu"][0]).T)
            want = O.rb(O.rb(F.gelu(g, approximate="tanh")) * u)
            assert _rel(reg("act", torch.bfloat16, (50, 4096)), want) < 1e-3
        elif stage == 6:
            keep["d_acc"] = reg("d_acc", torch.float32, (50, 1024))
            want = f(reg("act", torch.bfloat16, (50, 4096))) @ f(dev["wd"][0]).T
            assert _rel(keep["d_acc"], want) < 1e-4
            keep["h"] = f(reg("h", torch.bfloat16, (50, 1024)))
        elif stage == 7:
            mod = reg("mod", torch.float32, (10, 37, 3072))
            hn = O.rb(keep["h"] + O.rb(O.rb(keep["d_acc"]) * O.rb(mod[0, 1, 2048:])))
            got_h = reg("h", torch.bfloat16, (50, 1024))
            _assert_one_ulp(f(got_h), hn)
            an, _ = O.ada_rms(got_h.cpu(), mod[0, 2].cpu(), O._cast(False))
            assert _rel(reg("an_attn", torch.bfloat16, (50, 1024)).cpu(), an) < 1e-3
    arm.close()


@pytest.mark.parametrize("steps,layers", [(1, 1), (2, 2), (1, 18), (3, 5)])
def test_truncated_chunks(case128, steps, layers):
    geo, ogeo, cpu, dev = case128
    arm = _arm(geo, f"b200-s{steps}-l{layers}")
    arm.bind(dev)
    got = _run(arm)
    want, exact = O.chunk(cpu, ogeo, False, steps, layers), O.chunk(cpu, ogeo, True, steps, layers)
    assert O.band(want, got, exact)["pass"]
    arm.close()


def test_band_three_seeds_in_place_refresh_mutation_idempotence():
    """The reference harness's correctness protocol (bench.py:220-256): three seeds, inputs overwritten in
    place between seeds, refresh_weights(), band against the FP32 oracle, a second launch, and the
    (sum, abs-sum) fingerprints of every input unchanged."""
    geo, ogeo = FX.Geometry(prefix=128), O.Geo(prefix=128)
    cpu = FX.make_inputs(geo, FX.SEEDS[0], "cpu")
    dev = {k: v.cuda() for k, v in cpu.items()}
    arm = _arm(geo)
    arm.bind(dev)
    for n, seed in enumerate(FX.SEEDS):
        if n:
            cpu = FX.make_inputs(geo, seed, "cpu")
            for k, v in cpu.items():
                dev[k].copy_(v)
            arm.refresh_weights()
            torch.cuda.synchronize()
        want, exact = O.chunk(cpu, ogeo, False), O.chunk(cpu, ogeo, True)
        snap = O.snapshot(dev)
        got = _run(arm)
        d = O.band(want, got, exact)
        assert d["pass"], (seed, d)
        again = _run(arm)
        # split-K partial sums meet in FP32 atomics, so a repeat may differ in the last bits of each layer;
        # it has to stay inside the same band
        assert O.band(want, again, exact)["pass"]
        assert O.snapshot(dev) == snap
    arm.close()


@pytest.mark.parametrize("name", ["full_p128_s7301", "full_p128_s8917", "full_p128_s42811", "full_p256_pad"])
def test_against_stored_reference_outputs(name):
    """Band against actions the unmodified reference and its FP32 oracle produced (tests/golden)."""
    geo, ogeo, seed, mask, fps, want, exact = load_full(name)
    cpu = FX.make_inputs(geo, seed, "cpu", "pad" if "pad" in name else "full")
    if not fingerprints_match(cpu, fps):
        # on a GPU box a silent skip would hollow the pin against the stored reference outputs: fail instead
        pytest.fail("this torch build draws different random inputs than the one that made the golden vectors; "
                    "regenerate them with tests/golden/make_golden.py")
    assert torch.equal(cpu["prefix_mask"], mask)
    arm = _arm(geo)
    arm.bind({k: v.cuda() for k, v in cpu.items()})
    got = _run(arm)
    d = O.band(want, got, exact)
    assert d["pass"], d
    arm.close()


@pytest.mark.parametrize("prefix,mask", [(1, "full"), (40, "scatter"), (64, "pad"), (65, "full"),
                                         (512, "scatter"), (968, "pad")])
def test_prefix_sweep_with_masks(prefix, mask):
    """Runtime prefix length and general validity masks: one chunk-loop iteration, a ragged last chunk,
    scattered and right-padded masks, the longest prefix.  Weights are shared with prefix 128 (same seed)."""
    geo, ogeo = FX.Geometry(prefix=prefix), O.Geo(prefix=prefix)
    cpu = FX.make_inputs(geo, FX.SEEDS[1], "cpu", mask)
    arm = _arm(geo, "b200-s2-l3" if prefix not in (512, 968) else "b200")
    arm.bind({k: v.cuda() for k, v in cpu.items()})
    got = _run(arm)
    want = O.chunk(cpu, ogeo, False, arm.steps, arm.layers)
    exact = O.chunk(cpu, ogeo, True, arm.steps, arm.layers)
    d = O.band(want, got, exact)
    assert d["pass"], d
    # masked-out keys must not matter
    poisoned = dict(cpu)
    k = cpu["prefix_k"].clone()
    k[:, ~cpu["prefix_mask"]] = 50.0
    poisoned["prefix_k"] = k
    if not bool(cpu["prefix_mask"].all()):
        arm2 = _arm(geo, arm.variant)
        arm2.bind({k_: v.cuda() for k_, v in poisoned.items()})
        d2 = O.band(want, _run(arm2), exact)
        assert d2["pass"], d2
        arm2.close()
    arm.close()


def test_wait_that_runs_out_reports_and_engine_recovers(case128):
    """Failure detection without faulting the GPU: a stage-completion signal is withheld on purpose, the
    bounded waits on it give up after ~20 ms, the kernel drains and exits, pi05_status reports which wait
    and where, and the next launch on the same handle is correct again."""
    geo, ogeo, cpu, dev = case128
    arm = _arm(geo, "b200-s1-l2")
    arm.bind(dev)
    good = _run(arm)
    arm.debug(-1, 40_000_000, _lib.EVENT_ATTENTION_DONE)
    arm.launch()
    with pytest.raises(_lib.EngineError) as info:
        arm.status()
    assert info.value.code == _lib.ERR_DEVICE_TIMEOUT
    # a chunk that gave up must not leave an earlier chunk's actions behind
    assert bool(torch.isnan(arm.outputs()["actions"]).all())
    arm.debug(-1, WAIT_DEFAULT, -1)
    again = _run(arm)
    want, exact = O.chunk(cpu, ogeo, False, 1, 2), O.chunk(cpu, ogeo, True, 1, 2)
    assert O.band(want, again, exact)["pass"]
    assert float((again - good).abs().max()) < 1e-2
    arm.close()


def test_abi_state_errors(case128):
    geo, ogeo, cpu, dev = case128
    lib = _lib.load()
    h = ctypes.c_void_p()
    assert lib.pi05_create(0, 128, 1, 0, 1, ctypes.byref(h)) == _lib.OK
    assert lib.pi05_launch(h, 10, 18, None, None) == _lib.ERR_NOT_BOUND
    n = ctypes.c_size_t()
    assert lib.pi05_workspace_bytes(h, ctypes.byref(n)) == _lib.OK and n.value > 4_000_000
    ws = torch.empty(n.value, dtype=torch.uint8, device="cuda")
    actions = torch.empty(50, 32, device="cuda")
    ptrs = (ctypes.c_void_p * 25)(*[dev[k].data_ptr() for k in FX.ORDER])
    assert lib.pi05_bind(h, ptrs, 129, 1, actions.data_ptr(), ws.data_ptr(), n.value) == _lib.ERR_ARGUMENT
    assert lib.pi05_bind(h, ptrs, 128, 2, actions.data_ptr(), ws.data_ptr(), n.value) == _lib.ERR_UNSUPPORTED
    assert lib.pi05_bind(h, ptrs, 128, 1, actions.data_ptr(), ws.data_ptr(), n.value - 1) == _lib.ERR_ARGUMENT
    assert lib.pi05_bind(h, ptrs, 128, 1, actions.data_ptr(), ws.data_ptr() + 8, n.value) == _lib.ERR_ARGUMENT
    bad = (ctypes.c_void_p * 25)(*[dev[k].data_ptr() for k in FX.ORDER])
    bad[3] = None
    assert lib.pi05_bind(h, bad, 128, 1, actions.data_ptr(), ws.data_ptr(), n.value) == _lib.ERR_ARGUMENT
    assert lib.pi05_bind(h, ptrs, 128, 1, actions.data_ptr(), ws.data_ptr(), n.value) == _lib.OK
    assert lib.pi05_launch(h, 11, 18, None, None) == _lib.ERR_ARGUMENT
    assert lib.pi05_launch(h, 10, 18, None, None) == _lib.OK
    code, where = ctypes.c_int(), ctypes.c_int()
    assert lib.pi05_status(h, ctypes.byref(code), ctypes.byref(where)) == _lib.OK and code.value == 0
    cnt = ctypes.c_ulonglong()
    assert lib.pi05_launch_count(h, ctypes.byref(cnt)) == _lib.OK and cnt.value == 1
    assert lib.pi05_destroy(h) == _lib.OK


@pytest.mark.parametrize("batch,variant", [(2, "b200-s2-l3"), (4, "b200"), (16, "b200-s1-l2")])
def test_batched_observations(batch, variant):
    """Several independent observations in one launch (shared weights, own prefix cache / mask / noise each):
    every observation's result must sit in the band of its own oracle run, and must not depend on its
    neighbours (the first observation equals a batch-of-one run up to split-K summation order)."""
    geo, ogeo = FX.Geometry(prefix=128), O.Geo(prefix=128)
    masks = ["full", "pad", "scatter", "full"] * 4
    stacked, per = FX.make_batch(geo, FX.SEEDS[0], batch, "cpu", masks[:batch])
    arm = _arm(geo, variant)
    arm.close()
    from pi05_megakernel_b200.arm import Pi05Arm
    arm = Pi05Arm(geo, variant, "cuda", batch=batch)
    arm.bind({k: v.cuda() for k, v in stacked.items()})
    got = _run(arm)
    assert tuple(got.shape) == (batch, 50, 32)
    for b in range(batch):
        want = O.chunk(per[b], ogeo, False, arm.steps, arm.layers)
        exact = O.chunk(per[b], ogeo, True, arm.steps, arm.layers)
        d = O.band(want, got[b], exact)
        assert d["pass"], (b, d)
    one = Pi05Arm(geo, variant, "cuda", batch=1)
    one.bind({k: v.cuda() for k, v in per[0].items()})
    alone = _run(one)
    assert float((alone - got[0]).abs().max()) <= 2 * (O.ATOL + O.RTOL * float(alone.abs().max()))
    one.close()
    arm.close()


@pytest.mark.parametrize("per_mma,batch", [(1, 3), (1, 5), (1, 8), (2, 2), (2, 3), (2, 7)])
def test_observations_per_mma(per_mma, batch, monkeypatch):
    """The batched kernels put one or two observations side by side in every MMA of the GEMM CTAs (two only when the
    tuning variable asks for it), from three observations on the schedule names, entry by entry, the group of
    observations it serves, and from five on the groups form two streams half a layer pass apart.  Every combination
    must give every observation a result in the band of its own oracle run, also when the batch does not fill the last
    group (3 of 4, 7 of 8), when the two streams have different numbers of groups (5, 7), and with the spare
    accumulator columns holding whatever the ring held before."""
    from pi05_megakernel_b200.arm import Pi05Arm
    monkeypatch.setenv("PI05_OBS_PER_MMA", str(per_mma))
    geo, ogeo = FX.Geometry(prefix=128), O.Geo(prefix=128)
    masks = ["scatter", "full", "pad", "full"] * 2
    stacked, per = FX.make_batch(geo, FX.SEEDS[1], batch, "cpu", masks[:batch])
    arm = Pi05Arm(geo, "b200-s1-l2", "cuda", batch=batch)
    arm.bind({k: v.cuda() for k, v in stacked.items()})
    got = _run(arm)
    again = _run(arm)
    arm.close()
    for b in range(batch):
        want = O.chunk(per[b], ogeo, False, 1, 2)
        exact = O.chunk(per[b], ogeo, True, 1, 2)
        d = O.band(want, got[b], exact)
        assert d["pass"], (per_mma, b, d)
    assert float((again - got).abs().max()) <= 2 * (O.ATOL + O.RTOL * float(got.abs().max()))


def _pool_from_dense(dense, page_tokens, num_pages, order, token_pad, fill):
    """Scatter a dense cache [B][L][P][1][256] into a pool [pages][L][page_tokens][1][256 + token_pad] (the returned
    view drops the padding) whose unused pages, padding and rows behind the prefix hold `fill`."""
    B, L, P = dense.shape[0], dense.shape[1], dense.shape[2]
    per = (P + page_tokens - 1) // page_tokens
    pool = torch.full((num_pages, L, page_tokens, 1, 256 + token_pad), fill, dtype=torch.bfloat16)
    table = []
    for b in range(B):
        row = []
        for lp in range(per):
            phys = order[b * per + lp]
            n = min(page_tokens, P - lp * page_tokens)
            pool[phys, :, :n, :, :256] = dense[b, :, lp * page_tokens:lp * page_tokens + n]
            row.append(phys)
        table.append(row)
    return pool, table


@pytest.mark.parametrize("prefix,page_tokens,batch,variant", [(300, 1024, 1, "b200-s2-l3"), (512, 128, 2, "b200-s2-l2"),
                                                              (968, 64, 1, "b200-s1-l2")])
def test_prefix_cache_view(prefix, page_tokens, batch, variant):
    """The prefix cache read where a producer left it: pages in shuffled order inside a larger pool, padding between
    tokens, one over-long page per observation or many 64-token pages.  Unused pages, the padding and the rows
    behind the prefix hold NaN, so any read of them would poison the result; the result must match the dense bind."""
    from pi05_megakernel_b200.arm import PagedPrefix, Pi05Arm
    geo, ogeo = FX.Geometry(prefix=prefix), O.Geo(prefix=prefix)
    masks = ["scatter", "pad"][:batch]
    stacked, per = FX.make_batch(geo, FX.SEEDS[1], batch, "cpu", masks)
    dense_k = stacked["prefix_k"].reshape(batch, geo.layers, prefix, 1, 256)
    dense_v = stacked["prefix_v"].reshape(batch, geo.layers, prefix, 1, 256)
    pages_per = (prefix + page_tokens - 1) // page_tokens
    num_pages = batch * pages_per + 3
    order = torch.randperm(num_pages, generator=torch.Generator().manual_seed(5)).tolist()
    pool_k, table = _pool_from_dense(dense_k, page_tokens, num_pages, order, 64, float("nan"))
    pool_v, _ = _pool_from_dense(dense_v, page_tokens, num_pages, order, 64, float("nan"))
    dev = {k: v.cuda() for k, v in stacked.items()}
    if batch == 1:
        dev = {k: (v[0] if k in FX.OBSERVATION else v) for k, v in dev.items()}
    arm = Pi05Arm(geo, variant, "cuda", batch=batch)
    arm.bind(dev)
    dense = _run(arm).reshape(batch, 50, 32)
    gk, gv = pool_k.cuda(), pool_v.cuda()
    view = PagedPrefix(gk[..., :256], gv[..., :256], table)
    rest = {k: v for k, v in dev.items() if k not in ("prefix_k", "prefix_v")}
    arm.bind(rest, kv_pages=view)
    paged = _run(arm).reshape(batch, 50, 32)
    assert torch.isfinite(paged).all()
    assert float((paged - dense).abs().max()) <= 2 * (O.ATOL + O.RTOL * float(dense.abs().max()))
    for b in range(batch):
        want = O.chunk(per[b], ogeo, False, arm.steps, arm.layers)
        exact = O.chunk(per[b], ogeo, True, arm.steps, arm.layers)
        assert O.band(want, paged[b], exact)["pass"], b
    arm.close()


def test_prefix_cache_view_rejects_bad_views():
    from pi05_megakernel_b200 import _lib
    from pi05_megakernel_b200.arm import PagedPrefix, Pi05Arm
    geo = FX.Geometry(prefix=200)
    dev = {k: v.cuda() for k, v in FX.make_inputs(geo, FX.SEEDS[0], "cpu").items()}
    rest = {k: v for k, v in dev.items() if k not in ("prefix_k", "prefix_v")}
    arm = Pi05Arm(geo, "b200-s1-l1", "cuda")
    pool = torch.zeros((4, geo.layers, 100, 1, 256), dtype=torch.bfloat16, device="cuda")
    for table, why in (([[0, 1]], "page_tokens not a multiple of 64"), ([[0]], "pages do not cover the prefix"),
                       ([[0, 9]], "entry outside the pool")):
        with pytest.raises(_lib.EngineError) as err:
            arm.bind(rest, kv_pages=PagedPrefix(pool, pool, table))
        assert err.value.code == _lib.ERR_ARGUMENT, why
    odd = torch.zeros((1, geo.layers, 256, 1, 260), dtype=torch.bfloat16, device="cuda")[..., :256]
    with pytest.raises(_lib.EngineError):
        arm.bind(rest, kv_pages=PagedPrefix(odd, odd, [[0]]))      # token stride 260 is not a multiple of 8 elements
    with pytest.raises(_lib.EngineError):
        arm.launch()                                                # nothing is bound after a failed bind
    arm.close()


def test_plain_cooperative_launch_without_clusters():
    """The engine launches the grid as clusters of two CTAs when the device takes it that way; the plain cooperative
    launch (selected here through the tuning variable) must give a result in the band as well."""
    import subprocess
    import sys
    code = (
        "import json, torch\n"
        "from oracle import pi05_oracle as O\n"
        "from pi05_megakernel_b200 import fixture as FX\n"
        "from pi05_megakernel_b200.arm import Pi05Arm\n"
        "geo = FX.Geometry(prefix=128)\n"
        "cpu = FX.make_inputs(geo, FX.SEEDS[2], 'cpu')\n"
        "arm = Pi05Arm(geo, 'b200-s2-l3', 'cuda')\n"
        "arm.bind({k: v.cuda() for k, v in cpu.items()})\n"
        "arm.launch(); arm.status()\n"
        "got = arm.outputs()['actions'].cpu()\n"
        "g = O.Geo(prefix=128)\n"
        "d = O.band(O.chunk(cpu, g, False, arm.steps, arm.layers), got, O.chunk(cpu, g, True, arm.steps, arm.layers))\n"
        "print(json.dumps({'pass': bool(d['pass']), 'clusters': arm.config.get('clusters_of_2')}))\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PI05_NO_CLUSTER="1", PYTHONPATH=root)
    out = subprocess.run([sys.executable, "-c", code], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    result = json.loads(out.stdout.strip().splitlines()[-1])
    assert result == {"pass": True, "clusters": False}
