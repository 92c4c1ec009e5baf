"""Host-side logic that needs no GPU: fixtures, variants, the C ABI's exports and argument checks."""
import ctypes
import os
import re

import pytest
import torch

from pi05_megakernel_b200 import _lib, build
from pi05_megakernel_b200 import fixture as FX
from pi05_megakernel_b200.arm import parse_variant

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    build.build()
    return _lib.load()


def test_header_and_library_agree(lib):
    """Every function include/pi05_b200.h declares is exported, and nothing else is bound."""
    text = open(os.path.join(ROOT, "include", "pi05_b200.h")).read()
    declared = set(re.findall(r"\b(pi05_[a-z_]+)\s*\(", text))
    assert declared == set(_lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib, name)


def test_error_strings(lib):
    assert lib.pi05_error_string(_lib.OK) == b"ok"
    for code in range(1, 7):
        assert lib.pi05_error_string(code) not in (b"ok", b"unknown error")
    assert lib.pi05_error_string(99) == b"unknown error"


def test_argument_errors_never_touch_a_gpu(lib):
    h = ctypes.c_void_p()
    assert lib.pi05_create(0, 128, 1, 0, 1, None) == _lib.ERR_ARGUMENT
    assert lib.pi05_create(-1, 128, 1, 0, 1, ctypes.byref(h)) == _lib.ERR_ARGUMENT
    assert lib.pi05_create(0, 0, 1, 0, 1, ctypes.byref(h)) == _lib.ERR_ARGUMENT
    assert lib.pi05_create(0, 128, 1, 2, 2, ctypes.byref(h)) == _lib.ERR_ARGUMENT
    assert lib.pi05_create(0, 128, 17, 0, 1, ctypes.byref(h)) == _lib.ERR_UNSUPPORTED
    assert lib.pi05_create(0, 128, 1, 0, 3, ctypes.byref(h)) == _lib.ERR_UNSUPPORTED     # 2, 4 or 8 ranks
    assert lib.pi05_create(0, 128, 2, 0, 2, ctypes.byref(h)) == _lib.ERR_UNSUPPORTED     # one observation per launch
    n = ctypes.c_size_t()
    assert lib.pi05_workspace_bytes(None, ctypes.byref(n)) == _lib.ERR_ARGUMENT
    assert lib.pi05_launch(None, 10, 18, None, None) == _lib.ERR_ARGUMENT
    assert lib.pi05_destroy(None) == _lib.ERR_ARGUMENT
    if not torch.cuda.is_available():
        assert lib.pi05_create(0, 128, 1, 0, 1, ctypes.byref(h)) == _lib.ERR_NO_DEVICE
        assert not h.value


def test_prefill_argument_errors_never_touch_a_gpu(lib):
    """The prefill entry points check their arguments before they look for a device, and the Python wrapper has no CPU path."""
    h = ctypes.c_void_p()
    assert lib.pi05_prefill_create(0, 968, None) == _lib.ERR_ARGUMENT
    assert lib.pi05_prefill_create(-1, 968, ctypes.byref(h)) == _lib.ERR_ARGUMENT
    assert lib.pi05_prefill_create(0, 0, ctypes.byref(h)) == _lib.ERR_ARGUMENT
    assert lib.pi05_prefill_create(0, 4097, ctypes.byref(h)) == _lib.ERR_ARGUMENT
    n = ctypes.c_size_t()
    assert lib.pi05_prefill_workspace_bytes(None, ctypes.byref(n)) == _lib.ERR_ARGUMENT
    assert lib.pi05_prefill_run(None, None, None, 1, None, None, 18, None) == _lib.ERR_ARGUMENT
    assert lib.pi05_prefill_destroy(None) == _lib.ERR_ARGUMENT
    if not torch.cuda.is_available():
        assert lib.pi05_prefill_create(0, 968, ctypes.byref(h)) == _lib.ERR_NO_DEVICE
        assert not h.value
        from pi05_megakernel_b200.prefill import Pi05Prefill
        with pytest.raises(RuntimeError):
            Pi05Prefill(FX.PrefillGeometry(tokens=64), "cuda")


@pytest.mark.parametrize("sms", [148, 132])
@pytest.mark.parametrize("tokens", [1, 64, 129, 200, 256, 300, 512, 513, 968, 4096])
def test_prefill_plan(lib, sms, tokens):
    """The launch decisions of the prefill, and for a stream-K down projection the partition of (tile, k block) units over
    the CTAs: every unit exactly once, contiguous ranges of equal size (+-1), and for every tile cut over several CTAs one
    owner (the CTA that has its k block 0) followed by contributors that are the next CTAs' FIRST segments - the order
    that lets an owner wait for CTAs of higher index only while contributors wait for nobody."""
    info, count = (ctypes.c_int * 6)(), ctypes.c_int()
    assert lib.pi05_prefill_plan(sms, tokens, 0, info, None, 0, ctypes.byref(count)) == _lib.OK
    m_tiles, pairs, sk, tiles, kblocks, ctas = list(info)
    assert m_tiles == (tokens + 127) // 128 and pairs == (m_tiles >= 2) and sk == (m_tiles * 16 * 2 <= sms)
    if not sk:
        assert (tiles, kblocks, ctas, count.value) == (0, 0, 0, 0)
        return
    assert (tiles, kblocks, ctas) == (m_tiles * 8, 256, min(sms, m_tiles * 8 * 256))
    assert lib.pi05_prefill_plan(sms, tokens, ctas, info, None, 0, ctypes.byref(count)) == _lib.ERR_ARGUMENT
    per_cta = []
    for cta in range(ctas):
        buf = (ctypes.c_int * (3 * 8))()
        assert lib.pi05_prefill_plan(sms, tokens, cta, info, buf, 8, ctypes.byref(count)) == _lib.OK
        assert 1 <= count.value <= 8
        per_cta.append([tuple(buf[3 * i: 3 * i + 3]) for i in range(count.value)])
    units = [(t, kb) for segs in per_cta for (t, a, b) in segs for kb in range(a, b)]
    assert units == [(t, kb) for t in range(tiles) for kb in range(kblocks)]          # every unit once, in order
    sizes = [sum(b - a for (_t, a, b) in segs) for segs in per_cta]
    assert max(sizes) - min(sizes) <= 1
    for cta, segs in enumerate(per_cta):
        for i, (t, a, b) in enumerate(segs):
            assert i == 0 or a == 0                      # only a CTA's first segment can start inside a tile
            if a == 0 and b < kblocks:                   # owner of a tile that goes on in the following CTAs
                assert i == len(segs) - 1
                end, peer = b, cta + 1
                while end < kblocks:
                    pt, pa, pb = per_cta[peer][0]
                    assert (pt, pa) == (t, end) and pa > 0
                    end, peer = pb, peer + 1


def test_prefill_fixture_is_deterministic():
    geo = FX.PrefillGeometry(tokens=96, layers=1)
    shapes = FX.prefill_shapes(geo)
    assert set(FX.PREFILL_WEIGHTS) <= set(shapes) and shapes["ld"][0] == (1, 2048, 16384)
    a, b = FX.make_prefill_inputs(geo, 5, "pad"), FX.make_prefill_inputs(geo, 5, "pad")
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert a["valid"].dtype == torch.bool and 48 <= int(a["valid"].sum()) <= 96
    assert bool(a["valid"][: int(a["valid"].sum())].all())          # right-padded: the valid tokens come first


def test_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    from pi05_megakernel_b200.arm import Pi05Arm
    with pytest.raises(RuntimeError):
        Pi05Arm(FX.Geometry(), "b200", "cuda")


def test_variants():
    assert parse_variant("b200") == {"steps": None, "layers": None}
    assert parse_variant("b200-s2-l3") == {"steps": 2, "layers": 3}
    for bad in ("k64", "b200-x", "b200-s2-s3", "b200-l"):
        with pytest.raises(ValueError):
            parse_variant(bad)


def test_fixture_shapes_and_determinism():
    geo = FX.Geometry(prefix=24, layers=2, hidden=64, intermediate=128, q_heads=2, head_dim=16)
    a, b = FX.make_inputs(geo, 5), FX.make_inputs(geo, 5)
    assert list(a) == list(FX.ORDER)
    for name, (shape, dtype) in FX.shapes(geo).items():
        assert tuple(a[name].shape) == tuple(shape) and a[name].dtype == dtype
        assert torch.equal(a[name], b[name])
    assert float(a["wq"].float().std()) == pytest.approx(0.02, rel=0.1)
    pad = FX.make_observation(geo, 5, "pad")["prefix_mask"]
    n = int(pad.sum())
    assert geo.prefix // 2 <= n <= geo.prefix and bool(pad[:n].all()) and not bool(pad[n:].any())
    sc = FX.make_observation(geo, 5, "scatter")["prefix_mask"]
    assert geo.prefix // 2 <= int(sc.sum()) <= geo.prefix


def test_bind_view_argument_errors(lib):
    view = _lib.KvView()
    ptrs = (ctypes.c_void_p * _lib.NUM_INPUTS)()
    assert lib.pi05_bind_view(None, ptrs, ctypes.byref(view), 128, 1, None, None, 0) == _lib.ERR_ARGUMENT
    assert lib.pi05_bind(None, ptrs, 128, 1, None, None, 0) == _lib.ERR_ARGUMENT


STAGES = {0: 8, 1: 16, 2: 8, 3: 32}          # 128-k stages of the full K of QKV, O, gate/up, down
TILES = {0: 20, 1: 8, 2: 64, 3: 8}           # 128-row weight tiles (QKV: 16 q + 2 k + 2 v)


@pytest.mark.parametrize("batch,prefix", [(1, 128), (1, 968), (2, 128), (3, 128), (4, 128), (5, 128), (7, 128),
                                          (8, 128), (12, 128), (16, 128)])
def test_schedule_plan_invariants(lib, batch, prefix, monkeypatch):
    """The work schedule of the GEMM CTAs on a 148-SM part, computed on the host.  Whatever the batch: every
    (GEMM, group of observations, tile) is covered over its whole K exactly once; the units per observation that
    the stage counters wait for are the same for every group; no row CTA appears; and with named groups every
    CTA's list follows one global order (cycle position, then group), which is what rules out circular waits."""
    for name in ("PI05_OBS_PER_MMA", "PI05_LATENCY_SCHEDULE", "PI05_ONE_STREAM", "PI05_ROW_GROUPS", "PI05_KEY_GROUPS"):
        monkeypatch.delenv(name, raising=False)
    entries, plan = _lib.schedule_plan(148, batch, prefix)
    ngroups = plan["groups"]
    assert ngroups == (batch + plan["obs_per_mma"] - 1) // plan["obs_per_mma"]
    assert plan["gemm_ctas"] == 148 - 25 * max(plan["row_groups"], plan["key_groups"])
    cover: dict = {}
    per_cta: dict = {}
    for cta, gemm, lag, group, tile, k0, nk in entries:
        assert 0 <= cta < plan["gemm_ctas"] and nk >= 1 and 0 <= tile < TILES[gemm]
        groups = range(ngroups) if group < 0 else [group]
        for g in groups:
            cover.setdefault((gemm, g, tile), []).append((k0, nk))
        per_cta.setdefault(cta, []).append((gemm, lag, group))
    for gemm in range(4):
        for g in range(ngroups):
            units = 0
            for tile in range(TILES[gemm]):
                runs = sorted(cover[(gemm, g, tile)])
                units += len(runs)
                pos = 0
                for k0, nk in runs:                       # contiguous, no overlap, whole K
                    assert k0 == pos
                    pos += nk
                assert pos == STAGES[gemm]
            assert units == list(plan["units"].values())[gemm]
    assert max(len(v) for v in per_cta.values()) <= 32
    if batch >= 5:
        assert plan["stream_split"] == (ngroups + 1) // 2
    named = [e for e in entries if e[3] >= 0]
    assert bool(named) == (batch >= 3)
    if named:
        split = plan["stream_split"]

        def position(gemm, lag, group):
            if not split:
                return (gemm, group)
            b = group >= split
            assert lag == (1 if b and gemm >= 2 else 0)
            # q(A) gate/up(B) O(A) down(B) gate/up(A) q(B) down(A) O(B)
            order = {(0, False): 0, (2, True): 1, (1, False): 2, (3, True): 3, (2, False): 4, (0, True): 5,
                     (3, False): 6, (1, True): 7}
            return (order[(gemm, b)], group)
        for cta, lst in per_cta.items():
            keys = [position(*e) for e in lst]
            assert keys == sorted(keys), (cta, lst)


def test_schedule_plan_argument_errors(lib):
    count, info = ctypes.c_int(), (ctypes.c_int * _lib.PLAN_INFO)()
    assert lib.pi05_schedule_plan(148, 0, 128, None, None, 0, ctypes.byref(count), info) == _lib.ERR_ARGUMENT
    assert lib.pi05_schedule_plan(148, 17, 128, None, None, 0, ctypes.byref(count), info) == _lib.ERR_ARGUMENT
    assert lib.pi05_schedule_plan(148, 1, 128, None, None, 4, ctypes.byref(count), info) == _lib.ERR_ARGUMENT
    assert lib.pi05_schedule_plan(148, 1, 128, None, None, 0, None, info) == _lib.ERR_ARGUMENT
    assert lib.pi05_schedule_plan(60, 1, 128, None, None, 0, ctypes.byref(count), info) == _lib.ERR_UNSUPPORTED


@pytest.mark.parametrize("sms", list(range(132, 161, 2)))
@pytest.mark.parametrize("batch,prefix", [(1, 128), (1, 968), (5, 128), (16, 128)])
def test_schedule_plan_on_other_sm_counts(lib, sms, batch, prefix):
    """Parts with a few SMs more or fewer than 148: the plan sheds groups of row CTAs until the GEMM side keeps the
    fewest CTAs a schedule needs, instead of refusing."""
    count, info = ctypes.c_int(), (ctypes.c_int * _lib.PLAN_INFO)()
    assert lib.pi05_schedule_plan(sms, batch, prefix, None, None, 0, ctypes.byref(count), info) == _lib.OK
    assert info[0] >= 72 and info[0] == sms - 25 * max(info[1], info[2])


def test_tuning_defaults_and_clamping(lib):
    t = _lib.Tuning()
    assert lib.pi05_tuning_defaults(ctypes.byref(t)) == _lib.OK
    assert (t.poll_ns, t.two_streams, t.grouped_from, t.streams_from, t.clusters) == (20, 1, 3, 5, 1)
    assert lib.pi05_tuning_defaults(None) == _lib.ERR_ARGUMENT
    assert lib.pi05_tune(None, ctypes.byref(t)) == _lib.ERR_ARGUMENT
    # the plan follows the struct, not the environment
    count, info = ctypes.c_int(), (ctypes.c_int * _lib.PLAN_INFO)()
    t.two_streams = 0
    assert lib.pi05_schedule_plan(148, 8, 128, ctypes.byref(t), None, 0, ctypes.byref(count), info) == _lib.OK
    assert info[5] == 0
    t.two_streams, t.row_groups = 1, 99          # out of range: clamped to 3
    assert lib.pi05_schedule_plan(148, 8, 128, ctypes.byref(t), None, 0, ctypes.byref(count), info) == _lib.OK
    assert info[5] == 4 and info[1] == 3


@pytest.mark.parametrize("size", [2, 4, 8])
def test_tensor_parallel_plans_partition_the_work(lib, size):
    """The ranks' schedules together cover exactly the one-GPU schedule's work: the q tiles, the K range of the O
    projection, the gate/up tiles and the K range of the down projection are cut into `size` disjoint shares, rank r
    taking share r (heads 8 r / size .., MLP columns 4096 r / size ..); the k / v tiles run on every rank."""
    cover: dict = {}
    for rank in range(size):
        entries, plan = _lib.schedule_plan(148, 1, 128, rank, size)
        assert plan["gemm_ctas"] == 123
        mine: dict = {}
        for cta, gemm, lag, group, tile, k0, nk in entries:
            assert lag == 0 and group == -1
            for k in range(k0, k0 + nk):
                mine.setdefault((gemm, tile), []).append(k)
        for (gemm, tile), ks in mine.items():
            assert len(ks) == len(set(ks))
            if gemm == 0 and tile >= 16:
                assert sorted(ks) == list(range(STAGES[0]))               # k / v: the whole K on every rank
                continue
            if gemm == 0:
                assert tile // (16 // size) == rank and sorted(ks) == list(range(STAGES[0]))
            elif gemm == 2:
                assert tile // (64 // size) == rank and sorted(ks) == list(range(STAGES[2]))
            else:
                share = STAGES[gemm] // size
                assert sorted(ks) == list(range(rank * share, (rank + 1) * share))
            for k in ks:
                assert (gemm, tile, k) not in cover
                cover[(gemm, tile, k)] = rank
        assert plan["units"]["qkv"] == 4 + (16 // size) * 4
    for gemm in range(4):
        tiles = 16 if gemm == 0 else TILES[gemm]
        assert sum(1 for key in cover if key[0] == gemm) == tiles * STAGES[gemm]
    count, info = ctypes.c_int(), (ctypes.c_int * _lib.PLAN_INFO)()
    assert lib.pi05_schedule_plan_tp(148, 1, 128, 2, 2, None, None, 0, ctypes.byref(count), info) == _lib.ERR_ARGUMENT
    assert lib.pi05_schedule_plan_tp(148, 2, 128, 0, 2, None, None, 0, ctypes.byref(count), info) == _lib.ERR_UNSUPPORTED
    assert lib.pi05_schedule_plan_tp(148, 1, 128, 0, 3, None, None, 0, ctypes.byref(count), info) == _lib.ERR_UNSUPPORTED


def test_reference_arm_prints_the_contract_line():
    """`bench.py --impl reference` runs on the host cores alone: the reference's own eager path where it is installed
    beside the benchmark, else the oracle port; its one JSON line carries the keys the driver of the benchmark reads."""
    import json
    import subprocess
    import sys
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "3"],
                          capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["unit"] == "chunks/s" and d["higher_is_better"] is True and d["n_gpus"] == 1
    assert d["steps"] == 1 and d["warmup"] >= 3 and d["value"] > 0 and abs(d["value"] * d["ms_per_step"] - 1e3) < 1e-6 * 1e3
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1
    assert d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "chunks/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert "workload" in d["config"]
