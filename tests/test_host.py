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
    assert lib.pi05_create(0, 128, 1, 0, 2, ctypes.byref(h)) == _lib.ERR_UNSUPPORTED
    n = ctypes.c_size_t()
    assert lib.pi05_workspace_bytes(None, ctypes.byref(n)) == _lib.ERR_ARGUMENT
    assert lib.pi05_launch(None, 10, 18, None, None) == _lib.ERR_ARGUMENT
    assert lib.pi05_destroy(None) == _lib.ERR_ARGUMENT
    if not torch.cuda.is_available():
        assert lib.pi05_create(0, 128, 1, 0, 1, ctypes.byref(h)) == _lib.ERR_NO_DEVICE
        assert not h.value


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
