"""The Gemma-2B prefix prefill on the GPU against the CPU oracle (and, through it, against the unmodified reference's
stored outputs, which the oracle matches bit for bit).

Tolerance: the reference harness's band, applied to the keys and the values of the valid tokens: the engine's error
against the FP32 oracle may be at most twice the BF16 eager path's own error plus rtol 0.003 (relative L2), and its
largest absolute error at most twice the eager path's plus atol 0.003 + 0.003 max|exact| (fixture.py:105-120 of the
reference).  Rows of padded tokens are not compared: the reference lets padded query rows attend uniformly to
everything, the engine lets them attend to the valid keys, and neither is ever read as a key or a value.
"""
import pytest
import torch

from oracle import pi05_oracle as O
from pi05_megakernel_b200 import fixture as FX
from tests.helpers import fingerprints_match, load_prefill

pytestmark = pytest.mark.gpu


def _band(got, want, exact):
    return O.band(want.float(), got.float(), exact.float())


def _run(geo, inputs, layers=None):
    from pi05_megakernel_b200.prefill import Pi05Prefill
    dev = {k: v.cuda() for k, v in inputs.items()}
    pre = Pi05Prefill(geo, "cuda")
    pre.bind(dev)
    k, v = pre.run(dev["embeddings"], dev["valid"], layers)
    pre.status()
    k2, v2 = pre.run(dev["embeddings"], dev["valid"], layers)       # a second run from the same handle: same answer
    pre.status()
    assert torch.equal(k, k2) and torch.equal(v, v2)
    pre.close()
    return k.cpu(), v.cpu()


@pytest.mark.parametrize("tokens,mask,layers", [(64, "full", 1), (200, "pad", 2), (131, "pad", 3), (300, "pad", 2), (650, "pad", 3)])
def test_first_layers_against_the_oracle(tokens, mask, layers):
    """Short runs: one to three layers, token counts that do not fill the 128-token tiles or the 64-key chunks.  Up to 512
    tokens the down projection runs as a stream-K launch (partial tiles summed through the workspace), beyond as whole
    tiles: the 650-token case covers that path and an attention of eleven key chunks.  From two 128-token tiles on the big
    GEMMs run on CTA pairs over 256 tokens: 300 tokens leave the second CTA of the last pair without any token."""
    geo = FX.PrefillGeometry(tokens=tokens)
    inputs = FX.make_prefill_inputs(geo, 31, mask)
    args = (inputs, inputs["embeddings"], inputs["valid"], geo.q_heads, geo.kv_heads, geo.head_dim)
    wk, wv = O.prefill(*args, widen=False, layers=layers)
    ek, ev = O.prefill(*args, widen=True, layers=layers)
    k, v = _run(geo, inputs, layers)
    rows = inputs["valid"]
    for name, got, want, exact in (("k", k[:layers], wk, ek), ("v", v[:layers], wv, ev)):
        d = _band(got[:, rows], want[:, rows], exact[:, rows])
        assert d["pass"], (name, d)
        # layer 0 keys and values depend on one GEMM and one norm only: far tighter than the band
        err = (got[0][rows].float() - want[0][rows].float()).norm() / want[0][rows].float().norm()
        assert float(err) < 4e-3, (name, float(err))


def test_full_depth_against_stored_reference_outputs():
    """All 18 layers at 160 tokens (right-padded mask): keys / values of layers 0, 8 and 17 against what the unmodified
    reference and its FP32 dispatch mode produced (tests/golden/prefill_full_p160.npz)."""
    geo, inputs, fps, kept, wk, wv, ek, ev = load_prefill("prefill_full_p160")
    if not fingerprints_match(inputs, fps):
        pytest.fail("this torch build draws different random inputs than the one that made the golden vectors; "
                    "regenerate them with tests/golden/make_golden.py")
    k, v = _run(geo, inputs)
    rows = inputs["valid"]
    for name, got, want, exact in (("k", k[kept], wk, ek), ("v", v[kept], wv, ev)):
        d = _band(got[:, rows], want[:, rows], exact[:, rows])
        assert d["pass"], (name, d)


def test_prefill_feeds_the_chunk_engine():
    """The prefill's outputs are the chunk engine's prefix cache as they are: bind them and run a short chunk; the
    result must sit in the band of the oracle's chunk over the oracle's own prefill."""
    from pi05_megakernel_b200.arm import Pi05Arm
    from pi05_megakernel_b200.prefill import Pi05Prefill
    pgeo = FX.PrefillGeometry(tokens=128)
    pin = FX.make_prefill_inputs(pgeo, 41, "pad")
    pdev = {k: v.cuda() for k, v in pin.items()}
    pre = Pi05Prefill(pgeo, "cuda")
    pre.bind(pdev)
    k, v = pre.run(pdev["embeddings"], pdev["valid"])
    pre.status()
    geo, ogeo = FX.Geometry(prefix=128), O.Geo(prefix=128)
    cpu = FX.make_inputs(geo, FX.SEEDS[0], "cpu")
    dev = {n: t.cuda() for n, t in cpu.items()}
    dev.update(prefix_k=k, prefix_v=v, prefix_mask=pdev["valid"])
    arm = Pi05Arm(geo, "b200-s2-l3", "cuda")
    arm.bind(dev)
    arm.launch()
    arm.status()
    got = arm.outputs()["actions"].cpu()
    ok_, ov_ = O.prefill(pin, pin["embeddings"], pin["valid"], 8, 1, 256)
    ref_in = dict(cpu, prefix_k=ok_, prefix_v=ov_, prefix_mask=pin["valid"])
    want, exact = O.chunk(ref_in, ogeo, False, 2, 3), O.chunk(ref_in, ogeo, True, 2, 3)
    # the cache itself carries the prefill's BF16 noise on top of the chunk's, so the chunk band is widened by the
    # relative difference between the two caches
    d = O.band(want, got, exact)
    drift = float((k.cpu().float() - ok_.float())[:, pin["valid"]].norm() / ok_.float()[:, pin["valid"]].norm())
    assert d["relative_error"] <= 2 * d["reference_relative_error"] + O.RTOL + drift, (d, drift)
    arm.close()
    pre.close()
