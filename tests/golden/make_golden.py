"""Generate the golden vectors under tests/golden/ from the UNMODIFIED reference.

Run once, in a container that has the reference checkout:

    python tests/golden/make_golden.py --reference /path/to/reference

The reference imports ``megabench`` (its parent project), which is not shipped
with it.  This script installs a small in-memory stand-in for the five names
the reference imports from it; only ``attention`` and ``Case`` are used on the
path exercised here.  ``attention`` follows the explicit statement of the same
computation in the reference's own ``prefill`` (reference/pi05.py:184-188).

Outputs (numpy .npz, small):
  full_p128_s<seed>.npz   actions of reference() and of fp32_reference() for the
                          full geometry at prefix 128 on the three graded seeds,
                          inputs regenerated from the seed (fingerprints stored)
  full_p256_pad.npz       prefix 256, right-padded random-length mask
  small_*.npz             reduced geometries with every input tensor stored
  prefill_small_*.npz     the Gemma prefix prefill (reference/pi05.py::prefill and the same under the FP32 oracle's
                          dispatch mode) on reduced geometries, every input stored
  prefill_full_p160.npz   the prefill at the full Gemma-2B geometry, 160 tokens with a right-padded mask, inputs
                          regenerated from the seed (fingerprints stored), keys / values of layers 0, 8 and 17 stored
"""

from __future__ import annotations

import argparse
import dataclasses
import importlib
import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from pi05_megakernel_b200 import fixture as FX  # noqa: E402

MASK_VALUE = -2.3819763e38


def install_megabench_standin() -> None:
    @dataclasses.dataclass
    class Case:
        id: str = ""
        family: str = ""
        model: str = ""
        phase: str = ""
        params: dict = dataclasses.field(default_factory=dict)
        category: str = ""
        suite: str = ""
        atol: float = 0.0
        rtol: float = 0.0
        bf16_rtol: float = 0.0
        ready: bool = True
        note: str = ""

    def attention(query, key, content, allowed):
        qh, kvh, d = query.shape[1], key.shape[1], query.shape[2]
        groups = qh // kvh
        q, k, v = (t.transpose(0, 1) for t in (query, key.repeat_interleave(groups, 1),
                                               content.repeat_interleave(groups, 1)))
        scores = (q @ k.transpose(-1, -2)) * d ** -0.5
        scores = scores + torch.where(allowed, 0.0, MASK_VALUE).to(scores.dtype)[None]
        return (F.softmax(scores, -1, dtype=torch.float32).to(q.dtype) @ v).transpose(0, 1)

    def fill_layer_weights(g, device, shape, fan_in):
        return (torch.randn(shape, generator=g, device=device) * fan_in ** -0.5).to(torch.bfloat16)

    def _unused(*a, **k):
        raise RuntimeError("not on the action-chunk path")

    mb = types.ModuleType("megabench")
    cases = types.ModuleType("megabench.cases")
    tasks = types.ModuleType("megabench.tasks")
    common = types.ModuleType("megabench.tasks.common")
    vision = types.ModuleType("megabench.tasks.vision")
    cases.Case = Case
    def rms(x, weight, gemma=False):
        # the Gemma RMSNorm the reference names as upstream: FP32 normalisation, scale (1 + weight), cast back
        assert gemma
        xf = x.float()
        normalized = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + 1e-6)
        return (normalized * (1.0 + weight.float())).to(x.dtype)

    common.attention, common.fill_layer_weights = attention, fill_layer_weights
    common.rms = rms
    common.random_norm = common.random_weight = _unused
    vision.vision_inputs = _unused
    for name, mod in (("megabench", mb), ("megabench.cases", cases), ("megabench.tasks", tasks),
                      ("megabench.tasks.common", common), ("megabench.tasks.vision", vision)):
        sys.modules[name] = mod


def load_reference(path: str):
    install_megabench_standin()
    parent, name = os.path.split(os.path.abspath(path.rstrip("/")))
    sys.path.insert(0, parent)
    fixture = importlib.import_module(f"{name}.fixture")
    return fixture


def case_for(fixture, geo: FX.Geometry):
    rgeo = fixture.Geometry(prefix=geo.prefix, horizon=geo.horizon, action_dim=geo.action_dim,
                            layers=geo.layers, steps=geo.steps, hidden=geo.hidden,
                            intermediate=geo.intermediate, q_heads=geo.q_heads,
                            kv_heads=geo.kv_heads, head_dim=geo.head_dim)
    return fixture.make_case(rgeo)


def run_reference(fixture, geo: FX.Geometry, inputs: dict):
    case = case_for(fixture, geo)
    with torch.no_grad():
        want = fixture.ref.reference(case, inputs)["actions"]
    exact = fixture.fp32_reference(fixture.ref, case, inputs)["actions"]
    return want, exact


def fingerprints(inputs: dict) -> dict:
    return {k: np.array([v.double().sum().item(), v.double().abs().sum().item()])
            for k, v in inputs.items()}


def to_np(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy()
    return t.numpy()


SMALL = {
    # name: (geometry, mask kind, seed)
    "small_gqa1": (FX.Geometry(prefix=7, horizon=5, action_dim=4, layers=2, steps=3, hidden=64,
                               intermediate=128, q_heads=4, kv_heads=1, head_dim=16), "scatter", 11),
    "small_gqa2": (FX.Geometry(prefix=12, horizon=6, action_dim=8, layers=3, steps=2, hidden=96,
                               intermediate=160, q_heads=4, kv_heads=2, head_dim=32), "pad", 12),
    "small_full": (FX.Geometry(prefix=16, horizon=50, action_dim=32, layers=2, steps=10, hidden=128,
                               intermediate=256, q_heads=8, kv_heads=1, head_dim=32), "full", 13),
}


PREFILL_SMALL = {
    "prefill_small_a": (FX.PrefillGeometry(tokens=24, layers=2, hidden=64, intermediate=128, q_heads=2, kv_heads=1,
                                           head_dim=16), "pad", 21),
    "prefill_small_b": (FX.PrefillGeometry(tokens=40, layers=3, hidden=128, intermediate=256, q_heads=8, kv_heads=1,
                                           head_dim=32), "full", 22),
}
PREFILL_FULL = ("prefill_full_p160", FX.PrefillGeometry(tokens=160), "pad", 23, (0, 8, 17))


def run_reference_prefill(fixture, geo: FX.PrefillGeometry, inputs: dict):
    """reference/pi05.py::prefill as it is, and the same call under the FP32 oracle's dispatch mode."""
    from types import SimpleNamespace
    case = SimpleNamespace(params={"head_dim": geo.head_dim, "q_heads": geo.q_heads, "kv_heads": geo.kv_heads,
                                   "layers": geo.layers})
    oracle = importlib.import_module(fixture.__name__.rsplit(".", 1)[0] + ".reference.oracle")
    with torch.no_grad():
        k, v = fixture.ref.prefill(case, inputs, inputs["embeddings"], inputs["valid"])
        with oracle.WidenBf16():
            ke, ve = fixture.ref.prefill(case, inputs, inputs["embeddings"], inputs["valid"])
    return k, v, ke.float(), ve.float()


def make_prefill(fixture) -> None:
    for name, (geo, mask, seed) in PREFILL_SMALL.items():
        inputs = FX.make_prefill_inputs(geo, seed, mask)
        k, v, ke, ve = run_reference_prefill(fixture, geo, inputs)
        blob = {"in_" + key: to_np(val) for key, val in inputs.items()}
        blob.update(k=to_np(k), v=to_np(v), k_exact=ke.numpy(), v_exact=ve.numpy(),
                    geo=np.array(dataclasses.astuple(geo), dtype=np.int64))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
        print(name, "k", float(k.float().abs().max()), "diff", float((k.float() - ke).abs().max()))
    name, geo, mask, seed, keep = PREFILL_FULL
    inputs = FX.make_prefill_inputs(geo, seed, mask)
    k, v, ke, ve = run_reference_prefill(fixture, geo, inputs)
    blob = {"fp_" + key: val for key, val in fingerprints(inputs).items()}
    blob.update(seed=np.int64(seed), valid=inputs["valid"].numpy(), layers_kept=np.array(keep, dtype=np.int64),
                k=to_np(k[list(keep)].contiguous()), v=to_np(v[list(keep)].contiguous()),
                k_exact=ke[list(keep)].numpy(), v_exact=ve[list(keep)].numpy(),
                geo=np.array(dataclasses.astuple(geo), dtype=np.int64))
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
    print(name, "rel k", float((k.float() - ke).norm() / ke.norm()), "rel v", float((v.float() - ve).norm() / ve.norm()))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of garv901/pi05-megakernel (its top-level directory)")
    ap.add_argument("--skip-full", action="store_true")
    ap.add_argument("--only-prefill", action="store_true")
    args = ap.parse_args()
    torch.manual_seed(0)
    fixture = load_reference(args.reference)
    make_prefill(fixture)
    if args.only_prefill:
        return

    for name, (geo, mask, seed) in SMALL.items():
        inputs = FX.make_inputs(geo, seed, "cpu", mask)
        want, exact = run_reference(fixture, geo, inputs)
        blob = {"in_" + k: to_np(v) for k, v in inputs.items()}
        blob.update(want=want.numpy(), exact=exact.numpy(),
                    geo=np.array(dataclasses.astuple(geo), dtype=np.int64))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
        print(name, "want", float(want.abs().max()), "diff", float((want - exact).abs().max()))

    if args.skip_full:
        return
    full = [(f"full_p128_s{s}", FX.Geometry(prefix=128), "full", s) for s in FX.SEEDS]
    full.append(("full_p256_pad", FX.Geometry(prefix=256), "pad", FX.SEEDS[0]))
    for name, geo, mask, seed in full:
        inputs = FX.make_inputs(geo, seed, "cpu", mask)
        want, exact = run_reference(fixture, geo, inputs)
        blob = {"fp_" + k: v for k, v in fingerprints(inputs).items()}
        blob.update(want=want.numpy(), exact=exact.numpy(), seed=np.int64(seed),
                    mask=inputs["prefix_mask"].numpy(),
                    geo=np.array(dataclasses.astuple(geo), dtype=np.int64))
        np.savez_compressed(os.path.join(HERE, name + ".npz"), **blob)
        rel = float((want.double() - exact.double()).norm() / exact.double().norm())
        print(name, "rel_ref", rel, "maxabs_ref", float((want - exact).abs().max()),
              "max|exact|", float(exact.abs().max()))


if __name__ == "__main__":
    main()
