"""Shared helpers of the test-suite (loading golden vectors, geometry conversion)."""
import dataclasses
import os

import numpy as np
import torch

from oracle import pi05_oracle as O
from pi05_megakernel_b200 import fixture as FX

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_small(name: str):
    """Inputs, reference actions and oracle actions of a stored reduced-geometry case."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dims = [int(x) for x in z["geo"]]
    geo, ogeo = FX.Geometry(*dims), O.Geo(*dims)
    inputs = {}
    for key, (shape, dtype) in FX.shapes(geo).items():
        t = torch.from_numpy(z["in_" + key])
        inputs[key] = t.view(torch.bfloat16) if dtype == torch.bfloat16 else t
        assert tuple(inputs[key].shape) == tuple(shape)
    return geo, ogeo, inputs, torch.from_numpy(z["want"]), torch.from_numpy(z["exact"])


def load_full(name: str):
    """Geometry, seed, mask kind data and stored reference outputs of a full-geometry case."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    dims = [int(x) for x in z["geo"]]
    fps = {k[3:]: z[k] for k in z.files if k.startswith("fp_")}
    return (FX.Geometry(*dims), O.Geo(*dims), int(z["seed"]), torch.from_numpy(z["mask"]), fps,
            torch.from_numpy(z["want"]), torch.from_numpy(z["exact"]))


def fingerprints_match(inputs: dict, fps: dict) -> bool:
    for k, v in inputs.items():
        got = np.array([v.double().sum().item(), v.double().abs().sum().item()])
        if not np.allclose(got, fps[k], rtol=1e-12, atol=0):
            return False
    return True


def geo_tuple(geo) -> tuple:
    return dataclasses.astuple(geo)


def load_prefill(name: str):
    """A stored prefill case: geometry, inputs (regenerated from the seed for the full-geometry case, whose stored
    fingerprints are checked), and the keys / values of reference/pi05.py::prefill in BF16 and under the FP32 oracle
    (all layers for the small cases, the layers listed in ``layers_kept`` for the full one)."""
    z = np.load(os.path.join(GOLDEN, name + ".npz"))
    geo = FX.PrefillGeometry(*[int(x) for x in z["geo"]])
    bf = lambda a: torch.from_numpy(a).view(torch.bfloat16)
    if "seed" in z.files:
        inputs = FX.make_prefill_inputs(geo, int(z["seed"]), "pad")
        fps = {k[3:]: z[k] for k in z.files if k.startswith("fp_")}
        kept = [int(x) for x in z["layers_kept"]]
    else:
        inputs, fps, kept = {}, None, list(range(geo.layers))
        for key, (shape, dtype) in FX.prefill_shapes(geo).items():
            t = torch.from_numpy(z["in_" + key])
            inputs[key] = t.view(torch.bfloat16) if dtype == torch.bfloat16 else t
            assert tuple(inputs[key].shape) == tuple(shape)
    return geo, inputs, fps, kept, bf(z["k"]), bf(z["v"]), torch.from_numpy(z["k_exact"]), torch.from_numpy(z["v_exact"])
