"""Install the unmodified reference next to this file, under ``baseline/_ref`` (kept out of the history).

The reference is a sub-package of its author's ``megabench`` project and ships neither that parent nor a
``setup.py``, so there is nothing for pip to build: this recipe copies the files of the action-chunk path as they
are (``fixture.py``, ``megakernel.py``, ``reference/``, ``mk/pi05_mk.cu``) to ``_ref/megabench/sota/pi05/`` - the
package path its own relative imports expect - and writes a small stand-in for the five names it imports from
the missing parent (``megabench.cases.Case``, ``megabench.tasks.common.{attention, fill_layer_weights, random_norm,
random_weight, rms}``, ``megabench.tasks.vision.vision_inputs``).  Only ``Case``, ``attention`` and
``fill_layer_weights`` are reached on the action-chunk path; ``attention`` restates the explicit twin in the
reference's own ``prefill`` (reference/pi05.py:184-188).

    python baseline/install_reference.py --reference /path/to/reference [--prebuild 128:k16-nofgu 968:k64]

``--prebuild`` compiles the reference's CUDA extension for the given ``prefix:variant`` pairs with the reference's
own ``megakernel.load`` (``torch.utils.cpp_extension``; no GPU needed) into ``_ref/torch_ext``, so that a GPU box
that receives the folder only has to load it.
"""

from __future__ import annotations

import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")
PKG = os.path.join(DEST, "megabench", "sota", "pi05")
EXT_DIR = os.path.join(DEST, "torch_ext")

COPY = ("__init__.py", "fixture.py", "megakernel.py", "reference", os.path.join("mk", "pi05_mk.cu"))

CASES = '''"""Stand-in for megabench.cases: the fields the reference's fixture passes."""
import dataclasses


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
'''

COMMON = '''"""Stand-in for megabench.tasks.common (only attention and fill_layer_weights are on the action-chunk path)."""
import torch
import torch.nn.functional as F

MASK_VALUE = -2.3819763e38


def attention(query, key, content, allowed):
    """GQA attention as the reference's prefill states it explicitly (reference/pi05.py:184-188): scores and
    probabilities in the tensors' dtype, softmax in FP32, finite additive mask."""
    qh, kvh, d = query.shape[1], key.shape[1], query.shape[2]
    groups = qh // kvh
    q, k, v = (t.transpose(0, 1) for t in (query, key.repeat_interleave(groups, 1),
                                           content.repeat_interleave(groups, 1)))
    scores = (q @ k.transpose(-1, -2)) * d ** -0.5
    scores = scores + torch.where(allowed, 0.0, MASK_VALUE).to(scores.dtype)[None]
    return (F.softmax(scores, -1, dtype=torch.float32).to(q.dtype) @ v).transpose(0, 1)


def fill_layer_weights(g, device, shape, fan_in):
    return (torch.randn(shape, generator=g, device=device) * fan_in ** -0.5).to(torch.bfloat16)


def _unused(*args, **kwargs):
    raise RuntimeError("not on the action-chunk path")


random_norm = random_weight = rms = _unused
'''

VISION = '''"""Stand-in for megabench.tasks.vision (not on the action-chunk path)."""


def vision_inputs(*args, **kwargs):
    raise RuntimeError("not on the action-chunk path")
'''


def install(reference: str) -> None:
    if not os.path.isfile(os.path.join(reference, "megakernel.py")):
        raise SystemExit(f"{reference} does not look like the reference checkout")
    if os.path.isdir(os.path.join(DEST, "megabench")):
        shutil.rmtree(os.path.join(DEST, "megabench"))
    os.makedirs(PKG)
    for rel in COPY:
        src, dst = os.path.join(reference, rel), os.path.join(PKG, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        if os.path.isdir(src):
            shutil.copytree(src, dst, ignore=shutil.ignore_patterns("__pycache__"))
        else:
            shutil.copy2(src, dst)
    for rel, text in (("__init__.py", ""), ("cases.py", CASES), (os.path.join("sota", "__init__.py"), ""),
                      (os.path.join("tasks", "__init__.py"), ""), (os.path.join("tasks", "common.py"), COMMON),
                      (os.path.join("tasks", "vision.py"), VISION)):
        path = os.path.join(DEST, "megabench", rel)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            f.write(text)


def prebuild(pairs: list[str]) -> None:
    os.environ["TORCH_EXTENSIONS_DIR"] = EXT_DIR
    os.makedirs(EXT_DIR, exist_ok=True)
    sys.path.insert(0, DEST)
    from megabench.sota.pi05 import megakernel as MK
    for pair in pairs:
        prefix, variant = pair.split(":")
        pv = MK.parse_variant(variant)
        extra = tuple(flag for on, flag in ((pv["hoist_off"], "-DPI05_LOAD_HOIST=0"), (pv["spread_off"], "-DPI05_GEMM_SPREAD=0"),
                                            (pv["part_bf16_off"], "-DPI05_PART_BF16=0"), (pv["fgu_off"], "-DPI05_FG_UMMA=0"),
                                            (pv["att_k2_off"], "-DPI05_ATT_K2=0"), (pv["ab_umma_off"], "-DPI05_AB_UMMA=0"),
                                            (pv["h_umma_off"], "-DPI05_H_UMMA=0")) if on)
        print(f"building prefix {prefix} variant {variant} {extra}", flush=True)
        MK.load(int(prefix), pv["att_keys"], extra)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("PI05_REFERENCE_DIR", ""),
                    help="root of the reference's source tree (or set PI05_REFERENCE_DIR)")
    ap.add_argument("--prebuild", nargs="*", default=[])
    args = ap.parse_args()
    if not args.reference or not os.path.isdir(args.reference):
        raise SystemExit("give the reference's source tree with --reference DIR")
    install(args.reference)
    print("installed", PKG)
    if args.prebuild:
        prebuild(args.prebuild)


if __name__ == "__main__":
    main()
