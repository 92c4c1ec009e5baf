"""Geometry, input order and seeded synthetic inputs of the pi0.5 action chunk.

Mirrors the reference's ``fixture.py`` (``Geometry`` 30-47) and the input
order of its megakernel arm (``megakernel.py:21-25``).  Inputs are synthetic:
every weight and bias is drawn from N(0, 0.02) (BF16 for the seven expert
projections, FP32 for the time MLP, the action projections and the adaRMS
modulation layers), the per-layer prefix K/V from N(0, 1) rounded to BF16 and
the noise from N(0, 1), all from CPU generators so that the same seed gives the
same tensors on any machine with the same torch build.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

# Order in which tensors are handed to the engine (reference megakernel.py:21-25).
ORDER = ("action_in_weight", "action_in_bias", "time_in_weight", "time_in_bias",
         "time_out_weight", "time_out_bias", "action_out_weight", "action_out_bias",
         "wq", "wk", "wv", "wo", "wg", "wu", "wd",
         "attn_norm_weight", "attn_norm_bias", "ffn_norm_weight", "ffn_norm_bias",
         "final_norm_weight", "final_norm_bias", "noise", "prefix_k", "prefix_v", "prefix_mask")
OBSERVATION = ("noise", "prefix_k", "prefix_v", "prefix_mask")   # per-observation tensors; the rest are weights
SEEDS = (7301, 8917, 42811)          # reference bench.py:373
WEIGHT_STD = 0.02


@dataclass(frozen=True)
class Geometry:
    prefix: int = 128
    horizon: int = 50
    action_dim: int = 32
    layers: int = 18
    steps: int = 10
    hidden: int = 1024
    intermediate: int = 4096
    q_heads: int = 8
    kv_heads: int = 1
    head_dim: int = 256

    @property
    def id(self) -> str:
        return f"pi05-b1-p{self.prefix}"


def shapes(geo: Geometry) -> dict:
    """name -> (shape, dtype) of every input (reference/pi05.py:71-97)."""
    w, L, a = geo.hidden, geo.layers, geo.action_dim
    qd, kvd, inter = geo.q_heads * geo.head_dim, geo.kv_heads * geo.head_dim, geo.intermediate
    f32, bf16 = torch.float32, torch.bfloat16
    return {
        "action_in_weight": ((w, a), f32), "action_in_bias": ((w,), f32),
        "time_in_weight": ((w, w), f32), "time_in_bias": ((w,), f32),
        "time_out_weight": ((w, w), f32), "time_out_bias": ((w,), f32),
        "action_out_weight": ((a, w), f32), "action_out_bias": ((a,), f32),
        "wq": ((L, qd, w), bf16), "wk": ((L, kvd, w), bf16), "wv": ((L, kvd, w), bf16),
        "wo": ((L, w, qd), bf16), "wg": ((L, inter, w), bf16), "wu": ((L, inter, w), bf16),
        "wd": ((L, w, inter), bf16),
        "attn_norm_weight": ((L, 3 * w, w), f32), "attn_norm_bias": ((L, 3 * w), f32),
        "ffn_norm_weight": ((L, 3 * w, w), f32), "ffn_norm_bias": ((L, 3 * w), f32),
        "final_norm_weight": ((3 * w, w), f32), "final_norm_bias": ((3 * w,), f32),
        "noise": ((geo.horizon, a), f32),
        "prefix_k": ((L, geo.prefix, geo.kv_heads, geo.head_dim), bf16),
        "prefix_v": ((L, geo.prefix, geo.kv_heads, geo.head_dim), bf16),
        "prefix_mask": ((geo.prefix,), torch.bool),
    }


def make_weights(geo: Geometry, seed: int) -> dict:
    """Expert, time-MLP, action and modulation parameters (CPU tensors)."""
    g = torch.Generator().manual_seed(seed ^ 0xAC71)
    out = {}
    for name, (shape, dtype) in shapes(geo).items():
        if name in ("noise", "prefix_k", "prefix_v", "prefix_mask"):
            continue
        out[name] = (torch.randn(shape, generator=g) * WEIGHT_STD).to(dtype)
    return out


def make_observation(geo: Geometry, seed: int, mask: str = "full") -> dict:
    """Per-observation tensors: noise, prefix K/V and the prefix validity mask.

    ``mask``: "full" = every prefix token valid; "pad" = a right-padded prefix
    whose valid count is uniform in [prefix/2, prefix]; "scatter" = the same
    count of valid tokens at random places.
    """
    g = torch.Generator().manual_seed(seed ^ 0x9A11)
    kv = (geo.layers, geo.prefix, geo.kv_heads, geo.head_dim)
    out = {"noise": torch.randn((geo.horizon, geo.action_dim), generator=g),
           "prefix_k": torch.randn(kv, generator=g).to(torch.bfloat16),
           "prefix_v": torch.randn(kv, generator=g).to(torch.bfloat16)}
    if mask == "full":
        out["prefix_mask"] = torch.ones(geo.prefix, dtype=torch.bool)
    else:
        lo = geo.prefix // 2
        n = int(torch.randint(lo, geo.prefix + 1, (), generator=g))
        if mask == "pad":
            out["prefix_mask"] = torch.arange(geo.prefix) < n
        elif mask == "scatter":
            m = torch.zeros(geo.prefix, dtype=torch.bool)
            m[torch.randperm(geo.prefix, generator=g)[:n]] = True
            out["prefix_mask"] = m
        else:
            raise ValueError(f"unknown mask kind {mask!r}")
    return out


def make_inputs(geo: Geometry, seed: int, device: str = "cpu", mask: str = "full") -> dict:
    """All 25 inputs for one seed, in ``ORDER``, on ``device``."""
    values = make_weights(geo, seed)
    values.update(make_observation(geo, seed, mask))
    return {k: values[k].to(device) for k in ORDER}


def make_batch(geo: Geometry, seed: int, batch: int, device: str = "cpu", masks=None) -> tuple[dict, list[dict]]:
    """Weights of `seed` plus `batch` independent observations (seed + 1, seed + 2, ...).

    Returns the stacked inputs for the engine (observation tensors get a leading batch index) and the list of
    per-observation input dicts for a reference that works one observation at a time."""
    weights = make_weights(geo, seed)
    masks = masks or ["full"] * batch
    per = [{**weights, **make_observation(geo, seed + 1 + b, masks[b])} for b in range(batch)]
    stacked = dict(weights)
    for name in OBSERVATION:
        stacked[name] = torch.stack([o[name] for o in per]).contiguous()
    return {k: stacked[k].to(device) for k in ORDER}, [{k: o[k] for k in ORDER} for o in per]


def sol(geo: Geometry, batch: int = 1) -> dict:
    """HBM floor of the reference harness (bench.py:63-80), per launch of ``batch`` chunks."""
    L, W, I, S, T = geo.layers, geo.hidden, geo.intermediate, geo.steps, geo.horizon
    qd, kvd = geo.q_heads * geo.head_dim, geo.kv_heads * geo.head_dim
    layer_params = W * (qd + 2 * kvd) + qd * W + 3 * W * I
    expert = L * layer_params * 2
    fp32_once = (L * 2 + 1) * 3 * W * W * 4 + 2 * W * W * 4 + 2 * W * geo.action_dim * 4
    kv = L * geo.prefix * kvd * 2 * 2
    bytes_stream = S * (expert + batch * kv) + fp32_once
    flops = batch * S * (2 * T * L * layer_params + L * 4 * T * qd * (geo.prefix + T))
    return {"expert_weight_bytes": expert, "fp32_cond_weight_bytes": fp32_once,
            "prefix_kv_bytes": kv, "bytes_restream": bytes_stream, "flops": flops,
            "floor_restream_ms": bytes_stream / 8.0e12 * 1e3}


# ------------------------------------------------------------------------------------------- prefix prefill
# The step before the action chunk: the Gemma-2B prefix-LM prefill that produces the per-layer K/V cache
# (reference/pi05.py:167-195, weights as in reference/pi05.py:100-116).
PREFILL_WEIGHTS = ("ln1", "ln2", "lq", "lk", "lv", "lo", "lg", "lu", "ld")


@dataclass(frozen=True)
class PrefillGeometry:
    tokens: int = 968           # prefix length P: 3 x 256 image tokens + 200 prompt tokens in the graded case
    layers: int = 18
    hidden: int = 2048
    intermediate: int = 16384
    q_heads: int = 8
    kv_heads: int = 1
    head_dim: int = 256


def prefill_shapes(geo: PrefillGeometry) -> dict:
    h, L, inter = geo.hidden, geo.layers, geo.intermediate
    qd, kvd = geo.q_heads * geo.head_dim, geo.kv_heads * geo.head_dim
    bf16 = torch.bfloat16
    return {"ln1": ((L, h), bf16), "ln2": ((L, h), bf16),
            "lq": ((L, qd, h), bf16), "lk": ((L, kvd, h), bf16), "lv": ((L, kvd, h), bf16), "lo": ((L, h, qd), bf16),
            "lg": ((L, inter, h), bf16), "lu": ((L, inter, h), bf16), "ld": ((L, h, inter), bf16),
            "embeddings": ((geo.tokens, h), bf16), "valid": ((geo.tokens,), torch.bool)}


def make_prefill_inputs(geo: PrefillGeometry, seed: int, mask: str = "pad") -> dict:
    """Synthetic prefill inputs: projection weights N(0, 1/fan_in) in BF16 (the reference's ``fill_layer_weights``),
    norm weights N(0, 0.1), unit-variance embeddings, and a validity mask ("full", or "pad": a right-padded prompt as
    ``prompt`` builds it, reference/pi05.py:143-164, valid count uniform in [tokens/2, tokens])."""
    g = torch.Generator().manual_seed(seed ^ 0x9A11)
    out = {}
    for name, (shape, dtype) in prefill_shapes(geo).items():
        if name in ("ln1", "ln2"):
            out[name] = (torch.randn(shape, generator=g) * 0.1).to(dtype)
        elif name in PREFILL_WEIGHTS:
            out[name] = (torch.randn(shape, generator=g) * shape[-1] ** -0.5).to(dtype)
    out["embeddings"] = torch.randn((geo.tokens, geo.hidden), generator=g).to(torch.bfloat16)
    if mask == "full":
        out["valid"] = torch.ones(geo.tokens, dtype=torch.bool)
    elif mask == "pad":
        n = int(torch.randint(geo.tokens // 2, geo.tokens + 1, (), generator=g))
        out["valid"] = torch.arange(geo.tokens) < n
    else:
        raise ValueError(f"unknown mask kind {mask!r}")
    return out
