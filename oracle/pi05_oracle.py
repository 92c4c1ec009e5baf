"""CPU oracle for one pi0.5 action chunk.  TEST INFRASTRUCTURE ONLY.

This file is a checker, not a product path: only the tests, the smoke check and
the ``cpu_baseline`` / reference legs of the benchmark may import it.  The
shipped engine never calls it and has no CPU fallback.

It restates, with plain torch-on-CPU ops, the algorithm of the reference
project's eager definition of the chunk and of its FP32 oracle:

* ``chunk(inputs, geo, widen=False)`` follows ``reference/pi05.py:299-309``
  (``reference``) op by op, so the BF16 rounding schedule is the graded one.
* ``chunk(inputs, geo, widen=True)`` is the same graph with every BF16 tensor
  and every cast to BF16 widened to FP32, which is what
  ``reference/oracle.py:35-53`` (``WidenBf16`` / ``fp32_reference``) produces.
* ``attention`` restates ``megabench.tasks.common.attention``; that module is
  a dependency of the reference which is not shipped with it (no version pin).
  The restatement follows the explicit twin in ``reference/pi05.py:184-188``
  and the docstring at ``reference/pi05.py:21-22``.
* ``band`` / ``snapshot`` follow ``fixture.py:105-126``; ``sol_bytes`` follows
  ``bench.py:63-80``.

Pinning: ``tests/golden/make_golden.py`` imports the unmodified reference
(through a small stand-in for the missing ``megabench`` package) and stores
its outputs; ``tests/test_oracle.py`` checks this file against those vectors
bit for bit.  The one part with no vector from the reference's own tests is
``megabench.tasks.common.attention`` itself (parity unpinned for that single
function: the reference ships neither its source nor a test for it).

``stages`` additionally returns the intermediates of one layer pass in the
rounding schedule the CUDA engine uses, for stage-by-stage kernel checks.
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

MIN_PERIOD, MAX_PERIOD = 4e-3, 4.0          # reference/pi05.py:36
ROPE_THETA = 10_000.0                        # reference/pi05.py:37
EPS = 1e-6                                   # reference/pi05.py:38
MASK_VALUE = -2.3819763e38                   # reference/pi05.py:40
NOISE_FACTOR = 2.0                           # fixture.py:27
ATOL, RTOL, BF16_RTOL = 0.003, 0.003, 0.008  # fixture.py:62

BF16 = torch.bfloat16


@dataclass(frozen=True)
class Geo:
    """Shape of one chunk (fixture.py:30-47, expert part only)."""
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


def _cast(widen: bool):
    """BF16 cast of the graded schedule, or the FP32 widening of the oracle."""
    return (lambda t: t.float()) if widen else (lambda t: t.to(BF16))


def rope(x: torch.Tensor, positions: torch.Tensor, cast) -> torch.Tensor:
    """reference/pi05.py:218-229.  cos/sin are cast to the activation dtype."""
    width = x.shape[-1]
    inv = 1.0 / (ROPE_THETA ** (torch.arange(0, width, 2, dtype=torch.int64).float() / width))
    phase = positions.float()[:, None] * inv[None, :]
    phase = torch.cat((phase, phase), -1)
    cos, sin = cast(phase.cos())[:, None], cast(phase.sin())[:, None]
    half = width // 2
    return x * cos + torch.cat((-x[..., half:], x[..., :half]), -1) * sin


def time_embedding(time: torch.Tensor, width: int) -> torch.Tensor:
    """reference/pi05.py:232-237: FP64 sine-cosine embedding, cast to FP32."""
    fraction = torch.linspace(0.0, 1.0, width // 2, dtype=torch.float64)
    period = MIN_PERIOD * (MAX_PERIOD / MIN_PERIOD) ** fraction
    phase = time[..., None] * (1.0 / period * 2 * math.pi)
    return torch.cat((phase.sin(), phase.cos()), -1).to(time.dtype)


def ada_rms(x: torch.Tensor, modulation: torch.Tensor, cast):
    """reference/pi05.py:240-244."""
    normalized = x * torch.rsqrt(x.float().square().mean(-1, keepdim=True) + EPS)
    scale, shift, gate = modulation.chunk(3, -1)
    return cast(normalized * (1 + scale.float()) + shift.float()), cast(gate)


def time_condition(v: dict, time: torch.Tensor, width: int) -> torch.Tensor:
    """reference/pi05.py:247-251."""
    cond = time_embedding(time, width)
    cond = F.silu(F.linear(cond, v["time_in_weight"], v["time_in_bias"]))
    return F.silu(F.linear(cond, v["time_out_weight"], v["time_out_bias"]))


def attention(query, key, content, allowed, cast):
    """GQA attention of ``megabench.tasks.common.attention`` (source not shipped).

    Restated from reference/pi05.py:184-188: K/V repeated over the query heads,
    scores and probabilities in the activation dtype, softmax in FP32, additive
    finite mask.
    """
    qh, kvh, d = query.shape[1], key.shape[1], query.shape[2]
    groups = qh // kvh
    q, k, c = (t.transpose(0, 1) for t in (query, key.repeat_interleave(groups, 1),
                                           content.repeat_interleave(groups, 1)))
    scores = (q @ k.transpose(-1, -2)) * d ** -0.5
    bias = torch.where(allowed, 0.0, MASK_VALUE)
    scores = scores + cast(bias)[None]
    return (cast(F.softmax(scores, -1, dtype=torch.float32)) @ c).transpose(0, 1)


def suffix_layout(mask: torch.Tensor, horizon: int):
    """reference/pi05.py:290-296."""
    positions = mask.sum() + torch.arange(horizon)
    allowed = torch.cat((mask[None, :].expand(horizon, -1),
                         torch.ones((horizon, horizon), dtype=torch.bool)), 1)
    return positions, allowed


def _w(v: dict, name: str, layer: int, widen: bool) -> torch.Tensor:
    t = v[name][layer]
    return t.float() if widen else t


def expert_attention(v, geo: Geo, layer, normalized, positions, allowed, widen):
    """reference/pi05.py:254-265."""
    cast = _cast(widen)
    tokens, d, qh, kvh = normalized.shape[0], geo.head_dim, geo.q_heads, geo.kv_heads
    query = rope((normalized @ _w(v, "wq", layer, widen).T).view(tokens, qh, d), positions, cast)
    key = rope((normalized @ _w(v, "wk", layer, widen).T).view(tokens, kvh, d), positions, cast)
    content = (normalized @ _w(v, "wv", layer, widen).T).view(tokens, kvh, d)
    key = torch.cat((cast(v["prefix_k"][layer]), key))
    content = torch.cat((cast(v["prefix_v"][layer]), content))
    mixed = attention(query, key, content, allowed, cast).reshape(tokens, qh * d)
    return mixed @ _w(v, "wo", layer, widen).T


def expert(v, geo: Geo, h, cond, positions, allowed, widen, layers=None):
    """reference/pi05.py:268-279."""
    cast = _cast(widen)
    for layer in range(geo.layers if layers is None else layers):
        normalized, gate = ada_rms(h, F.linear(cond, v["attn_norm_weight"][layer],
                                               v["attn_norm_bias"][layer]), cast)
        h = h + expert_attention(v, geo, layer, normalized, positions, allowed, widen) * gate
        normalized, gate = ada_rms(h, F.linear(cond, v["ffn_norm_weight"][layer],
                                               v["ffn_norm_bias"][layer]), cast)
        gated = F.gelu(normalized @ _w(v, "wg", layer, widen).T, approximate="tanh") \
            * (normalized @ _w(v, "wu", layer, widen).T)
        h = h + (gated @ _w(v, "wd", layer, widen).T) * gate
    return ada_rms(h, F.linear(cond, v["final_norm_weight"], v["final_norm_bias"]), cast)[0]


def velocity(v, geo: Geo, x, time, positions, allowed, widen, layers=None):
    """reference/pi05.py:282-287."""
    cast = _cast(widen)
    cond = time_condition(v, time, geo.hidden)
    h = cast(F.linear(x, v["action_in_weight"], v["action_in_bias"]))
    h = expert(v, geo, h, cond, positions, allowed, widen, layers)
    return F.linear(h.float(), v["action_out_weight"], v["action_out_bias"])


def chunk(v: dict, geo: Geo, widen: bool = False, steps=None, layers=None) -> torch.Tensor:
    """reference/pi05.py:299-309 (``widen=False``) or the FP32 oracle of
    reference/oracle.py:51-53 (``widen=True``).  ``steps``/``layers`` run only
    the first Euler steps / expert layers (dt stays -1/geo.steps), matching the
    engine's truncated debug runs."""
    with torch.no_grad():
        positions, allowed = suffix_layout(v["prefix_mask"], geo.horizon)
        dt = -1.0 / geo.steps
        x = v["noise"]
        for step in range(geo.steps if steps is None else steps):
            time = torch.full((1,), 1.0 + step * dt, dtype=torch.float32)
            x = x + dt * velocity(v, geo, x, time, positions, allowed, widen, layers)
        return x


# ------------------------------------------------------------------ grading (fixture.py:105-126)
def band(want: torch.Tensor, got: torch.Tensor, exact: torch.Tensor,
         atol: float = ATOL, rtol: float = RTOL, bf16_rtol: float = BF16_RTOL) -> dict:
    """fixture.py:105-120: error against the FP32 oracle within 2x the BF16
    reference's own error plus rtol, on relative L2 and on max-abs."""
    exact = exact.double()
    error, ref_error = got.double() - exact, want.double() - exact
    scale = exact.norm().clamp_min(torch.finfo(torch.float64).tiny)
    r = bf16_rtol if want.dtype == BF16 else rtol
    k = NOISE_FACTOR
    d = {"relative_error": float(error.norm() / scale),
         "reference_relative_error": float(ref_error.norm() / scale),
         "max_abs_error": float(error.abs().max()),
         "reference_max_abs_error": float(ref_error.abs().max())}
    d["pass"] = bool(torch.isfinite(got).all()) and bool(
        d["relative_error"] <= k * d["reference_relative_error"] + r and
        d["max_abs_error"] <= (k * d["reference_max_abs_error"] + atol
                               + r * float(exact.abs().max())))
    return d


def snapshot(inputs: dict) -> dict:
    """fixture.py:123-126: per-tensor (sum, abs-sum) fingerprints."""
    return {k: (v.float().sum().item(), v.float().abs().sum().item()) for k, v in inputs.items()}


def sol_bytes(geo: Geo, batch: int = 1) -> dict:
    """bench.py:63-80: bytes of the HBM floor with the expert re-streamed every step."""
    L, W, I, S, T = geo.layers, geo.hidden, geo.intermediate, geo.steps, geo.horizon
    qd, kvd = geo.q_heads * geo.head_dim, geo.kv_heads * geo.head_dim
    layer_params = W * (qd + 2 * kvd) + qd * W + 3 * W * I
    expert_b = L * layer_params * 2
    fp32_once = (L * 2 + 1) * 3 * W * W * 4 + 2 * W * W * 4 + 2 * W * geo.action_dim * 4
    kv = L * geo.prefix * kvd * 2 * 2
    keys = geo.prefix + T
    return {"expert_weight_bytes": expert_b, "fp32_cond_weight_bytes": fp32_once,
            "prefix_kv_bytes": kv,
            "bytes_restream": S * (expert_b + batch * kv) + fp32_once,
            "flops": batch * S * (2 * T * L * layer_params + L * 4 * T * qd * keys)}


# ------------------------------------------------------------------ stage-level reference
def rb(t: torch.Tensor) -> torch.Tensor:
    """Round FP32 to BF16 and widen back (one BF16 rounding point)."""
    return t.to(BF16).float()


def stages(v: dict, geo: Geo, step: int, layer: int, h_in: torch.Tensor) -> dict:
    """One layer pass in the engine's rounding schedule, every intermediate kept.

    ``h_in`` is the BF16 residual stream [T, W] entering the layer.  The schedule
    equals the reference's except inside attention: probabilities are rounded to
    BF16 before normalisation and divided by the FP32 row sum afterwards.  All
    values are returned as FP32 tensors holding BF16-representable numbers where
    the engine stores BF16.
    """
    with torch.no_grad():
        T, d, qh = geo.horizon, geo.head_dim, geo.q_heads
        positions, allowed = suffix_layout(v["prefix_mask"], T)
        dt = -1.0 / geo.steps
        time = torch.full((1,), 1.0 + step * dt, dtype=torch.float32)
        cond = time_condition(v, time, geo.hidden)
        out = {"cond": cond[0]}
        mod_a = F.linear(cond, v["attn_norm_weight"][layer], v["attn_norm_bias"][layer])[0]
        mod_f = F.linear(cond, v["ffn_norm_weight"][layer], v["ffn_norm_bias"][layer])[0]
        out["mod_attn"], out["mod_ffn"] = mod_a, mod_f
        h = h_in.float()

        def norm(hh, mod):
            n = hh * torch.rsqrt(hh.square().mean(-1, keepdim=True) + EPS)
            sc, sh, g = mod.chunk(3, -1)
            return rb(n * (1 + sc) + sh), rb(g)

        an, gate_a = norm(h, mod_a)
        out["an_attn"] = an
        q = rb(an @ v["wq"][layer].float().T).view(T, qh, d)
        k = rb(an @ v["wk"][layer].float().T).view(T, 1, d)
        vv = rb(an @ v["wv"][layer].float().T).view(T, 1, d)
        inv = 1.0 / (ROPE_THETA ** (torch.arange(0, d, 2, dtype=torch.int64).float() / d))
        phase = positions.float()[:, None] * inv[None, :]
        phase = torch.cat((phase, phase), -1)
        cos, sin = rb(phase.cos())[:, None], rb(phase.sin())[:, None]

        def rot(x):
            r = torch.cat((-x[..., d // 2:], x[..., :d // 2]), -1)
            return rb(rb(x * cos) + rb(r * sin))

        q, k = rot(q), rot(k)
        out["q"], out["k"], out["v"] = q.reshape(T, qh * d), k.reshape(T, d), vv.reshape(T, d)
        keys = torch.cat((v["prefix_k"][layer].float()[:, 0], k[:, 0]))
        vals = torch.cat((v["prefix_v"][layer].float()[:, 0], vv[:, 0]))
        s = rb(rb(torch.einsum("thd,kd->thk", q, keys)) * d ** -0.5)
        s = torch.where(allowed[:, None, :], s, torch.full_like(s, float("-inf")))
        m = s.max(-1, keepdim=True).values
        e = torch.exp(s - m)
        p = rb(e)
        o = torch.einsum("thk,kd->thd", p, vals) / e.sum(-1, keepdim=True)
        attn = rb(o).reshape(T, qh * d)
        out["attn"] = attn
        o_acc = attn @ v["wo"][layer].float().T
        out["o_acc"] = o_acc
        h = rb(h + rb(rb(o_acc) * gate_a))
        out["h_attn"] = h
        an, gate_f = norm(h, mod_f)
        out["an_ffn"] = an
        g = rb(an @ v["wg"][layer].float().T)
        u = rb(an @ v["wu"][layer].float().T)
        act = rb(rb(F.gelu(g, approximate="tanh")) * u)
        out["act"] = act
        d_acc = act @ v["wd"][layer].float().T
        out["d_acc"] = d_acc
        h = rb(h + rb(rb(d_acc) * gate_f))
        out["h_out"] = h
        return out


# ------------------------------------------------------------------------------------------- prefix prefill
def rms_gemma(x: torch.Tensor, weight: torch.Tensor, cast) -> torch.Tensor:
    """``megabench.tasks.common.rms(x, weight, gemma=True)`` (source not shipped with the reference; call sites
    reference/pi05.py:178, 192).  Restated as the Gemma RMSNorm the reference's docstrings name as upstream (HF
    ``GemmaRMSNorm``): normalise in FP32, scale by (1 + weight), cast to the activation dtype.  Parity unpinned for
    this one function: the stand-in that generated the golden vectors holds the same restatement."""
    xf = x.float()
    normalized = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + EPS)
    return cast(normalized * (1.0 + weight.float()))


def prefill(v: dict, embeddings: torch.Tensor, valid: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
            widen: bool = False, layers=None):
    """reference/pi05.py:167-195: Gemma-2B prefix-LM prefill, returns the post-RoPE keys and the values of every layer
    ([layers, tokens, kv_heads, head_dim]).  ``widen`` = every BF16 tensor and cast widened to FP32 (the oracle of
    reference/oracle.py).  Scores are formed in the activation dtype, the finite additive mask is FP32, so the sum that
    enters the FP32 softmax is FP32 (type promotion), as in the reference."""
    cast = _cast(widen)
    steps, d = embeddings.shape[0], head_dim
    w = (lambda name, layer: v[name][layer].float()) if widen else (lambda name, layer: v[name][layer])
    x = cast(embeddings)
    positions = torch.cumsum(valid.long(), 0) - 1
    bias = torch.where(valid[None, :] & valid[:, None], 0.0, MASK_VALUE)
    nlayers = v["lq"].shape[0] if layers is None else layers
    keys, contents = [], []
    for layer in range(nlayers):
        normalized = rms_gemma(x, v["ln1"][layer], cast)
        query = rope((normalized @ w("lq", layer).T).view(steps, q_heads, d), positions, cast)
        key = rope((normalized @ w("lk", layer).T).view(steps, kv_heads, d), positions, cast)
        content = (normalized @ w("lv", layer).T).view(steps, kv_heads, d)
        keys.append(key)
        contents.append(content)
        groups = q_heads // kv_heads
        q, k, c = (t.transpose(0, 1) for t in (query, key.repeat_interleave(groups, 1),
                                               content.repeat_interleave(groups, 1)))
        scores = (q @ k.transpose(-1, -2)) * d ** -0.5 + bias
        mixed = (cast(F.softmax(scores, -1, dtype=torch.float32)) @ c).transpose(0, 1)
        x = x + mixed.reshape(steps, q_heads * d) @ w("lo", layer).T
        if layer + 1 == nlayers:
            break                       # the last MLP does not affect any cached K/V
        normalized = rms_gemma(x, v["ln2"][layer], cast)
        gated = F.gelu(normalized @ w("lg", layer).T, approximate="tanh") * (normalized @ w("lu", layer).T)
        x = x + gated @ w("ld", layer).T
    return torch.stack(keys), torch.stack(contents)
