"""The Gemma-2B prefix prefill as a callable: the step before the action chunk.

Same call as the reference's ``prefill(case, values, embeddings, valid)`` (reference/pi05.py:167-195) without the case
object: ``Pi05Prefill(geo, device)`` once, ``bind(values)`` with the nine BF16 weight tensors (kept by pointer, read in
place), then ``run(embeddings, valid) -> (keys, values)``, both ``[18, tokens, 1, 256]`` BF16 on the device - the tensors
``Pi05Arm.bind`` takes as ``prefix_k`` / ``prefix_v``, with ``valid`` as its ``prefix_mask``.  torch only supplies device
memory and the current stream; the work is done by ``libpi05_b200.so``.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from .fixture import PREFILL_WEIGHTS, PrefillGeometry, prefill_shapes


class Pi05Prefill:
    def __init__(self, geo: PrefillGeometry, device: str = "cuda") -> None:
        if (geo.layers, geo.hidden, geo.intermediate, geo.q_heads, geo.kv_heads, geo.head_dim) != (18, 2048, 16384, 8, 1, 256):
            raise ValueError("the prefill is specialised for Gemma-2B: 18 layers, width 2048 / 16384, 8 query heads over "
                             "1 KV head of 256")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the prefill has no CPU path")
        self.geo = geo
        self.lib = _lib.load()
        self.device = torch.device(device)
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.device = torch.device("cuda", index)
        handle = ctypes.c_void_p()
        self._check(self.lib.pi05_prefill_create(index, geo.tokens, ctypes.byref(handle)), None)
        self.handle = handle
        nbytes = ctypes.c_size_t()
        self._check(self.lib.pi05_prefill_workspace_bytes(handle, ctypes.byref(nbytes)))
        self.ws = torch.empty(nbytes.value, dtype=torch.uint8, device=self.device)
        self.weights: list[torch.Tensor] | None = None

    def _check(self, rc: int, handle="self") -> None:
        if rc != _lib.OK:
            h = self.handle if handle == "self" else handle
            detail = self.lib.pi05_prefill_last_error(h).decode() if h else ""
            raise _lib.EngineError(rc, self.lib.pi05_error_string(rc).decode() + (f" ({detail})" if detail else ""))

    def bind(self, values: dict) -> None:
        want = prefill_shapes(self.geo)
        tensors = []
        for name in PREFILL_WEIGHTS:
            t = values[name]
            shape, dtype = want[name]
            if tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise ValueError(f"{name}: expected {shape} {dtype}, got {tuple(t.shape)} {t.dtype}")
            if not t.is_contiguous() or t.device != self.device:
                raise ValueError(f"{name} must be contiguous and live on {self.device}")
            tensors.append(t)
        ptrs = (ctypes.c_void_p * _lib.PREFILL_NUM_WEIGHTS)(*[t.data_ptr() for t in tensors])
        self._check(self.lib.pi05_prefill_bind(self.handle, ptrs, self.ws.data_ptr(), self.ws.numel()))
        self.weights = tensors

    def run(self, embeddings: torch.Tensor, valid: torch.Tensor, layers: int | None = None,
            out: tuple[torch.Tensor, torch.Tensor] | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Asynchronous on the current stream.  ``embeddings`` [tokens, 2048] BF16, ``valid`` [tokens] bool."""
        tokens = embeddings.shape[0]
        if tuple(embeddings.shape) != (tokens, self.geo.hidden) or embeddings.dtype != torch.bfloat16 or \
                tuple(valid.shape) != (tokens,) or valid.dtype != torch.bool:
            raise ValueError("embeddings must be [tokens, 2048] bfloat16 and valid [tokens] bool")
        if not (embeddings.is_contiguous() and valid.is_contiguous()) or embeddings.device != self.device \
                or valid.device != self.device:
            raise ValueError(f"embeddings and valid must be contiguous and live on {self.device}")
        shape = (self.geo.layers, tokens, self.geo.kv_heads, self.geo.head_dim)
        k, v = out if out is not None else (torch.zeros(shape, dtype=torch.bfloat16, device=self.device),
                                            torch.zeros(shape, dtype=torch.bfloat16, device=self.device))
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self._check(self.lib.pi05_prefill_run(self.handle, embeddings.data_ptr(), valid.data_ptr(), tokens, k.data_ptr(),
                                              v.data_ptr(), self.geo.layers if layers is None else layers, stream))
        return k, v

    def status(self) -> None:
        """Synchronise the current stream; raises when a bounded device-side wait gave up."""
        code, where = ctypes.c_int(), ctypes.c_int()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        rc = self.lib.pi05_prefill_status(self.handle, stream, ctypes.byref(code), ctypes.byref(where))
        if rc == _lib.ERR_DEVICE_TIMEOUT:
            raise _lib.EngineError(rc, f"device wait kind {code.value} gave up in block {where.value}")
        self._check(rc)

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.pi05_prefill_destroy(self.handle)
            self.handle = None
        self.weights = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass
