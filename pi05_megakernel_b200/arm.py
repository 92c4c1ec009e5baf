"""The engine as a benchmark arm: the reference harness's arm protocol over the C ABI.

Same surface as the reference's ``MegakernelArm`` (megakernel.py:117-186) as the
harness uses it (bench.py:123-135, 209-216, 234-252): ``Arm(geo, variant,
device)``, ``bind(inputs)``, ``launch()`` (asynchronous on the current stream,
one whole chunk), ``outputs()["actions"]`` (a persistent [50, 32] FP32 buffer
the arm owns; [batch, 50, 32] when the arm was created with ``batch`` > 1, in which
case noise, prefix_k, prefix_v and prefix_mask carry a leading batch index), optional ``refresh_weights()``, ``config`` and ``close()``.
torch only supplies device memory and the current stream; the work is done by
``libpi05_b200.so``.
"""

from __future__ import annotations

import ctypes
import json

import torch

from . import _lib
from .fixture import OBSERVATION, ORDER, Geometry, shapes


def parse_variant(variant: str) -> dict:
    """``b200`` or ``b200-s<steps>-l<layers>``: the optional suffixes truncate the
    Euler steps / expert layers (debug runs; the graded chunk is the plain name)."""
    name, *suffixes = variant.split("-")
    if name != "b200":
        raise ValueError(f"bad variant {variant!r}: expected b200[-s<steps>][-l<layers>]")
    out = {"steps": None, "layers": None}
    for suffix in suffixes:
        if len(suffix) > 1 and suffix[0] == "s" and suffix[1:].isdigit() and out["steps"] is None:
            out["steps"] = int(suffix[1:])
        elif len(suffix) > 1 and suffix[0] == "l" and suffix[1:].isdigit() and out["layers"] is None:
            out["layers"] = int(suffix[1:])
        else:
            raise ValueError(f"bad variant suffix {suffix!r} in {variant!r}")
    return out


class PagedPrefix:
    """The prefix cache in the layout of whoever produced it.

    ``k`` and ``v`` are BF16 CUDA tensors ``[pages, layers, page_tokens, kv_heads(1), 256]`` with any strides whose
    last dimension is contiguous (a slice of a larger cache, a pool with padding between tokens, ...); ``table`` is an
    integer array ``[batch][pages_per_observation]`` (list or CPU tensor) naming, in order, the pages that hold each
    observation's tokens.  With more than one page per observation ``page_tokens`` must be a multiple of 64.
    """

    def __init__(self, k: torch.Tensor, v: torch.Tensor, table) -> None:
        if k.dim() != 5 or k.shape != v.shape or k.shape[3] != 1 or k.shape[4] != 256:
            raise ValueError("k and v must be [pages, layers, page_tokens, 1, 256]")
        if k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
            raise ValueError("k and v must be bfloat16")
        if k.stride() != v.stride() or k.stride(4) != 1:
            raise ValueError("k and v must share their strides and have a contiguous last dimension")
        self.k, self.v = k, v
        self.table = [[int(x) for x in row] for row in (table.tolist() if hasattr(table, "tolist") else table)]

    def as_view(self, arm: "Pi05Arm"):
        if self.k.device != arm.device or self.v.device != arm.device:
            raise ValueError(f"the prefix cache must live on {arm.device}")
        if len(self.table) != arm.batch or len({len(r) for r in self.table}) != 1:
            raise ValueError("the page table needs one row of equal length per observation")
        if self.k.shape[1] != arm.geo.layers:
            raise ValueError("wrong number of layers in the prefix cache")
        flat = [x for row in self.table for x in row]
        table = (ctypes.c_int * len(flat))(*flat)
        view = _lib.KvView(self.k.data_ptr(), self.v.data_ptr(), self.k.stride(2), self.k.stride(1), self.k.stride(0),
                           self.k.shape[2], self.k.shape[0], len(self.table[0]), table)
        return view, table


class Pi05Arm:
    name = "b200-megakernel"

    def __init__(self, geo: Geometry, variant: str = "b200", device: str = "cuda", batch: int = 1,
                 tp: tuple[int, int] = (0, 1)) -> None:
        """``tp = (rank, size)``: this arm is one of ``size`` arms, one per GPU, that compute the same observation
        together (tensor parallel; see ``tp_export`` / ``tp_attach``)."""
        if (geo.horizon, geo.action_dim, geo.layers, geo.steps, geo.hidden, geo.intermediate,
                geo.q_heads, geo.kv_heads, geo.head_dim) != (50, 32, 18, 10, 1024, 4096, 8, 1, 256):
            raise ValueError("the engine is specialised for horizon 50, action 32, 18 layers, 10 steps, "
                             "width 1024/4096, 8 query heads over 1 KV head of 256")
        pv = parse_variant(variant)
        if not 1 <= batch <= 16:
            raise ValueError("batch must be 1..16 observations per launch")
        self.geo, self.variant, self.batch = geo, variant, batch
        self.steps = geo.steps if pv["steps"] is None else pv["steps"]
        self.layers = geo.layers if pv["layers"] is None else pv["layers"]
        if not (1 <= self.steps <= geo.steps and 1 <= self.layers <= geo.layers):
            raise ValueError(f"variant {variant!r} asks for more steps or layers than the geometry has")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: the engine has no CPU path")
        self.lib = _lib.load()
        self.device = torch.device(device)
        index = self.device.index if self.device.index is not None else torch.cuda.current_device()
        self.device = torch.device("cuda", index)
        handle = ctypes.c_void_p()
        self.tp_rank, self.tp_size = tp
        _lib.check(self.lib, None, self.lib.pi05_create(index, geo.prefix, batch, self.tp_rank, self.tp_size,
                                                        ctypes.byref(handle)))
        self.handle = handle
        self.tuning = _lib.tuning_from_env(self.lib)         # defaults, or the PI05_* overrides of a development run
        _lib.check(self.lib, handle, self.lib.pi05_tune(handle, ctypes.byref(self.tuning)))
        nbytes = ctypes.c_size_t()
        _lib.check(self.lib, handle, self.lib.pi05_workspace_bytes(handle, ctypes.byref(nbytes)))
        self.ws = torch.empty(nbytes.value, dtype=torch.uint8, device=self.device)
        shape = (geo.horizon, geo.action_dim) if batch == 1 else (batch, geo.horizon, geo.action_dim)
        self.actions = torch.zeros(shape, dtype=torch.float32, device=self.device)
        self.tensors: list[torch.Tensor] | None = None
        self.stamps: torch.Tensor | None = None
        self.config = json.loads(self.lib.pi05_config_json(handle).decode())
        self.config.update(prefix=geo.prefix, steps=self.steps, layers=self.layers, batch=batch)

    # ------------------------------------------------------------------ arm protocol
    def bind(self, inputs: dict, kv_pages: "PagedPrefix | None" = None) -> None:
        """Record the 25 tensors (kept by pointer, read in place).  With ``kv_pages`` the prefix keys / values are read
        where their producer left them (a strided or paged pool, see ``PagedPrefix``) and ``inputs["prefix_k"]`` /
        ``inputs["prefix_v"]`` are not needed."""
        want = shapes(self.geo)
        tensors = []
        for name in ORDER:
            if kv_pages is not None and name in ("prefix_k", "prefix_v"):
                tensors.append(None)
                continue
            value = inputs[name]
            shape, dtype = want[name]
            if self.batch > 1 and name in OBSERVATION:
                shape = (self.batch, *shape)          # one observation per leading index, weights shared
            if tuple(value.shape) != tuple(shape) or value.dtype != dtype:
                raise ValueError(f"{name}: expected {shape} {dtype}, got {tuple(value.shape)} {value.dtype}")
            if not value.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
            if value.device != self.device:
                raise ValueError(f"{name} must live on {self.device}")
            tensors.append(value)
        ptrs = (ctypes.c_void_p * _lib.NUM_INPUTS)(*[None if t is None else t.data_ptr() for t in tensors])
        if kv_pages is None:
            _lib.check(self.lib, self.handle, self.lib.pi05_bind(
                self.handle, ptrs, self.geo.prefix, self.batch, self.actions.data_ptr(), self.ws.data_ptr(),
                self.ws.numel()))
        else:
            view, keep = kv_pages.as_view(self)
            _lib.check(self.lib, self.handle, self.lib.pi05_bind_view(
                self.handle, ptrs, ctypes.byref(view), self.geo.prefix, self.batch, self.actions.data_ptr(),
                self.ws.data_ptr(), self.ws.numel()))
            tensors += [kv_pages.k, kv_pages.v]
            del keep
        self.tensors = tensors
        # the engine chooses its schedule when it knows the batch: record what it chose
        self.config.update(json.loads(self.lib.pi05_config_json(self.handle).decode()))

    # ------------------------------------------------------------------ tensor parallel
    def tp_export(self) -> bytes:
        """After ``bind``: what the other ranks need to reach this arm's receive buffers (send it to them by any means)."""
        buf = ctypes.create_string_buffer(_lib.TP_HANDLE_BYTES)
        _lib.check(self.lib, self.handle, self.lib.pi05_tp_export(self.handle, buf, _lib.TP_HANDLE_BYTES))
        return buf.raw

    def tp_attach(self, peer_rank: int, exported: bytes) -> None:
        """Open rank ``peer_rank``'s receive buffers (its ``tp_export()``); needed for every peer before ``launch``."""
        buf = ctypes.create_string_buffer(exported, _lib.TP_HANDLE_BYTES)
        _lib.check(self.lib, self.handle, self.lib.pi05_tp_attach(self.handle, peer_rank, buf))

    def tp_attach_all(self, group=None) -> None:
        """The usual set-up under ``torch.distributed`` (one process per GPU): all-gather the exports, attach every peer,
        and line the ranks up so that nobody launches before everybody has attached."""
        import torch.distributed as dist
        blobs = [None] * self.tp_size
        dist.all_gather_object(blobs, self.tp_export(), group=group)
        for r, blob in enumerate(blobs):
            if r != self.tp_rank:
                self.tp_attach(r, blob)
        dist.barrier(group=group)

    def refresh_weights(self) -> None:
        _lib.check(self.lib, self.handle, self.lib.pi05_refresh(self.handle))

    def launch(self) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        stamps = self.stamps.data_ptr() if self.stamps is not None else None
        _lib.check(self.lib, self.handle, self.lib.pi05_launch(self.handle, self.steps, self.layers, stream, stamps))

    def outputs(self) -> dict:
        return {"actions": self.actions}

    def close(self) -> None:
        if getattr(self, "handle", None):
            self.lib.pi05_destroy(self.handle)
            self.handle = None
        self.tensors = None

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.close()
        except Exception:
            pass

    # ------------------------------------------------------------------ diagnostics
    def status(self) -> tuple[int, int]:
        """Synchronise and return (code, where) of the device status word; raises on a device timeout."""
        code, where = ctypes.c_int(), ctypes.c_int()
        rc = self.lib.pi05_status(self.handle, ctypes.byref(code), ctypes.byref(where))
        if rc == _lib.ERR_DEVICE_TIMEOUT:
            raise _lib.EngineError(rc, f"device wait kind {code.value} gave up at cta {where.value >> 16}, "
                                       f"stage {where.value & 0xffff}")
        _lib.check(self.lib, self.handle, rc)
        return code.value, where.value

    def debug(self, max_stage: int = -1, wait_limit_cycles: int = 0, drop_event: int = -1) -> None:
        _lib.check(self.lib, self.handle,
                   self.lib.pi05_debug(self.handle, max_stage, wait_limit_cycles, drop_event))

    def enable_stamps(self, on: bool = True) -> None:
        self.stamps = torch.zeros(_lib.NUM_STAMPS, dtype=torch.int64, device=self.device) if on else None

    def region(self, name: str, dtype: torch.dtype, shape: tuple) -> torch.Tensor:
        """A view of a named workspace buffer (stage-by-stage checks)."""
        off, nbytes = ctypes.c_size_t(), ctypes.c_size_t()
        _lib.check(self.lib, self.handle, self.lib.pi05_workspace_region(
            self.handle, name.encode(), ctypes.byref(off), ctypes.byref(nbytes)))
        return self.ws[off.value:off.value + nbytes.value].view(dtype).view(shape)

    def launch_count(self) -> int:
        n = ctypes.c_ulonglong()
        _lib.check(self.lib, self.handle, self.lib.pi05_launch_count(self.handle, ctypes.byref(n)))
        return n.value
