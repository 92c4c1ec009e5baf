"""ctypes binding of the C ABI declared in ``include/pi05_b200.h``.

There is no fallback: if the shared library is missing or a symbol is absent,
loading raises.
"""

from __future__ import annotations

import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("PI05_B200_LIB") or os.path.join(HERE, "libpi05_b200.so")   # the variable: another build of the same library
NUM_INPUTS = 25
NUM_STAMPS = 256
STATIC_SCRATCH_BYTES = 12 << 20
STATIC_MAX_PREFIX = 1024
PLAN_ENTRY, PLAN_INFO = 7, 10

EVENT_ATTENTION_DONE, EVENT_FFN_NORM_READY = 7, 9
WAIT_EVENT = 7
OK, ERR_ARGUMENT, ERR_UNSUPPORTED, ERR_CUDA, ERR_NOT_BOUND, ERR_DEVICE_TIMEOUT, ERR_NO_DEVICE = range(7)

_c = ctypes


class KvView(ctypes.Structure):
    """``pi05_kv_view`` of the header: the prefix cache as a pool of pages with strides (in BF16 elements)."""
    _fields_ = [("k", _c.c_void_p), ("v", _c.c_void_p),
                ("token_stride", _c.c_longlong), ("layer_stride", _c.c_longlong), ("page_stride", _c.c_longlong),
                ("page_tokens", _c.c_int), ("num_pages", _c.c_int), ("pages_per_obs", _c.c_int),
                ("page_table", _c.POINTER(_c.c_int))]


SIGNATURES = {
    "pi05_create": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_void_p)]),
    "pi05_workspace_bytes": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_size_t)]),
    "pi05_bind": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_void_p), _c.c_int, _c.c_int, _c.c_void_p,
                             _c.c_void_p, _c.c_size_t]),
    "pi05_bind_view": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_void_p), _c.POINTER(KvView), _c.c_int, _c.c_int,
                                  _c.c_void_p, _c.c_void_p, _c.c_size_t]),
    "pi05_refresh": (_c.c_int, [_c.c_void_p]),
    "pi05_launch": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "pi05_status": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "pi05_workspace_region": (_c.c_int, [_c.c_void_p, _c.c_char_p, _c.POINTER(_c.c_size_t),
                                         _c.POINTER(_c.c_size_t)]),
    "pi05_debug": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_longlong, _c.c_int]),
    "pi05_config_json": (_c.c_char_p, [_c.c_void_p]),
    "pi05_launch_count": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_ulonglong)]),
    "pi05_error_string": (_c.c_char_p, [_c.c_int]),
    "pi05_last_error": (_c.c_char_p, [_c.c_void_p]),
    "pi05_destroy": (_c.c_int, [_c.c_void_p]),
    "pi05_schedule_plan": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_int), _c.c_int,
                                      _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "pi05_chunk_static": (_c.c_int, [_c.c_int, _c.POINTER(_c.c_void_p), _c.c_int, _c.c_void_p, _c.c_int, _c.c_int,
                                     _c.c_void_p]),
}

_lib = None


class EngineError(RuntimeError):
    def __init__(self, code: int, message: str) -> None:
        super().__init__(f"pi05 engine error {code}: {message}")
        self.code = code


def load() -> ctypes.CDLL:
    """Load the native library (once) and declare every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is missing: build it with `python -m pi05_megakernel_b200.build` "
                          "(there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)       # AttributeError if the library does not export it
        fn.restype, fn.argtypes = restype, argtypes
    _lib = lib
    return lib


def check(lib, handle, rc: int) -> None:
    if rc != OK:
        detail = lib.pi05_last_error(handle).decode() if handle else ""
        raise EngineError(rc, lib.pi05_error_string(rc).decode() + (f" ({detail})" if detail else ""))


def schedule_plan(sms: int, batch: int, prefix: int) -> tuple[list[tuple[int, ...]], dict]:
    """The work schedule the engine would bind on a GPU of ``sms`` SMs (host arithmetic only, no GPU needed):
    entries ``(cta, gemm, lag, group, tile, k0, nk)`` in execution order per CTA, and the plan's summary."""
    lib = load()
    count, info = _c.c_int(), (_c.c_int * PLAN_INFO)()
    rc = lib.pi05_schedule_plan(sms, batch, prefix, None, 0, _c.byref(count), info)
    if rc != OK:
        raise EngineError(rc, lib.pi05_error_string(rc).decode())
    buf = (_c.c_int * (count.value * PLAN_ENTRY))()
    rc = lib.pi05_schedule_plan(sms, batch, prefix, buf, count.value, _c.byref(count), info)
    if rc != OK:
        raise EngineError(rc, lib.pi05_error_string(rc).decode())
    entries = [tuple(buf[i * PLAN_ENTRY:(i + 1) * PLAN_ENTRY]) for i in range(count.value)]
    names = ("gemm_ctas", "row_groups", "key_groups", "obs_per_mma", "groups", "stream_split")
    summary = dict(zip(names, info[:6]))
    summary["units"] = dict(zip(("qkv", "o", "gate_up", "down"), info[6:10]))
    return entries, summary
