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
TP_HANDLE_BYTES = 96
PREFILL_NUM_WEIGHTS = 9

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


class Tuning(ctypes.Structure):
    """``pi05_tuning`` of the header: run-time tuning settings of a handle."""
    _fields_ = [(name, _c.c_int) for name in (
        "poll_ns", "obs_per_mma", "two_streams", "entries_per_phase", "grouped_from", "streams_from",
        "latency_schedule", "key_groups", "row_groups", "clusters", "cta_perm")]


# Development aid of this host layer (the library itself reads no environment variable): PI05_* variables that
# override single tuning settings, so that two runs of the same command are an A/B pair.
ENV_TUNING = {"PI05_POLL_NS": ("poll_ns", int), "PI05_OBS_PER_MMA": ("obs_per_mma", int),
              "PI05_ONE_STREAM": ("two_streams", lambda v: 0), "PI05_ENTRIES_PER_PHASE": ("entries_per_phase", int),
              "PI05_GROUPED_FROM": ("grouped_from", int), "PI05_STREAMS_FROM": ("streams_from", int),
              "PI05_LATENCY_SCHEDULE": ("latency_schedule", lambda v: 1), "PI05_KEY_GROUPS": ("key_groups", int),
              "PI05_ROW_GROUPS": ("row_groups", int), "PI05_NO_CLUSTER": ("clusters", lambda v: 0),
              "PI05_CTA_PERM": ("cta_perm", int)}


def tuning_from_env(lib=None) -> "Tuning":
    """The library's default settings with the PI05_* overrides of the environment applied."""
    lib = lib or load()
    t = Tuning()
    rc = lib.pi05_tuning_defaults(_c.byref(t))
    if rc != OK:
        raise EngineError(rc, lib.pi05_error_string(rc).decode())
    for var, (field, conv) in ENV_TUNING.items():
        if var in os.environ:
            setattr(t, field, int(conv(os.environ[var])))
    return t


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
    "pi05_schedule_plan": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.POINTER(Tuning), _c.POINTER(_c.c_int), _c.c_int,
                                      _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "pi05_schedule_plan_tp": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.c_int, _c.POINTER(Tuning),
                                         _c.POINTER(_c.c_int), _c.c_int, _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "pi05_tp_export": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t]),
    "pi05_tp_attach": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p]),
    "pi05_tp_attach_pointer": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_void_p]),
    "pi05_prefill_create": (_c.c_int, [_c.c_int, _c.c_int, _c.POINTER(_c.c_void_p)]),
    "pi05_prefill_workspace_bytes": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_size_t)]),
    "pi05_prefill_bind": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_void_p), _c.c_void_p, _c.c_size_t]),
    "pi05_prefill_run": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_int,
                                    _c.c_void_p]),
    "pi05_prefill_status": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "pi05_prefill_plan": (_c.c_int, [_c.c_int, _c.c_int, _c.c_int, _c.POINTER(_c.c_int), _c.POINTER(_c.c_int), _c.c_int,
                                     _c.POINTER(_c.c_int)]),
    "pi05_prefill_last_error": (_c.c_char_p, [_c.c_void_p]),
    "pi05_prefill_destroy": (_c.c_int, [_c.c_void_p]),
    "pi05_tuning_defaults": (_c.c_int, [_c.POINTER(Tuning)]),
    "pi05_tune": (_c.c_int, [_c.c_void_p, _c.POINTER(Tuning)]),
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


def schedule_plan(sms: int, batch: int, prefix: int, tp_rank: int = 0, tp_size: int = 1) -> tuple[list[tuple[int, ...]], dict]:
    """The work schedule the engine would bind on a GPU of ``sms`` SMs (host arithmetic only, no GPU needed):
    entries ``(cta, gemm, lag, group, tile, k0, nk)`` in execution order per CTA, and the plan's summary; for rank
    ``tp_rank`` of ``tp_size`` when the observation is shared by several GPUs."""
    lib = load()
    tuning = tuning_from_env(lib)
    count, info = _c.c_int(), (_c.c_int * PLAN_INFO)()
    rc = lib.pi05_schedule_plan_tp(sms, batch, prefix, tp_rank, tp_size, _c.byref(tuning), None, 0, _c.byref(count), info)
    if rc != OK:
        raise EngineError(rc, lib.pi05_error_string(rc).decode())
    buf = (_c.c_int * (count.value * PLAN_ENTRY))()
    rc = lib.pi05_schedule_plan_tp(sms, batch, prefix, tp_rank, tp_size, _c.byref(tuning), buf, count.value,
                                   _c.byref(count), info)
    if rc != OK:
        raise EngineError(rc, lib.pi05_error_string(rc).decode())
    entries = [tuple(buf[i * PLAN_ENTRY:(i + 1) * PLAN_ENTRY]) for i in range(count.value)]
    names = ("gemm_ctas", "row_groups", "key_groups", "obs_per_mma", "groups", "stream_split")
    summary = dict(zip(names, info[:6]))
    summary["units"] = dict(zip(("qkv", "o", "gate_up", "down"), info[6:10]))
    return entries, summary
