"""ctypes binding of ``lib/libfmms_b200.so`` (the C ABI declared in include/fmms_b200.h).

Loading fails loudly when the shared object is absent: there is no CPU or
PyTorch fallback for the sampling path.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_size_t, c_ulonglong, c_void_p
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libfmms_b200.so"

# status codes / flags (include/fmms_b200.h)
OK, ERR_TIMEOUT, ERR_BAD_ARG, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA, ERR_ARCH, ERR_TOO_LARGE = range(8)
ERR_TOPK_OVERFLOW = 8
FLAG_GREEDY, FLAG_EXT_NOISE, FLAG_RETURN_LOGITS, FLAG_FORCE_GEMV, FLAG_FORCE_MMA, FLAG_TWO_STAGE = 1, 2, 4, 8, 16, 32
FLAG_SEED_DEVICE = 64
FLAG_LOGPROB = 128
FLAG_HOST_IO = 256
FLAG_NO_SYNC = 512
FLAG_W_FP8 = 2048
PATH_NONE, PATH_GEMV, PATH_MMA = 0, 1, 2

class FmmsCall(ctypes.Structure):
    """``fmms_call_t`` of include/fmms_b200.h, field for field."""

    _fields_ = [
        ("struct_bytes", c_size_t),
        ("W_bf16", c_void_p),
        ("H_bf16", c_void_p),
        ("temperature", c_void_p),
        ("temp_stride", c_int),
        ("V_local", c_int),
        ("D", c_int),
        ("B", c_int),
        ("S", c_int),
        ("seed", c_ulonglong),
        ("v_global_offset", c_longlong),
        ("flags", c_int),
        ("ext_noise", c_void_p),
        ("noise_ld", c_longlong),
        ("logits_out", c_void_p),
        ("out_idx", c_void_p),
        ("out_val", c_void_p),
        ("out_logprob", c_void_p),
        ("out_lse", c_void_p),
        ("workspace", c_void_p),
        ("workspace_bytes", c_size_t),
        ("status_dev", c_void_p),
        ("stream", c_void_p),
        ("tp_rank", c_int),
        ("tp_world", c_int),
        ("tp_max_items", c_int),
        ("tp_peer_buffers", ctypes.POINTER(c_void_p)),
        ("tp_epoch", ctypes.c_uint),
        ("tp_wait_limit_ns", c_ulonglong),
        ("staging", c_void_p),
        ("staging_bytes", c_size_t),
        ("status_host", c_void_p),
        ("top_k", c_int),
        ("top_p", c_float),
        ("topk_workspace", c_void_p),
        ("topk_workspace_bytes", c_size_t),
        ("w_scale", c_void_p),
    ]


# every symbol the header declares: name -> (restype, argtypes)
SIGNATURES = {
    "fmms_version": (c_int, []),
    "fmms_strerror": (c_char_p, [c_int]),
    "fmms_num_sms": (c_int, [ctypes.POINTER(c_int)]),
    "fmms_query_workspace": (c_int, [c_int, c_int, c_int, c_int, ctypes.POINTER(c_size_t)]),
    "fmms_sample": (
        c_int,
        [
            c_void_p,  # W
            c_void_p,  # H
            c_void_p,  # temperature
            c_int,  # temp_stride
            c_int,  # V_local
            c_int,  # D
            c_int,  # B
            c_int,  # S
            c_ulonglong,  # seed
            c_longlong,  # v_global_offset
            c_int,  # flags
            c_void_p,  # ext_noise
            c_longlong,  # noise_ld
            c_void_p,  # logits_out
            c_void_p,  # out_idx
            c_void_p,  # out_val
            c_void_p,  # workspace
            c_size_t,  # workspace_bytes
            c_void_p,  # status_dev
            c_void_p,  # stream
        ],
    ),
    "fmms_sample_tp": (
        c_int,
        [
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_ulonglong, c_longlong, c_int,
            c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p,
            c_int, c_int, c_int, ctypes.POINTER(c_void_p), ctypes.c_uint, c_ulonglong,
        ],
    ),
    "fmms_sample_logprobs": (
        c_int,
        [
            c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_ulonglong, c_longlong, c_int,
            c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_size_t, c_void_p, c_void_p,
            c_void_p, c_void_p,  # out_logprob, out_lse
        ],
    ),
    "fmms_run": (c_int, [ctypes.POINTER(FmmsCall)]),
    "fmms_query_staging": (c_int, [c_int, c_int, c_int, ctypes.POINTER(c_size_t)]),
    "fmms_query_topk_workspace": (c_int, [c_int, c_int, ctypes.POINTER(c_size_t), ctypes.POINTER(c_size_t)]),
    "fmms_last_path": (c_int, []),
    "fmms_l2_sweep": (c_int, [c_void_p, c_size_t, c_void_p]),
    "fmms_debug_stamps": (c_int, [c_void_p]),
    "fmms_plan": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int, ctypes.POINTER(c_int)]),
    "fmms_tp_buffer_bytes": (c_int, [c_int, c_int, ctypes.POINTER(c_size_t)]),
    "fmms_tp_alloc": (c_int, [c_size_t, ctypes.POINTER(c_void_p), c_void_p]),
    "fmms_tp_open": (c_int, [c_void_p, ctypes.POINTER(c_void_p)]),
    "fmms_tp_close": (c_int, [c_void_p]),
    "fmms_tp_free": (c_int, [c_void_p]),
    "fmms_tp_exchange": (
        c_int,
        [c_void_p, c_void_p, c_int, c_int, c_int, c_int, ctypes.POINTER(c_void_p), ctypes.c_uint,
         c_ulonglong, c_void_p, c_void_p, c_void_p, c_void_p],
    ),
    "fmms_static_max_items": (c_int, []),
    "fmms_static_reset": (c_int, [c_void_p]),
    "fmms_sample_static": (
        c_int,
        [
            c_void_p, c_void_p, c_void_p, c_int,  # W, H, temperature, temp_stride
            c_int, c_int, c_int, c_int,  # V_local, D, B, S
            c_ulonglong, c_longlong, c_int,  # seed, v_global_offset, flags
            c_void_p, c_longlong,  # ext_noise, noise_ld
            c_void_p, c_void_p, c_void_p,  # logits_out, out_idx, out_val
            c_void_p, c_void_p,  # status_dev, stream
        ],
    ),
}

_lib = None


class FmmsError(RuntimeError):
    def __init__(self, status: int, where: str):
        self.status = status
        super().__init__(f"{where}: {strerror(status)} (status {status})")


def load() -> ctypes.CDLL:
    """Load the CUDA library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m flashsampling_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def strerror(status: int) -> str:
    return load().fmms_strerror(int(status)).decode()


def check(status: int, where: str) -> None:
    if status != OK:
        raise FmmsError(status, where)


def query_workspace(v_local: int, d: int, b: int, s: int) -> int:
    n = c_size_t(0)
    check(load().fmms_query_workspace(v_local, d, b, s, ctypes.byref(n)), "fmms_query_workspace")
    return int(n.value)


def query_topk_workspace(v_local: int, b: int) -> tuple[int, int]:
    """(bytes with room for the exact second pass, bytes without it)."""
    full, small = c_size_t(0), c_size_t(0)
    check(load().fmms_query_topk_workspace(v_local, b, ctypes.byref(full), ctypes.byref(small)),
          "fmms_query_topk_workspace")
    return int(full.value), int(small.value)


def query_staging(d: int, b: int, s: int) -> int:
    n = c_size_t(0)
    check(load().fmms_query_staging(d, b, s, ctypes.byref(n)), "fmms_query_staging")
    return int(n.value)


PLAN_FIELDS = ("path", "grid", "tile_rows", "tiles_per_cta", "stages", "m_tiles", "smem_bytes", "candidate_rows")


def plan(v_local: int, d: int, b: int, s: int, flags: int = 0, num_sms: int = 148, max_smem: int = 232448) -> dict:
    """Host-side launch plan (no GPU needed); see fmms_plan in the header."""
    arr = (c_int * 8)()
    check(load().fmms_plan(v_local, d, b, s, flags, num_sms, max_smem, arr), "fmms_plan")
    return dict(zip(PLAN_FIELDS, list(arr)))
