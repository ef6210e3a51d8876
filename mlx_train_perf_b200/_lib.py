"""ctypes binding of `libb200tp.so` (declared in include/b200tp.h).

The library is loaded lazily and exactly once; a missing or unloadable library raises
`NativeLibraryError` -- there is no Python or CPU fallback for the numeric operators.
"""
from __future__ import annotations

import ctypes as C
import threading
from pathlib import Path

from mlx_train_perf_b200.errors import (
    AttentionInputError, DeviceTimeoutError, LossInputError, NativeLibraryError,
    UnsupportedAttentionError, UnsupportedHeadError,
)

LIB_PATH = Path(__file__).resolve().parent / "libb200tp.so"

F32, BF16 = 0, 1
IMPL = {"auto": 0, "kernel": 0, "tc": 1, "simt": 2}

OK = 0
ERR_LOSS_INPUT, ERR_UNSUPPORTED_HEAD, ERR_ATTN_INPUT, ERR_UNSUPPORTED_ATTN = 1, 2, 3, 4
ERR_WORKSPACE, ERR_CUDA, ERR_NO_DEVICE = 5, 6, 7


class CeArgs(C.Structure):
    _fields_ = [
        ("hidden", C.c_void_p), ("weight", C.c_void_p), ("w_q", C.c_void_p),
        ("scales", C.c_void_p), ("biases", C.c_void_p), ("targets", C.c_void_p),
        ("n", C.c_int64), ("d", C.c_int32), ("v_local", C.c_int64), ("v_offset", C.c_int64),
        ("dtype", C.c_int32), ("quant_bits", C.c_int32), ("group_size", C.c_int32),
        ("qparam_dtype", C.c_int32), ("ignore_index", C.c_int64), ("impl", C.c_int32),
        ("reserved", C.c_int32),
    ]


class AttnArgs(C.Structure):
    _fields_ = [
        ("b", C.c_int32), ("hq", C.c_int32), ("hkv", C.c_int32), ("s", C.c_int32), ("d", C.c_int32),
        ("dtype", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("o_stride", C.c_int64 * 3),
        ("scale", C.c_float), ("causal", C.c_int32),
        ("seg_id", C.c_void_p), ("seg_start", C.c_void_p),
        ("impl", C.c_int32), ("reserved", C.c_int32),
    ]


class PrestepArgs(C.Structure):
    _fields_ = [
        ("b", C.c_int32), ("l", C.c_int32), ("h", C.c_int32), ("d", C.c_int32),
        ("dtype", C.c_int32),
        ("x_stride", C.c_int64 * 3), ("y_stride", C.c_int64 * 3),
        ("weight", C.c_void_p), ("eps", C.c_float),
        ("cos", C.c_void_p), ("sin", C.c_void_p),
        ("cs_dtype", C.c_int32), ("cs_stride_b", C.c_int64), ("cs_stride_l", C.c_int64),
    ]


# name -> (restype, argtypes); every symbol include/b200tp.h declares
SIGNATURES = {
    "b200tp_status_string": (C.c_char_p, [C.c_int]),
    "b200tp_last_error": (C.c_char_p, []),
    "b200tp_version": (C.c_int, []),
    "b200tp_linear_ce_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(CeArgs)]),
    "b200tp_linear_ce_fwd": (C.c_int, [C.POINTER(CeArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "b200tp_linear_ce_fwd_static": (C.c_int, [C.POINTER(CeArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                              C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200tp_linear_ce_combine": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_int64,
                                           C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200tp_linear_ce_reduce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p]),
    "b200tp_linear_ce_cotangent": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p,
                                             C.c_void_p]),
    "b200tp_linear_ce_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(CeArgs), C.c_int32]),
    "b200tp_linear_ce_bwd": (C.c_int, [C.POINTER(CeArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                       C.c_int32, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "b200tp_linear_ce_bwd_stage": (C.c_int, [C.POINTER(CeArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                             C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.c_void_p,
                                             C.c_size_t, C.c_void_p, C.c_void_p]),
    "b200tp_linear_ce_bwd_train": (C.c_int, [C.POINTER(CeArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32,
                                             C.c_int32, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p,
                                             C.c_void_p]),
    "b200tp_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200tp_qk_norm_rope_fwd": (C.c_int, [C.POINTER(PrestepArgs), C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200tp_qk_norm_rope_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(PrestepArgs)]),
    "b200tp_qk_norm_rope_bwd": (C.c_int, [C.POINTER(PrestepArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.c_void_p, C.c_size_t, C.c_void_p]),
    "b200tp_dequant_int4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int32, C.c_int64, C.c_int64,
                                      C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p]),
    "b200tp_flash_fwd": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p]),
    "b200tp_flash_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(AttnArgs)]),
    "b200tp_flash_fwd_ws": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p]),
    "b200tp_flash_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(AttnArgs)]),
    "b200tp_flash_bwd": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_size_t, C.c_void_p, C.c_void_p]),
}

_lock = threading.Lock()
_lib = None


def load() -> C.CDLL:
    """Return the loaded library, loading it on first use."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not LIB_PATH.exists():
            raise NativeLibraryError(
                f"{LIB_PATH} is missing: build it with `python -m mlx_train_perf_b200.build` "
                "(needs nvcc; there is no CPU fallback)")
        try:
            lib = C.CDLL(str(LIB_PATH))
        except OSError as e:  # pragma: no cover - depends on the host
            raise NativeLibraryError(f"cannot load {LIB_PATH}: {e}") from e
        for name, (res, args) in SIGNATURES.items():
            try:
                fn = getattr(lib, name)
            except AttributeError as e:
                raise NativeLibraryError(f"{LIB_PATH} does not export {name}") from e
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


_ERRORS = {
    ERR_LOSS_INPUT: LossInputError,
    ERR_UNSUPPORTED_HEAD: UnsupportedHeadError,
    ERR_ATTN_INPUT: AttentionInputError,
    ERR_UNSUPPORTED_ATTN: UnsupportedAttentionError,
    ERR_WORKSPACE: NativeLibraryError,
    ERR_CUDA: NativeLibraryError,
    ERR_NO_DEVICE: NativeLibraryError,
}


def check(rc: int) -> None:
    """Raise the typed error a non-zero host return code maps to."""
    if rc == OK:
        return
    lib = load()
    detail = (lib.b200tp_last_error() or b"").decode()
    name = (lib.b200tp_status_string(rc) or b"").decode()
    raise _ERRORS.get(rc, NativeLibraryError)(f"{name}: {detail}")


def raise_for_device_status(code: int) -> None:
    """Raise `DeviceTimeoutError` for a non-zero device status word (read after a sync)."""
    if code == 0:
        return
    name = (load().b200tp_status_string(code) or b"").decode()
    raise DeviceTimeoutError(f"kernel reported status {code}: {name}")
