"""ctypes binding of libkd_attention.so (declarations: include/kd_attention.h).

The library is the only compute path of this package: if it cannot be loaded the import of
the operator fails with an error that says how to build it. There is no fallback.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import (POINTER, Structure, c_char_p, c_float, c_int32, c_int64, c_size_t, c_uint8,
                    c_void_p)
from pathlib import Path

KD_F16, KD_BF16, KD_F32 = 0, 1, 2
KD_TILE = 128
KD_TILE_EMPTY, KD_TILE_FULL, KD_TILE_PARTIAL = 0, 1, 2
KD_STATUS_TIMEOUT = 0x10000000
KD_STATUS_SPAN_RANGE = 0x20000000
KD_BWD_SPLIT, KD_BWD_FUSED = 0, 1

# KD_LIB_PATH selects another build of the same library (the wait time-out test loads one built with a short wait limit)
LIB_PATH = Path(os.environ.get("KD_LIB_PATH") or Path(__file__).resolve().parent / "_lib" / "libkd_attention.so")

EXPORTS = (
    "kd_version", "kd_last_error", "kd_plan_layout_get", "kd_classify", "kd_mask_dense",
    "kd_attn_fwd", "kd_attn_bwd", "kd_attn_bwd_static", "kd_workspace_bytes", "kd_workspace_bytes_fused", "kd_hadamard",
    "kd_metadata_from_tokens", "kd_span_index", "kd_span_mean",
)


class KdMeta(Structure):
    _fields_ = [
        ("B", c_int32), ("T", c_int32),
        ("in_span", c_void_p), ("span_id", c_void_p), ("is_prefix", c_void_p), ("lens", c_void_p),
        ("in_span_stride_b", c_int64), ("span_id_stride_b", c_int64), ("is_prefix_stride_b", c_int64),
        ("causal", c_int32), ("rules", c_int32),
    ]


class KdPlanLayout(Structure):
    _fields_ = [
        ("B", c_int32), ("T", c_int32), ("NT", c_int32), ("NP", c_int32),
        ("off_desc", c_size_t), ("off_summary", c_size_t), ("off_cls", c_size_t),
        ("off_fwd_cnt", c_size_t), ("off_fwd_list", c_size_t), ("off_bwd_cnt", c_size_t),
        ("off_bwd_list", c_size_t), ("off_tilebits", c_size_t), ("off_order", c_size_t), ("off_stats", c_size_t), ("off_status", c_size_t),
        ("total", c_size_t),
    ]


class KdTensor(Structure):
    _fields_ = [("ptr", c_void_p), ("stride_b", c_int64), ("stride_h", c_int64), ("stride_t", c_int64)]


class KdAttnParams(Structure):
    _fields_ = [
        ("B", c_int32), ("H", c_int32), ("T", c_int32), ("D", c_int32),
        ("dtype", c_int32), ("sm_scale", c_float),
        ("q", KdTensor), ("k", KdTensor), ("v", KdTensor), ("o", KdTensor), ("d_o", KdTensor),
        ("dq", KdTensor), ("dk", KdTensor), ("dv", KdTensor),
        ("lse", c_void_p), ("delta", c_void_p), ("plan", c_void_p), ("bwd_phases", c_int32), ("bwd_mode", c_int32),
        ("dq_acc", c_void_p), ("heads_per_cta", c_int32),
    ]


class KdError(RuntimeError):
    """A libkd_attention.so entry point rejected its arguments or a CUDA call failed."""


_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library once and declares the argument types of every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m kerneldev_b200.build` "
            "(needs nvcc; cross-compiles for sm_100a). This package has no other compute path.")
    lib = ctypes.CDLL(str(LIB_PATH))
    lib.kd_version.restype = c_int32
    lib.kd_last_error.restype = c_char_p
    lib.kd_plan_layout_get.argtypes = [c_int32, c_int32, POINTER(KdPlanLayout)]
    lib.kd_classify.argtypes = [POINTER(KdMeta), c_void_p, c_void_p]
    lib.kd_mask_dense.argtypes = [c_void_p, c_int32, c_int32, c_void_p, c_void_p]
    lib.kd_attn_fwd.argtypes = [POINTER(KdAttnParams), c_void_p]
    lib.kd_attn_bwd.argtypes = [POINTER(KdAttnParams), c_void_p]
    lib.kd_attn_bwd_static.argtypes = [POINTER(KdAttnParams), c_void_p]
    lib.kd_workspace_bytes.argtypes = [c_int32, c_int32, c_int32, c_int32, POINTER(c_size_t)]
    lib.kd_workspace_bytes_fused.argtypes = [c_int32, c_int32, c_int32, c_int32, POINTER(c_size_t)]
    lib.kd_hadamard.argtypes = [POINTER(KdTensor), POINTER(KdTensor), c_int32, c_int32, c_int32, c_int32,
                                c_int32, c_void_p, c_int32, c_void_p]
    lib.kd_span_index.argtypes = [c_void_p, c_int64, c_int32, c_int32, c_int64, c_int64, c_int64, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_void_p, c_void_p]
    lib.kd_span_mean.argtypes = [c_int32, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_int64, c_int32, c_int32, c_int32,
                                 c_int32, c_int32, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
    lib.kd_metadata_from_tokens.argtypes = [c_void_p, c_int64, c_int32, c_int32, c_int64, c_int64, c_int64, c_int64,
                                            c_void_p, c_void_p, c_void_p, c_void_p]
    for name in ("kd_plan_layout_get", "kd_classify", "kd_mask_dense", "kd_attn_fwd", "kd_attn_bwd", "kd_attn_bwd_static",
                 "kd_workspace_bytes", "kd_workspace_bytes_fused", "kd_hadamard", "kd_metadata_from_tokens", "kd_span_index", "kd_span_mean"):
        getattr(lib, name).restype = c_int32
    _lib = lib
    return lib


def check(rc: int) -> None:
    """Raises KdError with the library's message when an entry point returned a negative code."""
    if rc != 0:
        msg = load().kd_last_error().decode("utf-8", "replace")
        raise KdError(f"libkd_attention: error {rc}: {msg}")


def plan_layout(B: int, T: int) -> KdPlanLayout:
    out = KdPlanLayout()
    check(load().kd_plan_layout_get(B, T, ctypes.byref(out)))
    return out
