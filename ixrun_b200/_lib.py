"""ctypes binding of ``libixb200.so`` (the C ABI declared in ``include/ixb200.h``).

There is no fallback: if the library is missing and cannot be built, or a call
fails, an exception is raised.  torch is used only to own device memory and to
name the current stream; the library itself sees raw pointers.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

from . import build as _build

_HERE = os.path.dirname(os.path.abspath(__file__))
_lib = None

SYMBOLS = (
    "ixb_version", "ixb_last_error", "ixb_launch_count",
    "ixb_prefix_workspace_bytes", "ixb_prefix_tables",
    "ixb_decode", "ixb_gemv_scratch_bytes", "ixb_gemv", "ixb_gemv_static",
    "ixb_gemm_scratch_bytes", "ixb_gemm",
    "ixb_pack_workspace_bytes", "ixb_quantize_codes", "ixb_count_codes", "ixb_pack_codes", "ixb_group_scale", "ixb_tpab_decode", "ixb_tpab_gemv_scratch_bytes", "ixb_tpab_gemv",
    "ixb_p6_blocks", "ixb_p6_build", "ixb_p6_decode", "ixb_p6_gemv_scratch_bytes", "ixb_p6_gemv", "ixb_set_pdl",
    "ixb_p6_gemm_scratch_bytes", "ixb_p6_gemm",
    "ixb_allreduce_bytes", "ixb_allreduce", "ixb_p6_gemv_push", "ixb_allreduce_finish", "ixb_p6_gemv_allreduce", "ixb_allreduce_spin_limit",
    "ixb_add_rmsnorm", "ixb_allreduce_finish_add_rmsnorm", "ixb_swiglu", "ixb_rope_kv", "ixb_attn_scratch_bytes", "ixb_attn_decode", "ixb_conv_update", "ixb_gdn_step", "ixb_gdn_conv_step",
)


class IxbError(RuntimeError):
    """A call into libixb200 returned a non-zero status."""


class Packed(C.Structure):
    """Mirror of ``struct ixb_packed``."""

    _fields_ = [
        ("b1", C.c_void_p), ("b1_words", C.c_int64),
        ("b2", C.c_void_p), ("b2_words", C.c_int64),
        ("l1", C.c_void_p), ("l1_words", C.c_int64),
        ("l2", C.c_void_p), ("l2_words", C.c_int64),
        ("l3", C.c_void_p), ("l3_bytes", C.c_int64),
        ("scale", C.c_void_p),
        ("out_f", C.c_int64), ("in_f", C.c_int64),
    ]


class P6Struct(C.Structure):
    """Mirror of ``struct ixb_p6``."""

    _fields_ = [
        ("plane", C.c_void_p), ("blk_off", C.c_void_p), ("esc", C.c_void_p),
        ("n_esc", C.c_int64), ("scale", C.c_void_p), ("out_f", C.c_int64), ("in_f", C.c_int64),
        ("scale_stride", C.c_int64),
    ]


class TpabStruct(C.Structure):
    """Mirror of ``struct ixb_tpab``."""

    _fields_ = [("body", C.c_void_p), ("bits", C.c_void_p), ("scales", C.c_void_p), ("goff", C.c_void_p),
                ("gbase_bit", C.c_int32 * 8), ("out_f", C.c_int64), ("in_f", C.c_int64), ("tile_r", C.c_int64)]


def lib():
    """Load (building first if the in-tree .so is missing or stale)."""
    global _lib
    if _lib is not None:
        return _lib
    so = _build.SO
    if _build.is_stale():
        try:
            so = _build.build()
        except Exception as e:  # no silent fallback: a stale library is not loaded in place of a failed build
            raise IxbError(f"libixb200.so is missing or older than its sources and cannot be built here: {e}") from e
    L = C.CDLL(so)
    vp, i64, sz = C.c_void_p, C.c_int64, C.c_size_t
    L.ixb_version.restype = C.c_int
    L.ixb_last_error.restype = C.c_char_p
    L.ixb_launch_count.restype = i64
    L.ixb_prefix_workspace_bytes.restype = sz
    L.ixb_prefix_workspace_bytes.argtypes = [i64]
    L.ixb_prefix_tables.restype = C.c_int
    L.ixb_prefix_tables.argtypes = [C.POINTER(Packed), i64, i64, vp, vp, vp, sz, vp]
    L.ixb_decode.restype = C.c_int
    L.ixb_decode.argtypes = [C.POINTER(Packed), vp, vp, vp, C.c_int, vp]
    L.ixb_gemv_scratch_bytes.restype = sz
    L.ixb_gemv_scratch_bytes.argtypes = [i64, i64, i64]
    L.ixb_gemv.restype = C.c_int
    L.ixb_gemv.argtypes = [C.POINTER(Packed), vp, vp, vp, i64, vp, vp, C.c_int, vp, sz, vp]
    L.ixb_gemm_scratch_bytes.restype = sz
    L.ixb_gemm_scratch_bytes.argtypes = [i64, i64, i64]
    L.ixb_gemm.restype = C.c_int
    L.ixb_gemm.argtypes = [C.POINTER(Packed), vp, vp, vp, i64, vp, vp, C.c_int, vp, sz, vp]
    L.ixb_pack_workspace_bytes.restype = sz
    L.ixb_pack_workspace_bytes.argtypes = [i64]
    L.ixb_quantize_codes.restype = C.c_int
    L.ixb_quantize_codes.argtypes = [vp, i64, vp, vp, vp, vp, vp, C.POINTER(i64), vp, sz, vp]
    L.ixb_count_codes.restype = C.c_int
    L.ixb_count_codes.argtypes = [vp, i64, vp, vp, vp, C.POINTER(i64), vp, sz, vp]
    L.ixb_pack_codes.restype = C.c_int
    L.ixb_pack_codes.argtypes = [vp, C.POINTER(Packed), vp, vp, vp]
    L.ixb_p6_blocks.restype = i64
    L.ixb_p6_blocks.argtypes = [i64, i64]
    L.ixb_p6_build.restype = C.c_int
    L.ixb_p6_build.argtypes = [vp, vp, i64, i64, i64, vp, vp, vp, i64, vp, sz, vp]
    L.ixb_p6_decode.restype = C.c_int
    L.ixb_p6_decode.argtypes = [C.POINTER(P6Struct), vp, C.c_int, vp]
    L.ixb_p6_gemv_scratch_bytes.restype = sz
    L.ixb_p6_gemv_scratch_bytes.argtypes = [i64, i64, i64]
    L.ixb_p6_gemv.restype = C.c_int
    L.ixb_p6_gemv.argtypes = [C.POINTER(P6Struct), vp, i64, vp, vp, C.c_int, vp, sz, vp]
    L.ixb_set_pdl.restype = C.c_int
    L.ixb_set_pdl.argtypes = [C.c_int]
    L.ixb_allreduce_bytes.restype = sz
    L.ixb_allreduce_bytes.argtypes = [C.c_int, i64]
    L.ixb_allreduce.restype = C.c_int
    L.ixb_allreduce.argtypes = [vp, i64, C.POINTER(C.c_void_p), C.c_int, C.c_int, i64, vp, vp, C.c_int, vp]
    L.ixb_p6_gemv_push.restype = C.c_int
    L.ixb_p6_gemv_push.argtypes = [C.POINTER(P6Struct), vp, i64, C.POINTER(C.c_void_p), C.c_int, C.c_int, i64, vp, sz, vp]
    L.ixb_p6_gemv_allreduce.restype = C.c_int
    L.ixb_p6_gemv_allreduce.argtypes = [C.POINTER(P6Struct), vp, i64, C.POINTER(C.c_void_p), C.c_int, C.c_int, i64, vp, vp,
                                        C.c_int, vp, sz, vp]
    L.ixb_allreduce_finish.restype = C.c_int
    L.ixb_allreduce_finish.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, i64, i64, vp, vp, C.c_int, vp]
    L.ixb_allreduce_spin_limit.restype = C.c_uint32
    L.ixb_allreduce_spin_limit.argtypes = [C.c_uint32]
    f32 = C.c_float
    L.ixb_add_rmsnorm.restype = C.c_int
    L.ixb_add_rmsnorm.argtypes = [vp, vp, vp, f32, vp, i64, i64, vp]
    L.ixb_swiglu.restype = C.c_int
    L.ixb_swiglu.argtypes = [vp, vp, vp, i64, i64, i64, vp]
    L.ixb_rope_kv.restype = C.c_int
    L.ixb_rope_kv.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, f32, i64, i64, i64, i64, vp]
    L.ixb_allreduce_finish_add_rmsnorm.restype = C.c_int
    L.ixb_allreduce_finish_add_rmsnorm.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, i64, vp, vp, f32, vp, i64, i64, vp]
    L.ixb_p6_gemm_scratch_bytes.restype = sz
    L.ixb_p6_gemm_scratch_bytes.argtypes = [i64, i64, i64]
    L.ixb_p6_gemm.restype = C.c_int
    L.ixb_p6_gemm.argtypes = [C.POINTER(P6Struct), vp, i64, vp, vp, C.c_int, vp, sz, vp]
    L.ixb_tpab_decode.restype = C.c_int
    L.ixb_tpab_decode.argtypes = [C.POINTER(TpabStruct), vp, vp, vp, i64, vp, vp]
    L.ixb_tpab_gemv_scratch_bytes.restype = sz
    L.ixb_tpab_gemv_scratch_bytes.argtypes = [i64, i64, i64]
    L.ixb_tpab_gemv.restype = C.c_int
    L.ixb_tpab_gemv.argtypes = [C.POINTER(TpabStruct), vp, vp, vp, vp, vp, vp, C.c_int, vp, sz, vp]
    L.ixb_group_scale.restype = C.c_int
    L.ixb_group_scale.argtypes = [vp, vp, i64, i64, vp, vp]
    L.ixb_attn_scratch_bytes.restype = sz
    L.ixb_attn_scratch_bytes.argtypes = [i64, i64, i64]
    L.ixb_attn_decode.restype = C.c_int
    L.ixb_attn_decode.argtypes = [vp, vp, vp, vp, vp, i64, vp, vp, sz, i64, i64, i64, i64, f32, i64, i64, i64, i64, vp]
    L.ixb_conv_update.restype = C.c_int
    L.ixb_conv_update.argtypes = [vp, vp, vp, vp, vp, i64, i64, vp]
    L.ixb_gdn_conv_step.restype = C.c_int
    L.ixb_gdn_conv_step.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, f32, vp]
    L.ixb_gdn_step.restype = C.c_int
    L.ixb_gdn_step.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, f32, vp]
    L.ixb_gemv_static.restype = C.c_int
    L.ixb_gemv_static.argtypes = [C.POINTER(Packed), vp, vp, vp, i64, vp, vp, C.c_int, vp]
    _lib = L
    return L


def check(rc: int):
    if rc != 0:
        raise IxbError(f"ixb200 error {rc}: {lib().ixb_last_error().decode()}")


def stream_ptr(device=None) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def packed_struct(b1, b2, l1, l2, l3, scale, out_f: int, in_f: int) -> Packed:
    """Build the C struct from device tensors (kept alive by the caller)."""
    for t in (b1, b2, l1, l2, l3, scale):
        if not t.is_cuda:
            raise IxbError("packed streams must live on a CUDA device")
        if not t.is_contiguous():
            raise IxbError("packed streams must be contiguous")
    return Packed(
        _p(b1), b1.numel(), _p(b2), b2.numel(), _p(l1), l1.numel(), _p(l2), l2.numel(),
        _p(l3), l3.numel(), scale.data_ptr(), out_f, in_f,
    )
