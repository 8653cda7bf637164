"""The sibling group-scale format of the reference (``ixgs``: per-group fp16 scales, group size 64, codes within
-15 .. 16 so that level 3 is empty by construction) on this library's kernels.

Mirrors the reference's decode entry point and module (ixgs/kernels.py ``decode_weight_triton``, ixgs/linear.py
``Int8GSLinear``): the packed dict of ``ixgs.quantize.int8gs_quantize`` is consumed unchanged.  Its five streams are
the (3,5,8) streams of the main format with the same field offsets, so ``ixb_decode`` turns them into int8 codes and one
more kernel applies the group scales: ``w = bf16(f32(code) * f32(scale[e // group]))``.  The reference has no fused
GEMV for this format (its module decodes, then runs a dense matmul), and neither has this module.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import _lib
from .packed import DevicePacked

__all__ = ["decode_weight_triton", "Int8GSLinear"]


def _as_main_format(packed: dict) -> dict:
    """The group-scale dict in the main format's keys (exact stream lengths; the per-tensor scale is unused)."""
    n1, n2, n3 = (int(c) for c in packed["counts"])
    b2 = packed["b2"][: (n2 + n3 + 31) // 32]             # the reference pads empty streams to one element
    l3 = packed["l3"][:n3]
    return {"level_bits": (3, 5, 8), "out_f": packed["out_f"], "in_f": packed["in_f"], "N": packed["N"],
            "scale": torch.ones((), dtype=torch.bfloat16), "bitmaps": [packed["b1"], b2],
            "streams": [packed["l1"], packed["l2"], l3], "counts": [n1, n2, n3], "total_bytes": packed.get("total_bytes", 0)}


def decode_weight_triton(packed: dict, device=None, dtype=torch.bfloat16) -> torch.Tensor:
    """bf16 weight [out_f, in_f] of a group-scale packed dict (same name and result as ixgs/kernels.py:105-170)."""
    dp = DevicePacked(_as_main_format(packed), device)
    codes = dp.decode(kind="codes").reshape(-1)
    gs = packed["group_scales"].to(dp.device, torch.float16).contiguous()
    n, group = int(packed["N"]), int(packed["group_size"])
    if gs.numel() * group < n:
        raise ValueError("too few group scales")
    out = torch.empty(n, dtype=torch.bfloat16, device=dp.device)
    with torch.cuda.device(dp.device):
        _lib.check(_lib.lib().ixb_group_scale(codes.data_ptr(), gs.data_ptr(), n, group, out.data_ptr(), _lib.stream_ptr(dp.device)))
    w = out.view(packed["out_f"], packed["in_f"])
    return w if dtype == torch.bfloat16 else w.to(dtype)


class Int8GSLinear(nn.Module):
    """Drop-in for ixgs/linear.py:34-70: cache='full' decodes once at deploy, cache='none' re-decodes every forward."""

    def __init__(self, packed: dict, bias=None, cache: str = "full"):
        super().__init__()
        if cache not in ("full", "none"):
            raise ValueError("cache must be 'full' or 'none'")
        self.packed = packed
        self.out_features, self.in_features = packed["out_f"], packed["in_f"]
        self._cache = cache
        self._bias = None if bias is None else bias.detach().clone().cuda()
        self._w = decode_weight_triton(packed) if cache == "full" else None

    def forward(self, x):
        w = self._w if self._cache == "full" else decode_weight_triton(self.packed, x.device)
        bias = self._bias.to(x.dtype) if self._bias is not None else None
        return F.linear(x, w.to(x.dtype), bias)
