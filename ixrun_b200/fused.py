"""Fused decode + GEMV entry points with the reference's names and argument
meaning (ixrun/fused.py), backed by the CUDA library.

The reference needs one kernel for whole rows and a second, split-K kernel with
chunk-boundary prefixes for wide layers.  Here one kernel covers every shape:
work is split at 1024-element rank blocks (the gran=1024 prefix table), so the
`chunk` / `y32` arguments only select the output type the caller expects.
"""
from __future__ import annotations

import torch

from .packed import DevicePacked

__all__ = ["fused_gemv", "compute_row_prefixes", "FUSED_TILE", "_pick_split", "_pick_config"]

FUSED_TILE = 512  # the reference's inner tile; kept for callers that test `in_f % FUSED_TILE`

# rank tables derived per bitmap tensor, keyed by the tensor object's identity
_views: dict = {}
_MAX_VIEWS = 64


def compute_row_prefixes(packed, chunk: int | None = None, device=None):
    """(#L1, #L2) strictly before each row, or before each (row, chunk) start.

    Same values and index order (n * n_chunks + c) as ixrun/fused.py:35-78,
    computed on the GPU from the bitmaps.  Returned on the CPU like the
    reference unless `device` is given.
    """
    dp = packed if isinstance(packed, DevicePacked) else DevicePacked(packed)
    gran = dp.in_f if chunk is None else int(chunk)
    if chunk is not None and dp.in_f % gran:
        raise ValueError("chunk must divide in_f")
    q1, q2 = dp.prefix_tables(gran, dp.N // gran)
    if device is None:
        return q1.cpu(), q2.cpu()
    return q1.to(device), q2.to(device)


def _pick_config(out_f: int, in_f: int) -> tuple[int, int]:
    """(warps per CTA, elements per warp iteration) of the CUDA kernel: fixed."""
    return 8, 1024


def _pick_split(in_f: int) -> int:
    """Split factor the reference would use for a wide layer (ixrun/fused.py:196-203).

    Kept so that callers which size `chunk = in_f // _pick_split(in_f)` keep
    working; the CUDA kernel balances any shape without it.
    """
    for s in (2, 4):
        if in_f % s == 0 and (in_f // s) % 512 == 0:
            return s
    return 1


def _view(b1, b2, l1, l2, l3, scale, out_f, in_f) -> DevicePacked:
    key = id(b1)
    dp = _views.get(key)
    if dp is not None and dp.b1 is b1 and dp.out_f == out_f and dp.in_f == in_f and dp.l1 is l1:
        return dp
    dp = DevicePacked.from_device_streams(b1, b2, l1, l2, l3, scale, out_f, in_f)
    if len(_views) >= _MAX_VIEWS:          # bounded: the views keep their streams alive
        _views.pop(next(iter(_views)))
    _views[key] = dp
    return dp


@torch.no_grad()
def fused_gemv(x, b1, b2, l1, l2, l3, q1, q2, scale, out_f: int, in_f: int,
               chunk: int = 0, y32: torch.Tensor | None = None):
    """y = x @ W.T for one token with W decoded on the fly (ixrun/fused.py:297-347).

    x: bf16, numel == in_f.  q1/q2 (row or chunk prefixes) are accepted for
    signature compatibility; the kernel uses the gran=1024 table it derives from
    the bitmaps (cached per `b1` tensor).  chunk > 0 returns the fp32 result in
    `y32` (overwritten, not accumulated into: no pre-zeroing is needed), else a
    new bf16 [out_f] tensor is returned.
    """
    if x.dtype != torch.bfloat16 or x.numel() != in_f:
        raise ValueError("fused_gemv needs a bf16 activation with numel == in_f")
    dp = _view(b1, b2, l1, l2, l3, scale, out_f, in_f)
    xr = x.reshape(1, in_f)
    if chunk > 0:
        if y32 is None or y32.dtype != torch.float32 or y32.numel() != out_f:
            raise ValueError("split path needs an fp32 y32 buffer of out_f elements")
        dp.gemv(xr, out=y32.view(1, out_f))
        return y32
    return dp.gemv(xr).view(out_f)
