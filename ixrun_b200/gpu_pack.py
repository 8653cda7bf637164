"""Deploy-time quantise + pack on the GPU (replaces the CPU `int8x_quantize`,
ixrun/quantize.py:41-122, which takes minutes for a 27B model).

`quantize_pack_gpu` goes from a bf16 weight on the device to a ready
`DevicePacked` without touching the host except for the three level counts;
`int8x_quantize_gpu` returns the reference's packed dict (CPU tensors), bit for
bit what the CPU quantiser produces.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .packed import DevicePacked

__all__ = ["quantize_pack_gpu", "pack_codes_gpu", "int8x_quantize_gpu"]


def _pack(codes: torch.Tensor, scale: torch.Tensor, b1, q1, q2, counts, out_f: int, in_f: int) -> DevicePacked:
    dev = codes.device
    n1, n2, n3 = counts
    b2 = torch.empty((n2 + n3 + 31) // 32, dtype=torch.int32, device=dev)
    l1 = torch.empty((3 * n1 + 31) // 32, dtype=torch.int32, device=dev)
    l2 = torch.empty((5 * n2 + 31) // 32, dtype=torch.int32, device=dev)
    l3 = torch.empty(n3, dtype=torch.uint8, device=dev)
    st = _lib.packed_struct(b1, b2, l1, l2, l3, scale, out_f, in_f)
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().ixb_pack_codes(codes.data_ptr(), C.byref(st), q1.data_ptr(), q2.data_ptr(),
                                             _lib.stream_ptr(dev)))
    dp = DevicePacked.from_device_streams(b1, b2, l1, l2, l3, scale, out_f, in_f, blk_q1=q1, blk_q2=q2)
    dp.counts = [n1, n2, n3]
    dp.total_bytes = 2 + 4 * (b1.numel() + b2.numel() + l1.numel() + l2.numel()) + n3
    return dp


def _tables(n: int, dev):
    nb = (n + 1023) // 1024
    L = _lib.lib()
    ws = torch.empty(L.ixb_pack_workspace_bytes(n), dtype=torch.uint8, device=dev)
    b1 = torch.empty((n + 31) // 32, dtype=torch.int32, device=dev)
    q1 = torch.empty(nb, dtype=torch.int32, device=dev)
    q2 = torch.empty(nb, dtype=torch.int32, device=dev)
    return L, ws, b1, q1, q2


@torch.no_grad()
def quantize_pack_gpu(weight: torch.Tensor, return_codes: bool = False):
    """bf16 [out_f, in_f] on a CUDA device -> DevicePacked (and optionally the int8 codes)."""
    if not weight.is_cuda or weight.dtype != torch.bfloat16 or weight.dim() != 2:
        raise ValueError("quantize_pack_gpu needs a 2-D bf16 CUDA tensor")
    w = weight.contiguous()
    out_f, in_f = w.shape
    n, dev = w.numel(), w.device
    L, ws, b1, q1, q2 = _tables(n, dev)
    codes = torch.empty(n, dtype=torch.int8, device=dev)
    scale = torch.empty((), dtype=torch.bfloat16, device=dev)
    counts = (C.c_int64 * 3)()
    with torch.cuda.device(dev):
        _lib.check(L.ixb_quantize_codes(w.data_ptr(), n, scale.data_ptr(), codes.data_ptr(), b1.data_ptr(),
                                        q1.data_ptr(), q2.data_ptr(), counts, ws.data_ptr(), ws.numel(),
                                        _lib.stream_ptr(dev)))
    dp = _pack(codes, scale, b1, q1, q2, [int(c) for c in counts], out_f, in_f)
    return (dp, codes.view(out_f, in_f)) if return_codes else dp


@torch.no_grad()
def pack_codes_gpu(codes: torch.Tensor, scale: torch.Tensor, out_f: int, in_f: int) -> DevicePacked:
    """int8 codes on the device (+ the tensor's bf16 scale) -> DevicePacked."""
    if not codes.is_cuda or codes.dtype != torch.int8 or codes.numel() != out_f * in_f:
        raise ValueError("pack_codes_gpu needs out_f*in_f int8 codes on a CUDA device")
    c = codes.contiguous().reshape(-1)
    dev = c.device
    L, ws, b1, q1, q2 = _tables(c.numel(), dev)
    counts = (C.c_int64 * 3)()
    with torch.cuda.device(dev):
        _lib.check(L.ixb_count_codes(c.data_ptr(), c.numel(), b1.data_ptr(), q1.data_ptr(), q2.data_ptr(), counts,
                                     ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
    sc = scale.detach().to(dev, torch.bfloat16).reshape(()).contiguous()
    return _pack(c, sc, b1, q1, q2, [int(v) for v in counts], out_f, in_f)


@torch.no_grad()
def int8x_quantize_gpu(weight: torch.Tensor) -> dict:
    """Reference-format packed dict (CPU tensors) computed on the GPU."""
    dp = quantize_pack_gpu(weight.cuda() if not weight.is_cuda else weight)
    n = dp.N
    return {
        "level_bits": (3, 5, 8), "out_f": dp.out_f, "in_f": dp.in_f, "N": n, "scale": dp.scale.cpu(),
        "bitmaps": [dp.b1.cpu(), dp.b2.cpu()], "streams": [dp.l1.cpu(), dp.l2.cpu(), dp.l3.cpu()],
        "counts": list(dp.counts), "total_bytes": dp.total_bytes, "bits_per_weight": dp.total_bytes * 8 / n,
        "compression_vs_bf16": n * 2 / dp.total_bytes,
    }
