"""The TPAB tile format of the reference (ixrun/tpab.py, ixrun/tpab_gemv.py) on this library's kernels.

Same function names and arguments as the reference's staging / decode / fused-GEMV entry points, so its callers
(ixrun/tpab_linear.py) and tests read the same; the packed dict of ``ixrun.tpab.encode_tpab`` is consumed unchanged
(the encoder is a deploy-time search on the host and is not rebuilt here).
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

__all__ = ["stage_gpu", "decode_tpab_triton", "prepare_gemv_stage", "fused_gemv_tpab"]


def stage_gpu(packed: dict, device="cuda") -> dict:
    """Upload the packed arrays once (ixrun/tpab.py:262-275) and build the C struct."""
    dev = torch.device(device)
    if not torch.cuda.is_available():
        raise _lib.IxbError("a CUDA device is required (there is no CPU path)")
    st = dict(packed)
    body = torch.cat([b.reshape(-1).to(torch.int32) for b in packed["bodies"]])
    st["bodies_g"] = torch.cat([body, torch.zeros(2, dtype=torch.int32)]).to(dev)          # two readable words behind
    st["bits_g"] = packed["bits"].to(dev, torch.uint8).contiguous()
    st["scales_g"] = packed["scales"].to(dev, torch.float16).contiguous()
    st["goff_g"] = packed["goff"].to(dev, torch.int32).contiguous()
    st["gbase_g"] = packed["gbase_bit"].to(dev, torch.int32)
    st["ol_t_g"] = packed["ol_t"].to(dev, torch.int32).contiguous()
    st["ol_l_g"] = packed["ol_l"].to(dev, torch.int32).contiguous()
    st["ol_val_g"] = packed["ol_val"].to(dev, torch.float16).contiguous()
    out_f, in_f = packed["shape"]
    gb = [int(v) for v in packed["gbase_bit"].tolist()] + [0] * 8
    st["struct"] = _lib.TpabStruct(st["bodies_g"].data_ptr(), st["bits_g"].data_ptr(), st["scales_g"].data_ptr(),
                                   st["goff_g"].data_ptr(), (C.c_int32 * 8)(*gb[:8]), int(out_f), int(in_f),
                                   int(packed["tile_r"]))
    st["device"] = dev
    return st


def decode_tpab_triton(packed: dict, device="cuda", staged: dict | None = None) -> torch.Tensor:
    """Full decode to bf16 [O, I], outliers included (ixrun/tpab.py:287-307)."""
    st = staged or stage_gpu(packed, device)
    dev = st["device"]
    out_f, in_f = packed["shape"]
    out = torch.empty(out_f, in_f, dtype=torch.bfloat16, device=dev)
    n_ol = st["ol_t_g"].numel()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().ixb_tpab_decode(C.byref(st["struct"]), st["ol_t_g"].data_ptr() if n_ol else None,
                                              st["ol_l_g"].data_ptr() if n_ol else None,
                                              st["ol_val_g"].data_ptr() if n_ol else None, n_ol, out.data_ptr(),
                                              _lib.stream_ptr(dev)))
    return out


def prepare_gemv_stage(packed: dict, device="cuda", staged: dict | None = None) -> dict:
    """Stage for the GEMV: the arrays of ``stage_gpu`` + the outliers as per-row lists (ixrun/tpab_gemv.py:28-67)."""
    st = dict(staged) if staged is not None else stage_gpu(packed, device)
    dev = st["device"]
    out_f, in_f = packed["shape"]
    tile_r, tile_c = int(packed["tile_r"]), 64
    ol_t, ol_l = st["ol_t_g"].long(), st["ol_l_g"].long()
    r = ol_t // (in_f // tile_c) * tile_r + ol_l // tile_c
    k = (ol_t % (in_f // tile_c)) * tile_c + ol_l % tile_c
    order = torch.argsort(r, stable=True)
    offs = torch.zeros(out_f + 1, dtype=torch.int32, device=dev)
    offs[1:] = torch.bincount(r, minlength=out_f).cumsum(0).to(torch.int32)
    st["ol_row_k"] = k[order].to(torch.int32).contiguous()
    st["ol_row_v"] = st["ol_val_g"][order].contiguous()                 # fp16; rounded to bf16 in the kernel
    st["ol_offs"] = offs
    L = _lib.lib()
    st["scratch"] = torch.empty(max(1, L.ixb_tpab_gemv_scratch_bytes(out_f, in_f, tile_r)), dtype=torch.uint8, device=dev)
    return st


def fused_gemv_tpab(x: torch.Tensor, st: dict, out_f: int, in_f: int, tile_r: int = 64, bias: torch.Tensor | None = None,
                    out_dtype=torch.bfloat16) -> torch.Tensor:
    """y = x @ W.T for a single token, W decoded on the fly (ixrun/tpab_gemv.py:127-143); x: [in_f] bf16."""
    if x.dtype != torch.bfloat16 or x.numel() != in_f:
        raise ValueError("x must be bf16 with in_f elements")
    dev = st["device"]
    y = torch.empty(out_f, dtype=out_dtype, device=dev)
    n_ol = st["ol_row_k"].numel()
    xf = x.reshape(-1).contiguous()
    with torch.cuda.device(dev):
        _lib.check(_lib.lib().ixb_tpab_gemv(C.byref(st["struct"]), xf.data_ptr(), st["ol_offs"].data_ptr() if n_ol else None,
                                            st["ol_row_k"].data_ptr() if n_ol else None,
                                            st["ol_row_v"].data_ptr() if n_ol else None,
                                            None if bias is None else bias.data_ptr(), y.data_ptr(),
                                            1 if out_dtype == torch.float32 else 0, st["scratch"].data_ptr(),
                                            st["scratch"].numel(), _lib.stream_ptr(dev)))
    return y
