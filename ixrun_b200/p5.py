"""Resident re-layout "P5" of a packed tensor (see ``csrc/ixb_p5.cuh``).

The (3,5,8) streams remain the interchange format.  ``P5Packed.from_packed``
transcodes them on the GPU (decode to int8 codes, re-pack as a plane of fixed
5-bit fields in tensor-core fragment order + the level-3 weights of every
block as a short list); the int8 codes, and therefore every weight the reference would decode,
are preserved exactly.  The GEMV on this layout needs ~3 instructions per
weight instead of ~34 and costs the same for 1..8 activation rows.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .packed import DevicePacked

__all__ = ["P5Packed"]


class P5Packed:
    def __init__(self, codes: torch.Tensor, scale: torch.Tensor, out_f: int, in_f: int, n_esc: int | None = None,
                 total_bytes: int = 0):
        """codes: int8 [out_f*in_f] on a CUDA device; scale: bf16 scalar."""
        if not codes.is_cuda or codes.dtype != torch.int8 or codes.numel() != out_f * in_f:
            raise ValueError("P5Packed needs out_f*in_f int8 codes on a CUDA device")
        dev = codes.device
        self.device, self.out_f, self.in_f, self.N = dev, int(out_f), int(in_f), int(out_f) * int(in_f)
        self.total_bytes = int(total_bytes)          # the reference format's byte count of this tensor
        c = codes.contiguous().reshape(-1)
        if n_esc is None:
            n_esc = int((c.to(torch.int16).abs() > 15).sum().item())
        L = _lib.lib()
        nb = int(L.ixb_p5_blocks(self.out_f, self.in_f))
        # sizes include the slack that the GEMV's prefetch may read (4 blocks, 64 entries)
        self.w03 = torch.empty((nb + 4) * 32 * 4, dtype=torch.int32, device=dev)
        self.w4 = torch.empty((nb + 4) * 32, dtype=torch.int32, device=dev)
        self.blk_off = torch.empty(nb + 5, dtype=torch.int32, device=dev)
        self.esc = torch.empty(n_esc + 64, dtype=torch.int32, device=dev)
        self.n_esc = n_esc
        self.scale = scale.detach().to(dev, torch.bfloat16).reshape(()).contiguous()
        ws = torch.empty((nb + 5) * 4, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(L.ixb_p5_build(c.data_ptr(), self.scale.data_ptr(), self.out_f, self.in_f, self.w03.data_ptr(),
                                      self.w4.data_ptr(), self.blk_off.data_ptr(), self.esc.data_ptr(), n_esc,
                                      ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
        self.struct = _lib.P5Struct(self.w03.data_ptr(), self.w4.data_ptr(), self.blk_off.data_ptr(),
                                    self.esc.data_ptr(), n_esc, self.scale.data_ptr(), self.out_f, self.in_f)
        self.resident_bytes = 4 * (nb * 160 + nb + 1 + n_esc) + 2
        self._scratch = {}

    @classmethod
    def from_packed(cls, packed):
        """From the reference's packed dict or a DevicePacked: decode the streams to codes, re-lay out."""
        dp = packed if isinstance(packed, DevicePacked) else DevicePacked(packed)
        codes = dp.decode(kind="codes").reshape(-1)
        n_esc = dp.counts[2] if dp.counts is not None else None
        return cls(codes, dp.scale, dp.out_f, dp.in_f, n_esc=n_esc, total_bytes=dp.total_bytes)

    def decode(self, out: torch.Tensor | None = None, kind: str = "bf16") -> torch.Tensor:
        dtype = {"bf16": torch.bfloat16, "codes": torch.int8}[kind]
        if out is None:
            out = torch.empty(self.N, dtype=dtype, device=self.device)
        flat = out.reshape(-1)
        if flat.dtype != dtype or flat.numel() < self.N or not flat.is_contiguous():
            raise ValueError("decode output must be a contiguous tensor of the right dtype and size")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_p5_decode(C.byref(self.struct), flat.data_ptr(), 0 if kind == "codes" else 1,
                                                _lib.stream_ptr(self.device)))
        return flat[: self.N].view(self.out_f, self.in_f)

    def gemv(self, x: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
             out_dtype=torch.bfloat16) -> torch.Tensor:
        """y[M, out_f] = x[M, in_f] @ W.T, 1 <= M <= 8."""
        if x.dtype != torch.bfloat16:
            raise ValueError("activations must be bf16")
        x2 = x.reshape(-1, self.in_f)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        m = x2.shape[0]
        if out is None:
            out = torch.empty(m, self.out_f, dtype=out_dtype, device=self.device)
        elif out.dtype not in (torch.bfloat16, torch.float32) or out.numel() != m * self.out_f or not out.is_contiguous():
            raise ValueError("gemv output must be a contiguous bf16/fp32 tensor of M*out_f elements")
        if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != self.out_f):
            raise ValueError("bias must be bf16 [out_f]")
        s = self._scratch.get(m)
        if s is None:
            s = torch.zeros(_lib.lib().ixb_p5_gemv_scratch_bytes(self.out_f, self.in_f, m), dtype=torch.uint8,
                            device=self.device)
            self._scratch[m] = s
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_p5_gemv(C.byref(self.struct), x2.data_ptr(), m,
                                              None if bias is None else bias.data_ptr(), out.data_ptr(),
                                              1 if out.dtype == torch.float32 else 0, s.data_ptr(), s.numel(),
                                              _lib.stream_ptr(self.device)))
        return out
