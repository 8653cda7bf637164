"""Resident re-layout "P6" of a packed tensor (see ``csrc/ixb_p6.cuh``).

The (3,5,8) streams remain the interchange format; ``P6Packed.from_packed``
transcodes them on the GPU, keeping every int8 code.  P6 spends 6 plane bits per weight on a field that *is* part of the
bf16 number ``1 + code/32`` (codes -16..31), so one fused multiply-add per pair
of weights yields the reference's ``bf16(code * scale)``; every other code goes
to a short list that the GEMV adds on the CUDA cores.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .packed import DevicePacked

__all__ = ["P6Packed", "set_pdl", "GemvScratch"]


def set_pdl(on: bool) -> bool:
    """Programmatic dependent launch for the P6 GEMV (process-wide; returns the previous setting).

    When on, a GEMV launch may begin fetching its weights while the kernel ahead of it in the stream finishes; it
    still waits for that kernel before touching activations, output or scratch.  Turn it on after deployment, once
    the device has been synchronised: a layout still being built would be read too early."""
    return bool(_lib.lib().ixb_set_pdl(1 if on else 0))

CODE_MIN, CODE_MAX = -16, 31     # codes that the plane holds
SLACK_BLOCKS, SLACK_ENTRIES, BLOCK_BYTES = 5, 64, 768


class GemvScratch:
    """Scratch of the P6 GEMV on one device: zero between launches (every launch leaves it as it found it), so ONE
    buffer serves every layer that runs on the same stream, whatever its shape.  Launches that may overlap on the
    GPU (different streams without ordering) need separate instances."""

    MIN_BYTES = 1 << 20
    _per_device: dict = {}

    def __init__(self, device):
        self.device = torch.device(device)
        self.buf = torch.zeros(0, dtype=torch.uint8, device=self.device)
        self._retired = []      # outgrown buffers stay allocated: a captured CUDA graph may still point at them

    @classmethod
    def shared(cls, device) -> "GemvScratch":
        device = torch.device(device)
        key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
        s = cls._per_device.get(key)
        if s is None:
            s = cls._per_device[key] = cls(device)
        return s

    def reserve(self, nbytes: int) -> torch.Tensor:
        if self.buf.numel() < nbytes:
            if self.buf.numel():
                self._retired.append(self.buf)
            self.buf = torch.zeros(max(int(nbytes), self.MIN_BYTES), dtype=torch.uint8, device=self.device)
        return self.buf


class P6Packed:
    def __init__(self, codes: torch.Tensor, scale: torch.Tensor, out_f: int, in_f: int, total_bytes: int = 0,
                 scratch: GemvScratch | None = None):
        """codes: int8 [out_f*in_f] on a CUDA device; scale: one bf16 value, or one per 16-row tile (a tensor fused
        row-wise from several, see ``fuse``)."""
        if not codes.is_cuda or codes.dtype != torch.int8 or codes.numel() != out_f * in_f:
            raise ValueError("P6Packed needs out_f*in_f int8 codes on a CUDA device")
        dev = codes.device
        self.device, self.out_f, self.in_f, self.N = dev, int(out_f), int(in_f), int(out_f) * int(in_f)
        self.total_bytes = int(total_bytes)          # the reference format's byte count of this tensor
        c = codes.contiguous().reshape(-1)
        n_esc = int(((c < CODE_MIN) | (c > CODE_MAX)).sum().item())
        L = _lib.lib()
        nb = int(L.ixb_p6_blocks(self.out_f, self.in_f))
        # sizes include the slack that the GEMV's prefetch may read
        self.plane = torch.empty((nb + SLACK_BLOCKS) * BLOCK_BYTES // 4, dtype=torch.int32, device=dev)
        self.blk_off = torch.empty(nb + 1, dtype=torch.int32, device=dev)
        self.esc = torch.empty(n_esc + SLACK_ENTRIES, dtype=torch.int32, device=dev)
        self.n_esc = n_esc
        self.scale = scale.detach().to(dev, torch.bfloat16).reshape(-1).contiguous()
        if self.scale.numel() not in (1, (self.out_f + 15) // 16):
            raise ValueError("scale must hold one value, or one per 16-row tile")
        stride = 0 if self.scale.numel() == 1 else 1
        self.sections = [(0, self.out_f)]            # (first row, rows) of every fused part
        ws = torch.empty((nb + 1) * 4, dtype=torch.uint8, device=dev)
        with torch.cuda.device(dev):
            _lib.check(L.ixb_p6_build(c.data_ptr(), self.scale.data_ptr(), stride, self.out_f, self.in_f, self.plane.data_ptr(),
                                      self.blk_off.data_ptr(), self.esc.data_ptr(), n_esc,
                                      ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev)))
        self.struct = _lib.P6Struct(self.plane.data_ptr(), self.blk_off.data_ptr(), self.esc.data_ptr(), n_esc,
                                    self.scale.data_ptr(), self.out_f, self.in_f, stride)
        self.resident_bytes = nb * BLOCK_BYTES + 4 * (nb + 1 + n_esc) + 2
        self.scratch = scratch if scratch is not None else GemvScratch.shared(dev)

    @classmethod
    def from_packed(cls, packed, **kw):
        """From the reference's packed dict or a DevicePacked: decode the streams to codes, re-lay out."""
        dp = packed if isinstance(packed, DevicePacked) else DevicePacked(packed)
        codes = dp.decode(kind="codes").reshape(-1)
        return cls(codes, dp.scale, dp.out_f, dp.in_f, total_bytes=dp.total_bytes, **kw)

    @classmethod
    def fuse(cls, parts, **kw):
        """One resident tensor from several packed tensors that share their input (q|k|v, gate|up, the four
        in-projections of a gated-delta-rule layer): the parts' codes stacked row-wise, every part padded with zero
        codes to a whole number of 16-row tiles and keeping its own per-tensor scale, so the fused GEMV gives every
        part's outputs bit for bit as the part alone would.  ``sections`` lists (first row, rows) of every part in
        the fused output; ``split(y)`` cuts a one-row output into the parts' views."""
        dps = [p if isinstance(p, DevicePacked) else DevicePacked(p) for p in parts]
        in_f = dps[0].in_f
        if any(d.in_f != in_f for d in dps):
            raise ValueError("fused tensors must share in_f")
        dev = dps[0].device
        codes, scales, sections, row = [], [], [], 0
        for d in dps:
            c = d.decode(kind="codes").reshape(d.out_f, in_f)
            pad = (-d.out_f) % 16
            if pad:
                c = torch.cat([c, torch.zeros(pad, in_f, dtype=torch.int8, device=dev)])
            codes.append(c)
            scales.append(d.scale.detach().to(dev, torch.bfloat16).reshape(1).expand((d.out_f + pad) // 16))
            sections.append((row, d.out_f))
            row += d.out_f + pad
        self = cls(torch.cat(codes).reshape(-1), torch.cat(scales), row, in_f,
                   total_bytes=sum(d.total_bytes for d in dps), **kw)
        self.sections = sections
        return self

    def split(self, y: torch.Tensor):
        """Views of a one-row output [1, out_f] (or [out_f]) per fused part."""
        flat = y.reshape(-1)
        if flat.numel() != self.out_f:
            raise ValueError("split takes a one-row output")
        return [flat[a:a + n] for a, n in self.sections]

    def decode(self, out: torch.Tensor | None = None, kind: str = "bf16") -> torch.Tensor:
        dtype = {"bf16": torch.bfloat16, "codes": torch.int8}[kind]
        if out is None:
            out = torch.empty(self.N, dtype=dtype, device=self.device)
        flat = out.reshape(-1)
        if flat.dtype != dtype or flat.numel() < self.N or not flat.is_contiguous():
            raise ValueError("decode output must be a contiguous tensor of the right dtype and size")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_p6_decode(C.byref(self.struct), flat.data_ptr(), 0 if kind == "codes" else 1,
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
        L = _lib.lib()
        with torch.cuda.device(self.device):
            s = self.scratch.reserve(L.ixb_p6_gemv_scratch_bytes(self.out_f, self.in_f, m))
            _lib.check(L.ixb_p6_gemv(C.byref(self.struct), x2.data_ptr(), m,
                                     None if bias is None else bias.data_ptr(), out.data_ptr(),
                                     1 if out.dtype == torch.float32 else 0, s.data_ptr(), s.numel(),
                                     _lib.stream_ptr(self.device)))
        return out

    GEMM_MAX_ROWS = 64

    def gemm(self, x: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
             out_dtype=torch.bfloat16) -> torch.Tensor:
        """y[M, out_f] = x[M, in_f] @ W.T for 1 <= M <= 64 on the tensor cores, reading the resident layout once
        (in_f a multiple of 64).  The scratch (split-K partial sums) is kept per tensor shape on this object."""
        if x.dtype != torch.bfloat16:
            raise ValueError("activations must be bf16")
        x2 = x.reshape(-1, self.in_f)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        m = x2.shape[0]
        if out is None:
            out = torch.empty(m, self.out_f, dtype=out_dtype, device=self.device)
        elif out.dtype not in (torch.bfloat16, torch.float32) or out.numel() != m * self.out_f or not out.is_contiguous():
            raise ValueError("gemm output must be a contiguous bf16/fp32 tensor of M*out_f elements")
        if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != self.out_f):
            raise ValueError("bias must be bf16 [out_f]")
        L = _lib.lib()
        need = int(L.ixb_p6_gemm_scratch_bytes(self.out_f, self.in_f, m))
        if need == 0:
            raise ValueError(f"unsupported GEMM shape: {m} rows")
        ws = getattr(self, "_gemm_ws", None)
        if ws is None or ws.numel() < need:
            ws = self._gemm_ws = torch.empty(need, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(L.ixb_p6_gemm(C.byref(self.struct), x2.data_ptr(), m, None if bias is None else bias.data_ptr(),
                                     out.data_ptr(), 1 if out.dtype == torch.float32 else 0, ws.data_ptr(), ws.numel(),
                                     _lib.stream_ptr(self.device)))
        return out

    def gemv_push(self, x: torch.Tensor, ar) -> int:
        """Row-parallel shard: y = x @ W.T as fp32 partial sums stored straight into every rank's all-reduce buffer
        (``ar``: a parallel.PeerAllReduce) from the GEMV's epilogue.  Returns the number of values pushed; follow it
        with ``ar.finish(n, out, bias)`` on the same stream."""
        if x.dtype != torch.bfloat16:
            raise ValueError("activations must be bf16")
        x2 = x.reshape(-1, self.in_f)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        m = x2.shape[0]
        L = _lib.lib()
        with torch.cuda.device(self.device):
            s = self.scratch.reserve(L.ixb_p6_gemv_scratch_bytes(self.out_f, self.in_f, m))
            _lib.check(L.ixb_p6_gemv_push(C.byref(self.struct), x2.data_ptr(), m, ar._ptrs, ar.rank, ar.world, ar.n_max,
                                          s.data_ptr(), s.numel(), _lib.stream_ptr(self.device)))
        return m * self.out_f

    def gemv_allreduce(self, x: torch.Tensor, ar, out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                       out_dtype=torch.bfloat16) -> torch.Tensor:
        """Row-parallel shard, ONE kernel: y = sum over the ranks of x @ W.T (+ bias).  The GEMV stores its partial
        sums into every rank's all-reduce buffer as its tiles finish, and its warps then add up all ranks' words."""
        if x.dtype != torch.bfloat16:
            raise ValueError("activations must be bf16")
        x2 = x.reshape(-1, self.in_f)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        m = x2.shape[0]
        if out is None:
            out = torch.empty(m, self.out_f, dtype=out_dtype, device=self.device)
        elif out.dtype not in (torch.bfloat16, torch.float32) or out.numel() != m * self.out_f or not out.is_contiguous():
            raise ValueError("output must be a contiguous bf16/fp32 tensor of M*out_f elements")
        if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != self.out_f):
            raise ValueError("bias must be bf16 [out_f]")
        L = _lib.lib()
        with torch.cuda.device(self.device):
            s = self.scratch.reserve(L.ixb_p6_gemv_scratch_bytes(self.out_f, self.in_f, m))
            _lib.check(L.ixb_p6_gemv_allreduce(C.byref(self.struct), x2.data_ptr(), m, ar._ptrs, ar.rank, ar.world, ar.n_max,
                                               None if bias is None else bias.data_ptr(), out.data_ptr(),
                                               1 if out.dtype == torch.float32 else 0, s.data_ptr(), s.numel(),
                                               _lib.stream_ptr(self.device)))
        return out
