"""Device-resident packed tensor: the five INT8-X streams, the per-1024-element
rank tables and the scratch the fused kernels need, plus thin wrappers over the
C ABI.  Every packed-linear module of this package owns one of these.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

BLOCK = 1024


def _dev_tensor(t: torch.Tensor, device, dtype) -> torch.Tensor:
    t = t.to(device=device)
    if t.dtype != dtype:
        t = t.view(dtype) if t.element_size() == torch.empty((), dtype=dtype).element_size() else t.to(dtype)
    return t.contiguous()


class DevicePacked:
    """Streams of one packed [out_f, in_f] tensor on a CUDA device."""

    def __init__(self, packed: dict, device=None):
        if tuple(packed["level_bits"]) != (3, 5, 8):
            raise ValueError(f"only the (3, 5, 8) scheme is supported, got {packed['level_bits']}")
        if not torch.cuda.is_available():
            raise _lib.IxbError("a CUDA device is required (there is no CPU path)")
        device = torch.device("cuda" if device is None else device)
        self.device = device
        self.out_f, self.in_f, self.N = int(packed["out_f"]), int(packed["in_f"]), int(packed["N"])
        self.counts = list(packed["counts"])
        self.total_bytes = int(packed.get("total_bytes", 0))
        n1, n2, n3 = self.counts
        if n1 + n2 + n3 != self.N or self.N != self.out_f * self.in_f:
            raise ValueError("packed dict is inconsistent: counts do not sum to out_f*in_f")
        b1, b2 = packed["bitmaps"]
        l1, l2, l3 = packed["streams"]
        want = [(self.N + 31) // 32, (n2 + n3 + 31) // 32, (3 * n1 + 31) // 32, (5 * n2 + 31) // 32, n3]
        for name, t, w in zip(("B1", "B2", "L1", "L2", "L3"), (b1, b2, l1, l2, l3), want):
            if t.numel() != w:
                raise ValueError(f"packed dict is inconsistent: {name} has {t.numel()} entries, expected {w}")
        self.b1 = _dev_tensor(b1, device, torch.int32)
        self.b2 = _dev_tensor(b2, device, torch.int32)
        self.l1 = _dev_tensor(l1, device, torch.int32)
        self.l2 = _dev_tensor(l2, device, torch.int32)
        self.l3 = _dev_tensor(l3, device, torch.uint8)
        self.scale = packed["scale"].to(device=device, dtype=torch.bfloat16).reshape(()).contiguous()
        self._init_tables()

    @classmethod
    def from_device_streams(cls, b1, b2, l1, l2, l3, scale, out_f: int, in_f: int, blk_q1=None, blk_q2=None):
        """Wrap streams that already live on the device (no copies); the gran=1024 rank tables are
        computed unless given."""
        self = cls.__new__(cls)
        self.device = b1.device
        self.out_f, self.in_f, self.N = int(out_f), int(in_f), int(out_f) * int(in_f)
        self.counts = None
        self.total_bytes = 0
        self.b1, self.b2, self.l1, self.l2, self.l3 = b1, b2, l1, l2, l3
        self.scale = scale.reshape(()).to(torch.bfloat16)
        self._init_tables(blk_q1, blk_q2)
        return self

    # ------------------------------------------------------------ plumbing --
    def _init_tables(self, blk_q1=None, blk_q2=None):
        self.struct = _lib.packed_struct(self.b1, self.b2, self.l1, self.l2, self.l3, self.scale,
                                         self.out_f, self.in_f)
        self.n_blocks = (self.N + BLOCK - 1) // BLOCK
        if blk_q1 is None or blk_q2 is None:
            blk_q1, blk_q2 = self.prefix_tables(BLOCK, self.n_blocks)
        self.blk_q1, self.blk_q2 = blk_q1, blk_q2
        self._scratch = {}

    def prefix_tables(self, gran: int, n_units: int | None = None):
        """(#L1, #L2) before flat positions u*gran, as int32 device tensors."""
        L = _lib.lib()
        if n_units is None:
            n_units = (self.N + gran - 1) // gran
        q1 = torch.empty(n_units, dtype=torch.int32, device=self.device)
        q2 = torch.empty(n_units, dtype=torch.int32, device=self.device)
        ws_bytes = L.ixb_prefix_workspace_bytes(self.N)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(L.ixb_prefix_tables(C.byref(self.struct), gran, n_units, q1.data_ptr(), q2.data_ptr(),
                                           ws.data_ptr(), ws_bytes, _lib.stream_ptr(self.device)))
        # the workspace may be freed while the kernels are still queued: torch's
        # caching allocator only reuses it on this same stream, which is safe
        return q1, q2

    def decode(self, out: torch.Tensor | None = None, kind: str = "bf16") -> torch.Tensor:
        """Packed streams -> int8 codes or bf16 weights, [out_f, in_f]."""
        dtype = {"bf16": torch.bfloat16, "codes": torch.int8}[kind]
        if out is None:
            out = torch.empty(self.N, dtype=dtype, device=self.device)
        flat = out.reshape(-1)
        if flat.dtype != dtype or flat.numel() < self.N or not flat.is_contiguous():
            raise ValueError("decode output must be a contiguous tensor of the right dtype and size")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_decode(C.byref(self.struct), self.blk_q1.data_ptr(), self.blk_q2.data_ptr(),
                                             flat.data_ptr(), 0 if kind == "codes" else 1,
                                             _lib.stream_ptr(self.device)))
        return flat[: self.N].view(self.out_f, self.in_f)

    def scratch(self, m_rows: int) -> torch.Tensor:
        s = self._scratch.get(m_rows)
        if s is None:
            nbytes = _lib.lib().ixb_gemv_scratch_bytes(self.out_f, self.in_f, m_rows)
            s = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            self._scratch[m_rows] = s
        return s

    def gemv(self, x: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
             out_dtype=torch.bfloat16) -> torch.Tensor:
        """y[M, out_f] = x[M, in_f] @ W.T with W decoded on the fly (1 <= M <= 8)."""
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
        s = self.scratch(m)
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_gemv(C.byref(self.struct), self.blk_q1.data_ptr(), self.blk_q2.data_ptr(),
                                           x2.data_ptr(), m, None if bias is None else bias.data_ptr(),
                                           out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
                                           s.data_ptr(), s.numel(), _lib.stream_ptr(self.device)))
        return out

    def gemm(self, x: torch.Tensor, bias: torch.Tensor | None = None, out: torch.Tensor | None = None,
             out_dtype=torch.bfloat16) -> torch.Tensor:
        """y[M, out_f] = x[M, in_f] @ W.T on the tensor cores, 1 <= M <= 64, in_f % 1024 == 0."""
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
        key = ("gemm", m)
        s = self._scratch.get(key)
        if s is None:
            nbytes = _lib.lib().ixb_gemm_scratch_bytes(self.out_f, self.in_f, m)
            if nbytes == 0:
                raise _lib.IxbError(f"tensor-core gemm needs in_f % 1024 == 0 (in_f={self.in_f})")
            s = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            self._scratch[key] = s
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_gemm(C.byref(self.struct), self.blk_q1.data_ptr(), self.blk_q2.data_ptr(),
                                           x2.data_ptr(), m, None if bias is None else bias.data_ptr(),
                                           out.data_ptr(), 1 if out.dtype == torch.float32 else 0,
                                           s.data_ptr(), s.numel(), _lib.stream_ptr(self.device)))
        return out
