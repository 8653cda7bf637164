"""Tensor-parallel sharding of packed linears (no counterpart in the
single-GPU reference; parity is defined against the unsharded result).

Column-parallel layers (q/k/v, gate, up) split the output rows and need no
communication; row-parallel layers (o_proj, down_proj) split `in_f` and their
fp32 partial outputs are summed with one all-reduce.  A shard is a slice of the
*unsharded* int8 codes re-packed with the *unsharded* scale, so every shard
decodes to exactly the slice of the full tensor's decode.
"""
from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist

from .quantize import pack_codes

__all__ = ["shard_bounds", "shard_codes", "shard_packed", "RowParallelLinear", "ColumnParallelLinear", "PeerAllReduce"]


def shard_bounds(n: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """[lo, hi) of `rank`'s contiguous share of n items, in units of `multiple`."""
    if n % (world * multiple):
        raise ValueError(f"{n} is not divisible into {world} shards of a multiple of {multiple}")
    step = n // world
    return rank * step, (rank + 1) * step


def shard_codes(codes, out_f: int, in_f: int, world: int, rank: int, mode: str, sections=None) -> np.ndarray:
    """Slice of the [out_f, in_f] code matrix owned by `rank`.

    mode 'row'    : columns [lo, hi) of every row (row-parallel linear; in_f/world must be a multiple of 32)
    mode 'column' : rows [lo, hi); with `sections` (e.g. the q|k|v row counts of a fused projection) every
                    section is split on its own and the pieces are concatenated in section order
    """
    c = codes.detach().cpu().numpy() if isinstance(codes, torch.Tensor) else np.asarray(codes)
    c = c.reshape(out_f, in_f)
    if mode == "row":
        lo, hi = shard_bounds(in_f, world, rank, 32)
        return np.ascontiguousarray(c[:, lo:hi])
    if mode == "column":
        secs = [out_f] if sections is None else list(sections)
        if sum(secs) != out_f:
            raise ValueError("sections must sum to out_f")
        parts, base = [], 0
        for n in secs:
            lo, hi = shard_bounds(n, world, rank)
            parts.append(c[base + lo: base + hi])
            base += n
        return np.ascontiguousarray(np.concatenate(parts, axis=0))
    raise ValueError("mode must be 'row' or 'column'")


def shard_packed(codes, scale: torch.Tensor, out_f: int, in_f: int, world: int, rank: int, mode: str,
                 sections=None) -> dict:
    """Packed dict of `rank`'s shard (scale of the unsharded tensor)."""
    s = shard_codes(codes, out_f, in_f, world, rank, mode, sections)
    return pack_codes(s.reshape(-1), scale, s.shape[0], s.shape[1])


class ColumnParallelLinear(torch.nn.Module):
    """Rows of the layer owned by this rank; output stays sharded."""

    def __init__(self, packed_shard: dict, bias_shard=None):
        super().__init__()
        from .engine import StreamingLinear

        self.inner = StreamingLinear(packed_shard, bias=bias_shard)

    def forward(self, x):
        return self.inner(x)


class RowParallelLinear(torch.nn.Module):
    """Columns of the layer owned by this rank, on the resident P6 layout.  With a ``PeerAllReduce`` the fp32
    partial sums leave the GEMV's epilogue as peer stores into every rank's buffer and one small kernel adds them up
    (+ the replicated bias, after the bf16 rounding as in ixrun/engine.py:166-168); without one (or for more than 8
    rows) the partial sums go through an NCCL all-reduce."""

    def __init__(self, packed_shard: dict, bias=None, group=None, allreduce: "PeerAllReduce | None" = None):
        super().__init__()
        from .p6 import P6Packed

        self.res = P6Packed.from_packed(packed_shard)
        self.out_features, self.in_features = self.res.out_f, self.res.in_f
        self.group = group
        self.ar = allreduce
        self.bias = None if bias is None else bias.detach().to(self.res.device, torch.bfloat16)

    def forward(self, x_shard):
        rows = x_shard.numel() // self.in_features
        x2 = x_shard.reshape(rows, self.in_features)
        if self.ar is not None and rows <= 8:
            n = self.res.gemv_push(x2, self.ar)
            y = torch.empty(rows, self.out_features, dtype=torch.bfloat16, device=x2.device)
            bias = None if self.bias is None else self.bias.expand(rows, -1).contiguous()
            self.ar.finish(n, y, bias=bias)
            return y.view(x_shard.shape[:-1] + (self.out_features,))
        if rows <= 8:
            y32 = self.res.gemv(x2, out_dtype=torch.float32)
        else:
            y32 = torch.nn.functional.linear(x2, self.res.decode(kind="bf16")).float()
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y32, group=self.group)
        y = y32.to(torch.bfloat16)
        if self.bias is not None:
            y = y + self.bias
        return y.view(x_shard.shape[:-1] + (self.out_features,))


class PeerAllReduce:
    """Sum of a short fp32 vector over the ranks in one kernel over peer memory (``ixb_allreduce``).

    Every rank allocates one symmetric-memory buffer, exchanges the peer pointers once, and from then on a call is a
    single launch of this library on the current stream: peer stores of the data, every word marked with the call
    number, a bounded wait for the marks, a local sum in rank order.  It can be captured in a CUDA graph together
    with the GEMVs around it.  The sending half can also run inside the GEMV (``P6Packed.gemv_push``), followed by
    ``finish``.  world_size 1 works on one GPU (the buffer is the rank's own).
    """

    def __init__(self, n_max: int, device, group=None):
        import ctypes as C

        import torch.distributed as dist

        from . import _lib

        self.n_max = int(n_max)
        self.device = torch.device(device)
        self.world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        L = _lib.lib()
        nbytes = int(L.ixb_allreduce_bytes(self.world, self.n_max))
        if nbytes == 0:
            raise ValueError(f"unsupported all-reduce geometry: world={self.world}, n_max={self.n_max}")
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem

            self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            self.buf.zero_()
            grp = group if group is not None else dist.group.WORLD
            self._hdl = symm_mem.rendezvous(self.buf, group=grp)
            ptrs = [int(p) for p in self._hdl.buffer_ptrs]
            torch.cuda.synchronize(self.device)
            dist.barrier(group)                      # every rank's buffer is zero before anyone's first call
        else:
            self.buf = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
            ptrs = [self.buf.data_ptr()]
        self._ptrs = (C.c_void_p * self.world)(*ptrs)
        self._nbytes = nbytes

    @classmethod
    def loopback(cls, n_max: int, device, world: int, rank: int = 0, share: "PeerAllReduce | None" = None) -> "PeerAllReduce":
        """One GPU playing rank `rank` of `world`: every peer pointer is this rank's own buffer.  With world > 1 the
        other ranks never send, so a wait runs out -- the way to exercise the bounded wait and the error word on one
        GPU (set a short limit with ``set_spin_limit`` first).  With `share` (another loopback object of the same
        geometry) the two use one buffer: the ranks' sending halves (``P6Packed.gemv_push``) can then be run one after
        the other on one GPU, each as its own rank, before a single finishing call adds them up."""
        import ctypes as C

        from . import _lib

        self = cls.__new__(cls)
        self.n_max, self.device, self.world, self.rank = int(n_max), torch.device(device), int(world), int(rank)
        nbytes = int(_lib.lib().ixb_allreduce_bytes(self.world, self.n_max))
        if nbytes == 0:
            raise ValueError(f"unsupported all-reduce geometry: world={world}, n_max={n_max}")
        if share is not None and (share.world, share.n_max) != (self.world, self.n_max):
            raise ValueError("shared loopback objects must have the same geometry")
        self.buf = share.buf if share is not None else torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self._ptrs = (C.c_void_p * self.world)(*([self.buf.data_ptr()] * self.world))
        self._nbytes = nbytes
        self._loopback = True
        return self

    @staticmethod
    def set_spin_limit(polls: int) -> int:
        """Polls after which a wait gives up (process-wide; 0 restores the default); returns the previous value."""
        from . import _lib

        return int(_lib.lib().ixb_allreduce_spin_limit(int(polls)))

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, bias: torch.Tensor | None = None,
                 out_dtype=torch.bfloat16) -> torch.Tensor:
        from . import _lib

        if x.dtype != torch.float32 or not x.is_contiguous() or x.numel() > self.n_max or x.numel() % 4:
            raise ValueError("all-reduce input must be a contiguous fp32 tensor of a multiple of 4, at most n_max, values")
        if out is None:
            out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        elif out.dtype not in (torch.bfloat16, torch.float32) or out.numel() != x.numel() or not out.is_contiguous():
            raise ValueError("all-reduce output must be a contiguous bf16/fp32 tensor of the input's size")
        if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != x.numel()):
            raise ValueError("bias must be bf16 with one value per element")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_allreduce(x.data_ptr(), x.numel(), self._ptrs, self.rank, self.world, self.n_max,
                                                None if bias is None else bias.data_ptr(), out.data_ptr(),
                                                1 if out.dtype == torch.float32 else 0, _lib.stream_ptr(self.device)))
        return out

    def finish(self, n: int, out: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
        """Second half of the exchange after ``P6Packed.gemv_push``: wait for every rank's `n` marked words of this
        call, add them in rank order (+ bias), write `out` (bf16 or fp32, n elements)."""
        from . import _lib

        if n % 4 or n > self.n_max or out.numel() != n or not out.is_contiguous() or out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("finish needs n (a multiple of 4, at most n_max) and a contiguous bf16/fp32 output of n elements")
        if bias is not None and (bias.dtype != torch.bfloat16 or bias.numel() != n):
            raise ValueError("bias must be bf16 with one value per element")
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().ixb_allreduce_finish(self._ptrs, self.rank, self.world, n, self.n_max,
                                                       None if bias is None else bias.data_ptr(), out.data_ptr(),
                                                       1 if out.dtype == torch.float32 else 0, _lib.stream_ptr(self.device)))
        return out

    def reset(self, group=None):
        """After a wait gave up (``timed_out()``): zero this rank's buffer (slots, call counters, error word) and meet
        the other ranks at a barrier, as before the first call.  Every rank must call it at the same point, with
        nothing of the exchange in flight."""
        torch.cuda.synchronize(self.device)
        self.buf.zero_()
        torch.cuda.synchronize(self.device)
        if self.world > 1 and not getattr(self, "_loopback", False):
            dist.barrier(group)

    def timed_out(self) -> bool:
        """True if a wait inside any call so far gave up (the results since then are not to be trusted)."""
        return bool(self._err_word().item() != 0)

    def _err_word(self):
        # layout of the buffer: slots [2][world][n_max] x 8 bytes, call counters (one per 256 values), error word
        counters = (self.n_max + 255) // 256
        off = 2 * self.world * self.n_max * 8 + counters * 4
        return self.buf[off:off + 4].view(torch.int32)
