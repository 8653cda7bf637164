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

__all__ = ["shard_bounds", "shard_codes", "shard_packed", "RowParallelLinear", "ColumnParallelLinear"]


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
    """Columns of the layer owned by this rank: fp32 partial sums, one
    all-reduce, then the bf16 rounding and the (replicated) bias."""

    def __init__(self, packed_shard: dict, bias=None, group=None):
        super().__init__()
        from .packed import DevicePacked

        self.dp = DevicePacked(packed_shard)
        self.out_features, self.in_features = self.dp.out_f, self.dp.in_f
        self.group = group
        self.bias = None if bias is None else bias.detach().to(self.dp.device, torch.bfloat16)

    def forward(self, x_shard):
        rows = x_shard.numel() // self.in_features
        y32 = self.dp.gemv(x_shard.reshape(rows, self.in_features), out_dtype=torch.float32)
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            dist.all_reduce(y32, group=self.group)
        y = y32.to(torch.bfloat16)
        if self.bias is not None:
            y = y + self.bias
        return y.view(x_shard.shape[:-1] + (self.out_features,))
