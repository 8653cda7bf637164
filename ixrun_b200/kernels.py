"""Decode entry points with the reference's names and argument meaning
(ixrun/triton_kernels.py), backed by the CUDA library.

There is no scatter fallback: without a CUDA device, or for a scheme other than
(3, 5, 8), these functions raise.
"""
from __future__ import annotations

import torch

from .config import RANK_BLOCK
from .packed import DevicePacked

__all__ = ["decode_weight", "decode_weight_triton", "decode_codes", "precompute_block_offsets"]


def _device_packed(packed, device=None) -> DevicePacked:
    if isinstance(packed, DevicePacked):
        return packed
    return DevicePacked(packed, device)


def precompute_block_offsets(packed, blk: int = RANK_BLOCK, device=None):
    """(b1_blk, b2_blk): number of level-1 / level-2 elements in blocks [0, k).

    Same result as ixrun/triton_kernels.py:180-220, computed on the GPU; any
    block size is accepted (the reference needs N % blk == 0).
    """
    dp = _device_packed(packed, device)
    n_blk = (dp.N + blk - 1) // blk
    if blk == RANK_BLOCK:
        return dp.blk_q1, dp.blk_q2
    return dp.prefix_tables(blk, n_blk)


@torch.no_grad()
def decode_weight(packed, device=None, dtype=torch.bfloat16, out: torch.Tensor | None = None) -> torch.Tensor:
    """Packed dict -> bf16 weight [out_f, in_f] (ixrun/triton_kernels.py:224-259)."""
    dp = _device_packed(packed, device)
    w = dp.decode(out=out, kind="bf16")
    return w if dtype == torch.bfloat16 else w.to(dtype)


# drop-in name of the reference entry point
decode_weight_triton = decode_weight


@torch.no_grad()
def decode_codes(packed, device=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """Packed dict -> the int8 codes [out_f, in_f] the quantiser produced."""
    return _device_packed(packed, device).decode(out=out, kind="codes")
