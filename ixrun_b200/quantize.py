"""Host-side INT8-X quantiser / packer (deploy time, one-off per tensor).

Produces the same packed dict, key for key and bit for bit, as the reference's
``int8x_quantize`` (ixrun/quantize.py:41-122), so packed caches interoperate.
The packing itself is vectorised with ``numpy.packbits`` instead of the
reference's int64 bit-expansion (ixrun/bitpack.py:13-61).

``pack_codes`` packs already-quantised int8 codes with a given scale; tensor
parallel shards use it so that every shard keeps the scale of the unsharded
tensor (re-quantising a slice would pick a different scale).
"""
from __future__ import annotations

import numpy as np
import torch

DEFAULT_LEVELS = (3, 5, 8)
# largest |code| a level of b bits covers (sign-symmetric, offset-binary)
BIT_TO_THRESHOLD = {1: 0, 2: 1, 3: 3, 4: 7, 5: 15, 6: 31, 7: 63, 8: 127}

__all__ = ["int8x_quantize", "pack_codes", "quantize_codes", "DEFAULT_LEVELS", "BIT_TO_THRESHOLD"]


def _check_levels(level_bits) -> tuple:
    level_bits = tuple(sorted(level_bits))
    if level_bits[-1] != 8:
        raise ValueError("last level must be 8-bit to cover the full int8 range")
    if level_bits != DEFAULT_LEVELS:
        raise ValueError(f"only the (3, 5, 8) scheme is supported, got {level_bits}")
    return level_bits


def _pack_fields(vals: np.ndarray, bits: int) -> np.ndarray:
    """Consecutive `bits`-wide fields, LSB first, into little-endian int32 words."""
    n = vals.size
    if n == 0:
        return np.zeros(0, dtype=np.int32)
    words = (n * bits + 31) // 32
    out = np.zeros(words * 4, dtype=np.uint8)
    step = 1 << 22                      # bound the bit-expansion temporary
    # chunks hold a multiple of 32 values, so every chunk starts on a byte
    for s in range(0, n, step):
        v = vals[s:s + step].astype(np.uint8)
        b = ((v[:, None] >> np.arange(bits, dtype=np.uint8)) & 1).reshape(-1)
        pk = np.packbits(b, bitorder="little")
        o = s * bits // 8
        out[o:o + pk.size] = pk
    return out.view(np.int32)


def _pack_mask(mask: np.ndarray) -> np.ndarray:
    n = mask.size
    if n == 0:
        return np.zeros(0, dtype=np.int32)
    out = np.zeros(((n + 31) // 32) * 4, dtype=np.uint8)
    pk = np.packbits(mask, bitorder="little")
    out[:pk.size] = pk
    return out.view(np.int32)


@torch.no_grad()
def quantize_codes(weight: torch.Tensor):
    """bf16/fp weight -> (int8 codes [out_f*in_f] on CPU, bf16 0-d scale).

    scale = max|W| (floored at 1e-8) / 127, evaluated in the weight's own dtype
    and stored as bf16; code = clamp(round_half_even(float(W) / scale), +-127)
    (ixrun/quantize.py:64-73).
    """
    scale = weight.abs().max().clamp(min=1e-8) / 127.0
    codes = (weight.float() / scale).round().clamp(-127, 127).to(torch.int8).reshape(-1).cpu()
    return codes, scale.detach().cpu().bfloat16().reshape(())


def pack_codes(codes, scale: torch.Tensor, out_f: int, in_f: int, level_bits=DEFAULT_LEVELS) -> dict:
    """int8 codes (+ the tensor's bf16 scale) -> packed dict."""
    level_bits = _check_levels(level_bits)
    c = codes.detach().cpu().numpy() if isinstance(codes, torch.Tensor) else np.asarray(codes)
    c = np.ascontiguousarray(c, dtype=np.int8).reshape(-1)
    n = out_f * in_f
    if c.size != n:
        raise ValueError(f"{c.size} codes for a {out_f}x{in_f} tensor")
    a = np.abs(c.astype(np.int16))
    is1 = a <= BIT_TO_THRESHOLD[3]
    is2 = (~is1) & (a <= BIT_TO_THRESHOLD[5])
    is3 = ~(is1 | is2)
    counts = [int(is1.sum()), int(is2.sum()), int(is3.sum())]
    l1 = _pack_fields((c[is1].astype(np.int16) + 3), 3)
    l2 = _pack_fields((c[is2].astype(np.int16) + 15), 5)
    l3 = (c[is3].astype(np.int16) + 127).astype(np.uint8)
    b1 = _pack_mask(is1)
    b2 = _pack_mask(is2[~is1])           # indexed by rank among non-L1 elements
    total = 2 + 4 * (l1.size + l2.size + b1.size + b2.size) + l3.size
    return {
        "level_bits": level_bits,
        "out_f": out_f,
        "in_f": in_f,
        "N": n,
        "scale": scale.detach().cpu().bfloat16().reshape(()),
        "bitmaps": [torch.from_numpy(b1), torch.from_numpy(b2)],
        "streams": [torch.from_numpy(l1), torch.from_numpy(l2), torch.from_numpy(l3)],
        "counts": counts,
        "total_bytes": total,
        "bits_per_weight": (total * 8) / n,
        "compression_vs_bf16": (n * 2) / total,
    }


@torch.no_grad()
def int8x_quantize(weight: torch.Tensor, level_bits: tuple = DEFAULT_LEVELS) -> dict:
    """Quantise a 2-D weight into an INT8-X packed dict (reference keys)."""
    level_bits = _check_levels(level_bits)
    if weight.dim() != 2:
        raise ValueError("weight must be 2-D (out_features, in_features)")
    out_f, in_f = weight.shape
    codes, scale = quantize_codes(weight)
    return pack_codes(codes, scale, out_f, in_f, level_bits)
