"""Seeded synthetic weights with the value distribution of packed LLM layers.

Codes are round(Laplace(0, b)) clipped to +-127 with one element forced to
+-127; W = bf16(code * 2**-9) is exactly representable, so quantising W returns
the codes and a power-of-two scale.  With b = 4.4 about 55 % / 42 % / 3 % of
the codes fall in levels 1 / 2 / 3 (5.44 bit per weight packed).
"""
from __future__ import annotations

import numpy as np
import torch

SCALE_EXP2 = -9


def laplace_codes(out_f: int, in_f: int, seed: int, b: float = 4.4) -> np.ndarray:
    rng = np.random.default_rng(seed)
    n = out_f * in_f
    c = np.clip(np.rint(rng.laplace(0.0, b, size=n)), -127, 127).astype(np.int8)
    pos = int(rng.integers(0, n))
    c[pos] = 127 if rng.integers(0, 2) else -127
    return c


def synthetic_packed(out_f: int, in_f: int, seed: int) -> dict:
    """Packed dict of a synthetic [out_f, in_f] layer (scale 2**-9)."""
    from .quantize import pack_codes

    codes = laplace_codes(out_f, in_f, seed)
    scale = torch.tensor(2.0 ** SCALE_EXP2, dtype=torch.bfloat16)
    return pack_codes(codes, scale, out_f, in_f)


def codes_to_weight(codes: np.ndarray, out_f: int, in_f: int) -> torch.Tensor:
    """bf16 weight whose quantisation gives `codes` back."""
    w = torch.from_numpy(codes.astype(np.float32) * np.float32(2.0 ** SCALE_EXP2))
    return w.view(out_f, in_f).bfloat16()
