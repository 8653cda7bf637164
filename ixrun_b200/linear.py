"""Cached packed linear + model walker (API of ixrun/linear.py)."""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .config import MIN_LINEAR_ELEMS, SKIP_PATTERNS
from .packed import DevicePacked
from .quantize import int8x_quantize

__all__ = ["Int8XLinear", "deploy_model", "iter_quantizable_linears"]


def iter_quantizable_linears(model: nn.Module):
    """(name, module) of every nn.Linear that gets packed: large enough and not
    an embedding / head (rules of ixrun/linear.py:25-34)."""
    for name, mod in model.named_modules():
        if isinstance(mod, nn.Linear) and mod.weight.numel() >= MIN_LINEAR_ELEMS \
                and not any(s in name for s in SKIP_PATTERNS):
            yield name, mod


def _set_parent_child(model: nn.Module, dotted_name: str, new_module: nn.Module):
    *path, leaf = dotted_name.split(".")
    parent = model
    for p in path:
        parent = getattr(parent, p)
    setattr(parent, leaf, new_module)


class Int8XLinear(nn.Module):
    """nn.Linear backed by an INT8-X packed weight (ixrun/linear.py:45-100).

    cache='full' decodes once at construction and keeps the bf16 weight;
    cache='none' keeps only the packed streams on the device and decodes on
    every forward.  `use_triton` is accepted for signature compatibility: the
    decode always runs on the CUDA kernel.
    """

    def __init__(self, packed: dict, bias=None, cache: str = "full", use_triton: bool = True):
        super().__init__()
        if cache not in ("full", "none"):
            raise ValueError("cache must be 'full' or 'none'")
        self.out_features = packed["out_f"]
        self.in_features = packed["in_f"]
        self.packed = packed
        self.use_triton = use_triton
        self._cache = cache
        if bias is not None:
            self.register_buffer("_bias_buf", bias.detach().clone().cuda())
        else:
            self._bias_buf = None
        dp = DevicePacked(packed)
        if cache == "full":
            self._w = dp.decode(kind="bf16")
            self._dp = None          # packed streams are not kept on the device
        else:
            self._w = None
            self._dp = dp

    def _decode(self, device=None):
        return self._dp.decode(kind="bf16") if self._dp is not None else self._w

    def forward(self, x):
        w = self._w if self._cache == "full" else self._decode()
        bias = self._bias_buf.to(x.dtype) if self._bias_buf is not None else None
        return F.linear(x, w.to(x.dtype) if w.dtype != x.dtype else w, bias)

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, "
                f"levels={self.packed['level_bits']}, bpw={self.packed['bits_per_weight']:.2f}")


@torch.no_grad()
def deploy_model(model: nn.Module, level_bits=(3, 5, 8), cache: str = "full",
                 use_triton: bool = True, verbose: bool = True) -> dict:
    """Replace every quantisable Linear by Int8XLinear, in place; returns the
    stats dict of ixrun/linear.py:104-145."""
    targets = list(iter_quantizable_linears(model))
    total_bytes = n_elems = 0
    counts = [0, 0, 0]
    for name, mod in targets:
        packed = int8x_quantize(mod.weight.data, level_bits)
        bias = mod.bias.data if mod.bias is not None else None
        _set_parent_child(model, name, Int8XLinear(packed, bias=bias, cache=cache, use_triton=use_triton))
        total_bytes += packed["total_bytes"]
        n_elems += packed["N"]
        counts = [a + b for a, b in zip(counts, packed["counts"])]
    stats = {
        "n_layers": len(targets),
        "total_bytes": total_bytes,
        "n_elems": n_elems,
        "counts": counts,
        "bits_per_weight": (total_bytes * 8) / max(n_elems, 1),
        "compression_vs_bf16": (n_elems * 2) / max(total_bytes, 1),
    }
    if verbose:
        n = max(sum(counts), 1)
        print(f"[deploy] {stats['n_layers']} layers | {total_bytes / 1e6:.0f}MB packed "
              f"({stats['compression_vs_bf16']:.2f}x vs bf16) | bpw={stats['bits_per_weight']:.2f} | "
              f"L1={counts[0] / n * 100:.1f}% L2={counts[1] / n * 100:.1f}% L3={counts[2] / n * 100:.1f}%",
              flush=True)
    return stats
