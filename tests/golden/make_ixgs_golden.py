"""Golden fixture for the sibling group-scale format (ixgs): written by running the REFERENCE's own Python code
(ixgs.quantize.int8gs_quantize, ixgs.quantize.decode_weight_scatter) on seeded inputs.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_ixgs_golden.py /path/to/reference

The fixture (``ixgs_48x320.npz``) is committed; tests only read it.  bf16 / fp16 tensors are stored as uint16 bits.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_ixgs_golden.py <path to a checkout of the reference (dfytensor/ixrun)>")
sys.path.insert(0, sys.argv[1])

from ixgs.quantize import decode_weight_scatter, int8gs_quantize  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main():
    g = torch.Generator().manual_seed(123)
    out_f, in_f = 48, 320
    w = torch.randn(out_f, in_f, generator=g) * 0.02
    w[torch.rand(out_f, in_f, generator=g) < 0.01] *= 8.0           # heavy tail: groups with very different scales
    w[5, :64] = 0.0                                                    # an all-zero group (scale clamps to 1e-10 -> fp16 0)
    w = w.bfloat16()
    p = int8gs_quantize(w)
    dec = decode_weight_scatter(p, device="cpu")
    np.savez_compressed(os.path.join(HERE, "ixgs_48x320.npz"),
                        out_f=out_f, in_f=in_f, group_size=p["group_size"], counts=np.array(p["counts"], dtype=np.int64),
                        group_scales=bits(p["group_scales"]), b1=p["b1"].numpy(), b2=p["b2"].numpy(), l1=p["l1"].numpy(),
                        l2=p["l2"].numpy(), l3=p["l3"].numpy(), total_bytes=p["total_bytes"], w=bits(w), decoded=bits(dec))
    print("ixgs_48x320.npz: counts", p["counts"], "bits/weight", round(p["bits_per_weight"], 3))


if __name__ == "__main__":
    main()
