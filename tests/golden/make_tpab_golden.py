"""Golden fixtures for the TPAB tile format: written by running the REFERENCE's own Python code
(ixrun.tpab.encode_tpab / decode_tpab_ref) on seeded inputs.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_tpab_golden.py /path/to/reference

The fixtures (``tpab_*.npz``) are committed; tests only read them.  bf16 / fp16 tensors are stored as uint16 bits.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2:
    raise SystemExit("usage: make_tpab_golden.py <path to a checkout of the reference (dfytensor/ixrun)>")
sys.path.insert(0, sys.argv[1])

from ixrun.tpab import decode_tpab_ref, encode_tpab  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def case(name, out_f, in_f, seed, snr_db):
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(out_f, in_f, generator=g) * 0.02
    # column tiles of different character, so that the per-tile search picks different widths: two-valued, uniform,
    # Gaussian, heavy-tailed
    for ct in range(in_f // 64):
        blk = w[:, ct * 64:(ct + 1) * 64]
        kind = ct % 4
        if kind == 0:
            blk.copy_(torch.sign(blk) * 0.02)
        elif kind == 1:
            blk.copy_((torch.rand(blk.shape, generator=g) - 0.5) * 0.05)
        elif kind == 3:
            blk[torch.rand(blk.shape, generator=g) < 0.02] *= 12.0
    w = w.bfloat16()
    p = encode_tpab(w, snr_target_db=snr_db)
    dec = decode_tpab_ref(p)
    x = torch.randn(in_f, generator=g).bfloat16()
    y = torch.nn.functional.linear(x.float()[None], dec.float())[0]
    np.savez_compressed(os.path.join(HERE, name + ".npz"),
                        out_f=out_f, in_f=in_f, tile_r=p["tile_r"], T=p["T"], n_per=p["n_per"], bits=p["bits"].numpy(),
                        scales=bits(p["scales"]), goff=p["goff"].numpy(), gbase_bit=p["gbase_bit"].numpy(),
                        body=torch.cat(p["bodies"]).numpy(), ol_t=p["ol_t"].numpy(), ol_l=p["ol_l"].numpy(),
                        ol_val=bits(p["ol_val"]), total_bytes=p["total_bytes"], decoded=bits(dec), x=bits(x), y=y.numpy())
    widths = {int(b): int((p["bits"] == b).sum()) for b in (2, 3, 4, 5, 6)}
    print(name, "tile_r", p["tile_r"], "widths", widths, "outliers", p["n_outliers"], "bpw", round(p["bpw"], 3))


if __name__ == "__main__":
    case("tpab_128x256", 128, 256, 11, 20.0)
    case("tpab_48x192", 48, 192, 12, 24.0)
    case("tpab_64x512", 64, 512, 13, 14.0)
    case("tpab_64x128", 64, 128, 14, 30.0)
