"""Generate the golden fixtures in this folder by running the REFERENCE's own
Python code (dfytensor/ixrun) on seeded inputs.

Run once, in a container where the reference checkout is importable:

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

The fixtures (``*.npz`` / ``big_hashes.json``) are committed; the tests only read
them, so nothing at test time needs the reference.  bf16 tensors are stored as
uint16 bit patterns.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) < 2 and "IXRUN_REFERENCE" not in os.environ:
    raise SystemExit("usage: make_golden.py <path to a checkout of the reference (dfytensor/ixrun)>")
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ["IXRUN_REFERENCE"]
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from ixrun.bitpack import pack_bits_stream, unpack_bits_stream  # noqa: E402
from ixrun.fused import compute_row_prefixes  # noqa: E402
from ixrun.quantize import compute_positions, decode_to_weight, int8x_quantize  # noqa: E402
from ixrun.triton_kernels import decode_weight_scatter, precompute_block_offsets  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def pack_case(name: str, w: torch.Tensor, chunk: int | None, x_seed: int = 7, m_rows: int = 3):
    """Quantise with the reference, decode with the reference, save everything."""
    assert w.dtype == torch.bfloat16
    p = int8x_quantize(w, (3, 5, 8))
    out_f, in_f, n = p["out_f"], p["in_f"], p["N"]
    w_dec = decode_weight_scatter(p, device="cpu")
    w_dec2 = decode_to_weight(p, device="cpu")
    assert torch.equal(w_dec, w_dec2)
    # ground-truth codes exactly like the reference's own test does
    # (tests/test_core.py:45-50)
    scale_f32 = w.abs().max().clamp(min=1e-8) / 127.0
    codes = (w.float() / scale_f32).round().clamp(-127, 127).to(torch.int8).reshape(-1)
    w_gt = (codes.float() * p["scale"].float()).to(torch.bfloat16).reshape(out_f, in_f)
    assert torch.equal(w_gt, w_dec), name
    d = {
        "w_bits": bits(w),
        "scale_bits": bits(p["scale"].reshape(1)),
        "codes": codes.numpy(),
        "b1": p["bitmaps"][0].numpy(),
        "b2": p["bitmaps"][1].numpy(),
        "l1": p["streams"][0].numpy(),
        "l2": p["streams"][1].numpy(),
        "l3": p["streams"][2].numpy(),
        "counts": np.array(p["counts"], dtype=np.int64),
        "total_bytes": np.array([p["total_bytes"]], dtype=np.int64),
        "w_dec_bits": bits(w_dec),
    }
    pos = compute_positions(p)
    d["pos_counts"] = np.array([len(q) for q in pos], dtype=np.int64)
    d["pos_l3"] = pos[2].numpy()
    if n % 1024 == 0:
        a, c = precompute_block_offsets(p, 1024, device="cpu")
        d["blk_q1"], d["blk_q2"] = a.numpy(), c.numpy()
    q1, q2 = compute_row_prefixes(p)
    d["row_q1"], d["row_q2"] = q1.numpy(), q2.numpy()
    if chunk:
        q1c, q2c = compute_row_prefixes(p, chunk)
        d["chunk"] = np.array([chunk], dtype=np.int64)
        d["chunk_q1"], d["chunk_q2"] = q1c.numpy(), q2c.numpy()
    g = torch.Generator().manual_seed(x_seed)
    x = torch.randn(m_rows, in_f, generator=g).bfloat16()
    y = torch.nn.functional.linear(x.float(), w_dec.float())
    d["x_bits"] = bits(x)
    d["y_f32"] = y.numpy()
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **d)
    print(f"{name}: {out_f}x{in_f} counts={p['counts']} bytes={p['total_bytes']}")


def sha(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    # 1. the reference's own lossless-decode test input (tests/test_core.py:41-43)
    torch.manual_seed(42)
    w = (torch.randn(128, 256) * 0.03).bfloat16()
    pack_case("core_128x256", w, chunk=128)

    # 2. heavy-tail weights as in the reference's kernel parity scripts
    #    (tests/test_fused.py:17-22), small shape with in_f % 512 == 0
    torch.manual_seed(0)
    out_f, in_f = 64, 1024
    base = torch.randn(out_f, in_f) * 0.005
    flat = base.view(-1)
    idx = torch.randperm(flat.numel())[: int(out_f * in_f * 0.04)]
    flat[idx] = torch.randn(len(idx)) * 0.05
    pack_case("heavy_64x1024", base.bfloat16(), chunk=512)

    # 3. all-zero tensor: every element is level 1, B2/L2/L3 are empty
    pack_case("allzero_8x128", torch.zeros(8, 128).bfloat16(), chunk=None)

    # 4. only {0, +-max}: level 2 is empty, level 3 is not
    torch.manual_seed(3)
    w = (torch.randint(-1, 2, (16, 128)).float() * 0.25).bfloat16()
    pack_case("ternary_16x128", w, chunk=64)

    # 5. the benchmark's synthetic distribution (rounded Laplace codes, exact
    #    power-of-two scale): the reference quantiser must give the codes back
    from oracle import ixb_oracle as O

    c = O.laplace_codes(32, 2048, seed=11)
    wb = O.codes_to_weight_bits(c)
    w = torch.from_numpy(wb.view(np.int16).reshape(32, 2048)).view(torch.bfloat16)
    p = int8x_quantize(w, (3, 5, 8))
    assert float(p["scale"]) == 2.0 ** -9
    pack_case("laplace_32x2048", w, chunk=1024)

    # 6. ragged: N not a multiple of 1024, in_f a multiple of 32 only
    torch.manual_seed(5)
    w = (torch.randn(10, 96) * 0.02).bfloat16()
    pack_case("ragged_10x96", w, chunk=32)

    # 7. bit-stream packer (tests/test_core.py:15-35, small sizes)
    torch.manual_seed(0)
    v3 = torch.randint(0, 8, (1000,), dtype=torch.int32)
    v5 = torch.randint(0, 32, (777,), dtype=torch.int32)
    pk3, pk5 = pack_bits_stream(v3, 3), pack_bits_stream(v5, 5)
    assert torch.equal(unpack_bits_stream(pk3, 1000, 3), v3)
    assert torch.equal(unpack_bits_stream(pk5, 777, 5), v5)
    np.savez_compressed(os.path.join(HERE, "bitpack.npz"), v3=v3.numpy(), pk3=pk3.numpy(),
                        v5=v5.numpy(), pk5=pk5.numpy())

    # 8. full-size config-0 tensor (4096x4096): hashes only
    c = O.laplace_codes(4096, 4096, seed=0)
    wb = O.codes_to_weight_bits(c)
    w = torch.from_numpy(wb.view(np.int16).reshape(4096, 4096)).view(torch.bfloat16)
    p = int8x_quantize(w, (3, 5, 8))
    w_dec = decode_weight_scatter(p, device="cpu")
    a, cc = precompute_block_offsets(p, 1024, device="cpu")
    big = {
        "shape": [4096, 4096],
        "seed": 0,
        "counts": p["counts"],
        "total_bytes": p["total_bytes"],
        "scale_bits": int(bits(p["scale"].reshape(1))[0]),
        "sha_codes": sha(c),
        "sha_b1": sha(p["bitmaps"][0].numpy()),
        "sha_b2": sha(p["bitmaps"][1].numpy()),
        "sha_l1": sha(p["streams"][0].numpy()),
        "sha_l2": sha(p["streams"][1].numpy()),
        "sha_l3": sha(p["streams"][2].numpy()),
        "sha_w_dec": sha(bits(w_dec)),
        "sha_blk_q1": sha(a.numpy()),
        "sha_blk_q2": sha(cc.numpy()),
    }
    with open(os.path.join(HERE, "big_hashes.json"), "w") as f:
        json.dump(big, f, indent=1)
    print("big:", big["counts"], big["total_bytes"])


if __name__ == "__main__":
    main()
