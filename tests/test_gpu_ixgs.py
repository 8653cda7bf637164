"""Sibling group-scale format (ixgs) through this library: bit-exact against the reference's own decode (golden
fixture) and against the oracle on a larger seeded tensor; the module's forward against a dense matmul."""
import os

import numpy as np
import pytest
import torch

from oracle import ixb_oracle as O

pytestmark = pytest.mark.gpu


def torch_dict(d):
    return {"out_f": int(d["out_f"]), "in_f": int(d["in_f"]), "N": int(d["out_f"]) * int(d["in_f"]),
            "group_size": int(d["group_size"]), "counts": [int(c) for c in d["counts"]],
            "group_scales": torch.from_numpy(np.ascontiguousarray(d["group_scales"]).view(np.int16)).view(torch.float16),
            "b1": torch.from_numpy(d["b1"]), "b2": torch.from_numpy(d["b2"]), "l1": torch.from_numpy(d["l1"]),
            "l2": torch.from_numpy(d["l2"]), "l3": torch.from_numpy(d["l3"]), "total_bytes": int(d["total_bytes"])}


def test_group_scale_decode_golden(golden_dir):
    from ixrun_b200.ixgs import decode_weight_triton

    d = np.load(os.path.join(golden_dir, "ixgs_48x320.npz"))
    w = decode_weight_triton(torch_dict(d))
    got = w.cpu().view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(got, d["decoded"])


def test_group_scale_decode_against_the_oracle_and_linear():
    """A larger tensor packed in the group-scale way by this test (codes within -15 .. 16, fp16 scale per 64 elements),
    streams built by the oracle's packer."""
    from ixrun_b200.ixgs import Int8GSLinear, decode_weight_triton

    out_f, in_f, group = 256, 1024, 64
    rng = np.random.default_rng(7)
    codes = np.clip(np.rint(rng.laplace(0.0, 3.0, size=out_f * in_f)), -15, 15).astype(np.int8)
    p = O.pack_codes(codes, out_f, in_f, int(O.f32_to_bf16_bits(np.array([1.0], dtype=np.float32))[0]))
    scales = (rng.random(out_f * in_f // group).astype(np.float32) * 0.01 + 1e-4).astype(np.float16)
    d = {"out_f": out_f, "in_f": in_f, "group_size": group, "counts": p["counts"],
         "group_scales": scales.view(np.uint16), "b1": p["bitmaps"][0], "b2": p["bitmaps"][1],
         "l1": p["streams"][0], "l2": p["streams"][1], "l3": p["streams"][2], "total_bytes": 0}
    ref = O.ixgs_decode_bf16(d)
    pt = torch_dict(d)
    w = decode_weight_triton(pt)
    assert np.array_equal(w.cpu().view(torch.int16).numpy().view(np.uint16), ref)
    lin = Int8GSLinear(pt, bias=torch.randn(out_f).bfloat16())
    x = torch.randn(3, in_f, device="cuda").bfloat16()
    y = lin(x)
    want = torch.nn.functional.linear(x, w, lin._bias)
    assert torch.equal(y, want)
    assert torch.equal(Int8GSLinear(pt, cache="none")(x), torch.nn.functional.linear(x, w))
