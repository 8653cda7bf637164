"""GPU quantiser/packer against the reference fixtures and the host packer: bit-exact."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

CASES = ["core_128x256", "heavy_64x1024", "allzero_8x128", "ternary_16x128", "laplace_32x2048", "ragged_10x96"]


def bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


@pytest.mark.parametrize("name", CASES)
def test_gpu_quantize_matches_reference_fixture(golden_dir, name):
    from ixrun_b200.gpu_pack import int8x_quantize_gpu, quantize_pack_gpu

    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    w = bf16(g["w_bits"]).cuda()
    p = int8x_quantize_gpu(w)
    assert p["counts"] == [int(c) for c in g["counts"]] and p["total_bytes"] == int(g["total_bytes"][0])
    assert int(p["scale"].view(torch.int16).item()) & 0xFFFF == int(g["scale_bits"][0])
    for t, k in zip(p["bitmaps"] + p["streams"], ["b1", "b2", "l1", "l2", "l3"]):
        assert np.array_equal(t.numpy(), g[k]), k
    dp, codes = quantize_pack_gpu(w, return_codes=True)
    assert np.array_equal(codes.cpu().numpy().reshape(-1), g["codes"])
    # tables written by the packer equal the ones derived from the streams, and the result decodes back
    q1, q2 = dp.prefix_tables(1024)
    assert torch.equal(q1, dp.blk_q1) and torch.equal(q2, dp.blk_q2)
    assert np.array_equal(dp.decode(kind="codes").cpu().numpy().reshape(-1), g["codes"])


@pytest.mark.parametrize("out_f,in_f", [(5120, 5120), (96, 2176), (33, 96), (1, 32), (7, 1000)])
def test_gpu_pack_matches_host_packer(out_f, in_f):
    from ixrun_b200.gpu_pack import pack_codes_gpu, quantize_pack_gpu
    from ixrun_b200.quantize import int8x_quantize, pack_codes
    from ixrun_b200.synth import codes_to_weight, laplace_codes

    codes = laplace_codes(out_f, in_f, seed=out_f + in_f)
    scale = torch.tensor(0.0037, dtype=torch.bfloat16)
    host = pack_codes(codes, scale, out_f, in_f)
    dp = pack_codes_gpu(torch.from_numpy(codes).cuda(), scale, out_f, in_f)
    for a, b in zip([dp.b1, dp.b2, dp.l1, dp.l2, dp.l3], host["bitmaps"] + host["streams"]):
        assert torch.equal(a.cpu(), b)
    assert dp.counts == host["counts"] and dp.total_bytes == host["total_bytes"]
    # from a weight: same as the host quantiser, scale included
    w = (torch.randn(out_f, in_f) * 0.02).bfloat16()
    h2 = int8x_quantize(w)
    d2 = quantize_pack_gpu(w.cuda())
    assert torch.equal(d2.scale.cpu(), h2["scale"])
    for a, b in zip([d2.b1, d2.b2, d2.l1, d2.l2, d2.l3], h2["bitmaps"] + h2["streams"]):
        assert torch.equal(a.cpu(), b)
    if in_f % 32 == 0:
        x = torch.randn(1, in_f).bfloat16().cuda()
        from ixrun_b200.packed import DevicePacked

        assert torch.equal(d2.gemv(x), DevicePacked(h2).gemv(x))
