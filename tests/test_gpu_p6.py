"""Resident P6 layout: lossless on the codes, GEMV equal to the oracle."""
import os

import numpy as np
import pytest
import torch

from oracle import ixb_oracle as O

pytestmark = pytest.mark.gpu

SHAPES = [(64, 5120), (48, 5120), (40, 17408), (96, 2176), (7, 4352), (33, 96), (1, 32), (3, 1024), (300, 512),
          (10, 96), (5, 100), (17, 72), (512, 17408), (16, 64)]


def bits_to_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def rel_err(y, ref):
    return float(np.abs(y.astype(np.float64) - ref).max() / max(float(np.abs(ref).max()), 1e-30))


def make(out_f, in_f, seed, codes=None):
    from ixrun_b200.p6 import P6Packed

    if codes is None:
        codes = O.laplace_codes(out_f, in_f, seed)
    scale = torch.tensor(0.00251, dtype=torch.bfloat16)
    return codes, scale, P6Packed(torch.from_numpy(codes).cuda(), scale, out_f, in_f)


@pytest.mark.parametrize("out_f,in_f", SHAPES)
def test_p6_roundtrip_is_lossless(out_f, in_f):
    codes, scale, p6 = make(out_f, in_f, out_f + in_f)
    assert np.array_equal(p6.decode(kind="codes").cpu().numpy().reshape(-1), codes)
    sc_bits = int(scale.view(torch.int16).item()) & 0xFFFF
    w = p6.decode(kind="bf16").cpu().view(torch.int16).numpy().view(np.uint16).reshape(-1)
    assert np.array_equal(w, O.codes_to_bf16(codes, sc_bits))


@pytest.mark.parametrize("out_f,in_f", SHAPES)
@pytest.mark.parametrize("m", [1, 2, 5, 8])
def test_p6_gemv_matches_oracle(out_f, in_f, m):
    codes, scale, p6 = make(out_f, in_f, out_f * 5 + in_f + m)
    sc_bits = int(scale.view(torch.int16).item()) & 0xFFFF
    xb = O.f32_to_bf16_bits(np.random.default_rng(m).standard_normal((m, in_f)).astype(np.float32))
    ref = O.gemm_f32(codes, sc_bits, xb, out_f, in_f).astype(np.float64)
    x = bits_to_bf16(xb).cuda()
    bias = torch.randn(out_f).bfloat16().cuda()
    y32 = p6.gemv(x, out_dtype=torch.float32)
    assert rel_err(y32.cpu().numpy(), ref) < 2e-5
    assert torch.equal(p6.gemv(x), y32.bfloat16())
    assert torch.equal(p6.gemv(x, bias=bias), p6.gemv(x) + bias)
    assert torch.equal(p6.gemv(x, out_dtype=torch.float32), y32)


def test_p6_one_scratch_buffer_serves_layers_of_any_shape():
    """Layers whose row tiles are shared by three or more CTAs, by two, and by none run back to back on ONE scratch
    buffer (the library leaves it all zero after every launch), in both orders, and still match the oracle."""
    from ixrun_b200.p6 import GemvScratch

    shapes = [(16, 17408), (256, 17408), (5120, 2176), (64, 5120), (16, 17408), (5120, 2176), (300, 512)]
    scratch = GemvScratch("cuda")
    cases = []
    for i, (out_f, in_f) in enumerate(shapes):
        codes, scale, p6 = make(out_f, in_f, 100 + i)
        p6.scratch = scratch
        sc_bits = int(scale.view(torch.int16).item()) & 0xFFFF
        xb = O.f32_to_bf16_bits(np.random.default_rng(i).standard_normal((1, in_f)).astype(np.float32))
        cases.append((p6, bits_to_bf16(xb).cuda(), O.gemm_f32(codes, sc_bits, xb, out_f, in_f).astype(np.float64)))
    for order in (range(len(cases)), reversed(range(len(cases)))):
        for i in order:
            p6, x, ref = cases[i]
            assert rel_err(p6.gemv(x, out_dtype=torch.float32).cpu().numpy(), ref) < 2e-5
    assert int(scratch.buf.max().item()) == 0       # every launch left the scratch all zero


def test_p6_extreme_level_mixes_and_from_packed(golden_dir):
    from ixrun_b200.p6 import P6Packed

    out_f, in_f = 8, 1024
    n = out_f * in_f
    rng = np.random.default_rng(0)
    xb = O.f32_to_bf16_bits(rng.standard_normal((2, in_f)).astype(np.float32))
    for codes in (rng.choice(np.r_[-127:-16, 32:128], size=n).astype(np.int8),
                  rng.integers(-16, 32, size=n).astype(np.int8),
                  rng.integers(-3, 4, size=n).astype(np.int8),
                  np.where(np.arange(n) % 2 == 0, 1, 100).astype(np.int8),
                  np.zeros(n, dtype=np.int8)):
        c, scale, p6 = make(out_f, in_f, 0, codes=codes)
        assert np.array_equal(p6.decode(kind="codes").cpu().numpy().reshape(-1), codes)
        sc_bits = int(scale.view(torch.int16).item()) & 0xFFFF
        ref = O.gemm_f32(codes, sc_bits, xb, out_f, in_f).astype(np.float64)
        y = p6.gemv(bits_to_bf16(xb).cuda(), out_dtype=torch.float32).cpu().numpy()
        assert float(np.abs(y - ref).max()) <= 2e-5 * max(float(np.abs(ref).max()), 1e-30)
    # from the reference's packed streams (fixture written by the reference's own quantiser)
    g = dict(np.load(os.path.join(golden_dir, "heavy_64x1024.npz")))
    packed = {"level_bits": (3, 5, 8), "out_f": 64, "in_f": 1024, "N": 65536, "scale": bits_to_bf16(g["scale_bits"]).reshape(()),
              "bitmaps": [torch.from_numpy(g["b1"]), torch.from_numpy(g["b2"])],
              "streams": [torch.from_numpy(g["l1"]), torch.from_numpy(g["l2"]), torch.from_numpy(g["l3"])],
              "counts": [int(c) for c in g["counts"]], "total_bytes": int(g["total_bytes"][0])}
    p6 = P6Packed.from_packed(packed)
    assert np.array_equal(p6.decode(kind="codes").cpu().numpy().reshape(-1), g["codes"])
    y = p6.gemv(bits_to_bf16(g["x_bits"]).cuda(), out_dtype=torch.float32).cpu().numpy()
    assert rel_err(y, g["y_f32"].astype(np.float64)) < 2e-5


@pytest.mark.parametrize("out_f,in_f", [(5120, 17408), (17408, 5120), (5120, 5120), (1024, 5120), (2048, 2048)])
def test_p6_full_size_against_the_oracle(out_f, in_f):
    """The five benchmark shapes at full size, batch 1: the GEMV on the resident layout against the CPU oracle's
    fp32-accumulated product of the same codes, the decoded codes against the codes that were packed; twice for
    reproducibility; 8 rows against the fused kernel on the reference's streams (itself checked against the
    oracle)."""
    from ixrun_b200.p6 import P6Packed
    from ixrun_b200.packed import DevicePacked
    from ixrun_b200.synth import laplace_codes, synthetic_packed

    dp = DevicePacked(synthetic_packed(out_f, in_f, seed=3))
    codes = laplace_codes(out_f, in_f, seed=3)
    p6 = P6Packed.from_packed(dp)
    got = p6.decode(kind="codes")
    assert torch.equal(got, dp.decode(kind="codes"))
    assert np.array_equal(got.cpu().numpy().reshape(-1), codes.reshape(-1))
    sc_bits = int(dp.scale.view(torch.int16).item()) & 0xFFFF
    xb = O.f32_to_bf16_bits(np.random.default_rng(7).standard_normal((1, in_f)).astype(np.float32))
    ref = O.gemm_f32(codes.reshape(-1), sc_bits, xb, out_f, in_f).astype(np.float64)
    y = p6.gemv(bits_to_bf16(xb).cuda(), out_dtype=torch.float32)
    assert rel_err(y.cpu().numpy(), ref) < 2e-5
    assert torch.equal(p6.gemv(bits_to_bf16(xb).cuda(), out_dtype=torch.float32), y)
    x8 = torch.randn(8, in_f, device="cuda").bfloat16()
    ref8 = dp.gemv(x8, out_dtype=torch.float32)
    y8 = p6.gemv(x8, out_dtype=torch.float32)
    assert float((y8 - ref8).abs().max() / ref8.abs().max()) < 2e-5
    assert torch.equal(p6.gemv(x8, out_dtype=torch.float32), y8)
    assert p6.resident_bytes < 1.2 * dp.total_bytes


def test_p6_programmatic_dependent_launch_gives_the_same_result():
    """Back-to-back launches with programmatic dependent launch on (eagerly and replayed from a CUDA graph):
    every launch must still see the activations written just before it and produce the bits of a plain launch."""
    from ixrun_b200.p6 import set_pdl

    out_f, in_f = 512, 5120
    _, _, a = make(out_f, in_f, 11)
    _, _, b = make(in_f, out_f, 12)
    x = torch.randn(1, in_f, device="cuda").bfloat16()
    h_ref = a.gemv(x)
    y_ref = b.gemv(h_ref)
    torch.cuda.synchronize()
    prev = set_pdl(True)
    try:
        h = torch.empty_like(h_ref)
        y = torch.empty_like(y_ref)
        for _ in range(3):
            h.zero_()
            y.zero_()
            a.gemv(x, out=h)
            b.gemv(h, out=y)          # reads what the launch just ahead of it wrote
            assert torch.equal(h, h_ref) and torch.equal(y, y_ref)
        st = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for _ in range(4):
                    a.gemv(x, out=h)
                    b.gemv(h, out=y)
        h.zero_()
        y.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(h, h_ref) and torch.equal(y, y_ref)
    finally:
        set_pdl(prev)


@pytest.mark.parametrize("in_f,rows", [(512, (48, 100, 256)), (5120, (1536, 256, 6, 6)), (2048, (2048, 1024, 1024))])
def test_p6_fused_tensor_gives_every_part_its_own_result(in_f, rows):
    """Tensors fused row-wise keep their own per-tensor scales: decoding gives every part's weights bit for bit, the
    GEMV every part's outputs (the fp32 sums may be added in another order than in the part alone: 1e-6 of the
    largest output; the tile layout and the products are the same)."""
    from ixrun_b200.p6 import P6Packed
    from ixrun_b200.synth import synthetic_packed

    parts = [synthetic_packed(r, in_f, seed=11 + i) for i, r in enumerate(rows)]
    for i, p in enumerate(parts):                       # clearly different scales
        p["scale"] = (p["scale"].float() * (1.0 + 0.37 * i)).to(torch.bfloat16)
    alone = [P6Packed.from_packed(p) for p in parts]
    fused = P6Packed.fuse(parts)
    assert [n for _, n in fused.sections] == list(rows) and all(a % 16 == 0 for a, _ in fused.sections)
    w = fused.decode(kind="bf16")
    c = fused.decode(kind="codes").view(fused.out_f, in_f)
    for (a, n), one in zip(fused.sections, alone):
        assert torch.equal(w[a:a + n], one.decode(kind="bf16"))
        assert torch.equal(c[a:a + n], one.decode(kind="codes").view(n, in_f))
    for m in (1, 3):
        x = torch.randn(m, in_f, device="cuda").bfloat16()
        y = fused.gemv(x, out_dtype=torch.float32)
        yb = fused.gemv(x)
        for (a, n), one in zip(fused.sections, alone):
            ref = one.gemv(x, out_dtype=torch.float32)
            assert float((y[:, a:a + n] - ref).abs().max()) <= 1e-6 * float(ref.abs().max())
            assert float((yb[:, a:a + n].float() - ref).abs().max()) <= 2.0 ** -8 * float(ref.abs().max())
    if len(rows) == 3:
        q, k, v = fused.split(fused.gemv(torch.randn(1, in_f, device="cuda").bfloat16()))
        assert q.numel() == rows[0] and k.numel() == rows[1] and v.numel() == rows[2]


@pytest.mark.parametrize("out_f,in_f,m", [(128, 512, 16), (16, 1024, 64), (40, 5120, 33), (100, 1024, 9), (300, 512, 64),
                                          (512, 5120, 64), (1000, 2176, 17), (3, 3072, 1), (2048, 2048, 32)])
def test_p6_gemm_small_m_against_the_oracle(out_f, in_f, m):
    """tcgen05 GEMM on the resident layout (1..64 rows) against the oracle's fp32 result; bias, bf16 output and
    repeatability; within fp32 summation-order rounding of the GEMV for the rows both take."""
    codes, scale, p6 = make(out_f, in_f, out_f * 3 + m)
    sc_bits = int(scale.view(torch.int16).item()) & 0xFFFF
    xb = O.f32_to_bf16_bits(np.random.default_rng(m).standard_normal((m, in_f)).astype(np.float32))
    ref = O.gemm_f32(codes, sc_bits, xb, out_f, in_f).astype(np.float64)
    x = bits_to_bf16(xb).cuda()
    bias = torch.randn(out_f).bfloat16().cuda()
    y32 = p6.gemm(x, out_dtype=torch.float32)
    assert rel_err(y32.cpu().numpy(), ref) < 2e-5
    assert torch.equal(p6.gemm(x), y32.bfloat16())
    assert torch.equal(p6.gemm(x, bias=bias), p6.gemm(x) + bias)
    assert torch.equal(p6.gemm(x, out_dtype=torch.float32), y32)          # deterministic
    if m <= 8:
        assert rel_err(p6.gemv(x, out_dtype=torch.float32).cpu().numpy(), y32.cpu().numpy().astype(np.float64)) < 2e-5


@pytest.mark.parametrize("out_f,in_f", [(17408, 5120), (5120, 17408)])
@pytest.mark.parametrize("m", [16, 32, 64])
def test_p6_gemm_full_size(out_f, in_f, m):
    """The batched-serving shapes at full size: against an fp32 matmul on the decoded weights (the reference's
    decode + dense matmul in fp32; 1e-3 is the path's stated tolerance, the observed error is fp32 rounding)."""
    from ixrun_b200.p6 import P6Packed
    from ixrun_b200.synth import synthetic_packed

    p6 = P6Packed.from_packed(synthetic_packed(out_f, in_f, seed=3))
    x = torch.randn(m, in_f, device="cuda").bfloat16()
    w = p6.decode(kind="bf16")
    ref = x.double() @ w.double().t()
    y = p6.gemm(x, out_dtype=torch.float32)
    err = float((y.double() - ref).abs().max() / ref.abs().max())
    assert err < 2e-5, err
    assert torch.equal(p6.gemm(x), y.bfloat16())
