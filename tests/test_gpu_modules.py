"""Packed-linear modules and functional entry points (the reference's API
surface for this path) on the GPU, checked against the CPU oracle."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn

from oracle import ixb_oracle as O

pytestmark = pytest.mark.gpu


def bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


def bits(t):
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


def oracle_y(codes, scale_t, x, out_f, in_f):
    sc = int(bits(scale_t.reshape(1))[0])
    return O.gemm_f32(codes, sc, bits(x.reshape(-1, in_f)), out_f, in_f)


def make_layer(out_f, in_f, seed, bias=False):
    from ixrun_b200.quantize import int8x_quantize

    torch.manual_seed(seed)
    # heavy-tail weights like the reference's parity scripts (tests/test_fused.py:17-22)
    w = torch.randn(out_f, in_f) * 0.005
    flat = w.view(-1)
    idx = torch.randperm(flat.numel())[: int(flat.numel() * 0.04)]
    flat[idx] = torch.randn(len(idx)) * 0.05
    w = w.bfloat16()
    p = int8x_quantize(w)
    b = (torch.randn(out_f) * 0.1).bfloat16() if bias else None
    codes = O.quantize_bf16(bits(w))[0]
    return w, p, b, codes


@pytest.mark.parametrize("out_f,in_f", [(1536, 1536), (512, 4608), (300, 96)])
def test_streaming_linear_single_token(out_f, in_f):
    from ixrun_b200.engine import StreamingLinear

    w, p, b, codes = make_layer(out_f, in_f, 0, bias=True)
    x = torch.randn(1, 1, in_f).bfloat16().cuda()
    ref = torch.from_numpy(oracle_y(codes, p["scale"], x, out_f, in_f)).bfloat16() + b
    # the default keeps one copy of the weights (the resident layout); keep_streams=True keeps the reference's
    # buffers beside it; resident="streams" runs the fused kernel on the streams themselves
    for kw in ({}, {"keep_streams": True}, {"resident": "streams"}):
        sl = StreamingLinear(p, bias=b, **kw)
        assert sl.out_features == out_f and sl.in_features == in_f
        if kw:
            assert sl._use_fused == (in_f % 32 == 0) and sl._b1.is_cuda and sl._l3.is_cuda
            if sl._use_fused:
                assert sl._q1.numel() == (out_f * (in_f // sl._split_chunk) if sl._split_chunk else out_f)
        else:
            assert not hasattr(sl, "_b1") and sl._dp is None and sl.resident_bytes == sl._res.resident_bytes
        y = sl(x)
        assert y.shape == (1, 1, out_f) and y.dtype == torch.bfloat16
        # one bf16 ulp of slack for sums that sit on a rounding boundary
        assert (y.cpu().float().reshape(-1) - ref.float().reshape(-1)).abs().max() <= 2.0 ** -7 * ref.float().abs().max()


def test_streaming_linear_many_tokens_uses_decode_buffer():
    from ixrun_b200.engine import StreamingLinear

    out_f, in_f = 256, 1024
    w, p, b, codes = make_layer(out_f, in_f, 1, bias=True)
    sl = StreamingLinear(p, bias=b, keep_streams=True)
    x = torch.randn(2, 16, in_f).bfloat16().cuda()
    ref = oracle_y(codes, p["scale"], x, out_f, in_f).reshape(2, 16, out_f) + b.float().numpy()
    # 9..64 rows: the tensor-core GEMM on the resident layout, no decode buffer involved (the fused paths round the
    # sum to bf16 and then add the bias in bf16, ixrun/engine.py:166-168: up to one more bf16 ulp than the dense path)
    y_gemm = sl(x)
    assert np.abs(y_gemm.float().cpu().numpy() - ref).max() / np.abs(ref).max() < 1e-2
    assert torch.equal(y_gemm.reshape(32, out_f), sl._res.gemm(x.reshape(32, in_f)) + b.cuda())
    # more than 64 rows (or the GEMM switched off): decode into the shared buffer + dense matmul
    sl._use_p6_gemm = False
    with pytest.raises(RuntimeError):
        sl(x)                                  # no shared buffer yet
    buf = torch.empty(out_f * in_f + 100, dtype=torch.bfloat16, device="cuda")
    sl._set_shared_buf(buf)
    y = sl(x)
    x_many = torch.randn(100, in_f).bfloat16().cuda()
    sl._use_p6_gemm = True
    assert sl(x_many).shape == (100, out_f)    # beyond the GEMM's row count: the decode path
    sl._use_p6_gemm = False
    w_dec = bf16(O.decode_bf16({**p, "scale": int(bits(p["scale"].reshape(1))[0]),
                                "bitmaps": [t.numpy() for t in p["bitmaps"]],
                                "streams": [t.numpy() for t in p["streams"]]}))
    assert torch.equal(sl._decode().cpu(), w_dec)
    err = np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max()
    assert err < 5e-3
    # the same input through the tensor-core fused kernel (opt-in)
    sl._use_tc = True
    y_tc = sl(x)
    # the fused paths round the sum to bf16 and then add the bias in bf16 (ixrun/engine.py:166-168):
    # up to one more bf16 ulp than the dense path, which adds the bias before rounding
    assert np.abs(y_tc.float().cpu().numpy() - ref).max() / np.abs(ref).max() < 1e-2
    assert torch.equal(y_tc.reshape(32, out_f), sl._dp.gemm(x.reshape(32, in_f)) + b.cuda())


def test_fused_gemv_and_prefix_functions_golden(golden_dir):
    from ixrun_b200.fused import compute_row_prefixes, fused_gemv

    g = dict(np.load(os.path.join(golden_dir, "heavy_64x1024.npz")))
    out_f, in_f = g["w_bits"].shape
    p = {"level_bits": (3, 5, 8), "out_f": out_f, "in_f": in_f, "N": out_f * in_f,
         "scale": bf16(g["scale_bits"]).reshape(()), "bitmaps": [torch.from_numpy(g["b1"]), torch.from_numpy(g["b2"])],
         "streams": [torch.from_numpy(g["l1"]), torch.from_numpy(g["l2"]), torch.from_numpy(g["l3"])],
         "counts": [int(c) for c in g["counts"]]}
    q1, q2 = compute_row_prefixes(p)
    assert q1.device.type == "cpu" and np.array_equal(q1.numpy(), g["row_q1"]) and np.array_equal(q2.numpy(), g["row_q2"])
    chunk = int(g["chunk"][0])
    q1c, q2c = compute_row_prefixes(p, chunk)
    assert np.array_equal(q1c.numpy(), g["chunk_q1"]) and np.array_equal(q2c.numpy(), g["chunk_q2"])
    dev = "cuda"
    x = bf16(g["x_bits"])[0].to(dev)
    gb = [t.to(dev) for t in (*p["bitmaps"], *p["streams"])]
    y = fused_gemv(x, *gb, q1.to(dev), q2.to(dev), p["scale"].to(dev), out_f, in_f)
    ref = g["y_f32"][0]
    assert y.shape == (out_f,) and y.dtype == torch.bfloat16
    assert np.abs(y.float().cpu().numpy() - ref).max() / np.abs(ref).max() < 5e-3
    y32 = torch.full((out_f,), 7.0, dtype=torch.float32, device=dev)      # stale contents must not matter
    r = fused_gemv(x, *gb, q1c.to(dev), q2c.to(dev), p["scale"].to(dev), out_f, in_f, chunk=chunk, y32=y32)
    assert r is y32
    assert np.abs(y32.cpu().numpy() - ref).max() / np.abs(ref).max() < 2e-5


def test_decode_functions_and_cached_linear():
    from ixrun_b200.kernels import decode_codes, decode_weight_triton, precompute_block_offsets
    from ixrun_b200.linear import Int8XLinear

    out_f, in_f = 128, 256
    w, p, b, codes = make_layer(out_f, in_f, 2, bias=True)
    wd = decode_weight_triton(p, device="cuda")
    assert torch.equal(decode_codes(p).cpu().reshape(-1), torch.from_numpy(codes))
    sc = p["scale"].float()
    assert torch.equal(wd.cpu(), (torch.from_numpy(codes).float() * sc).bfloat16().view(out_f, in_f))
    a, c = precompute_block_offsets(p, 1024)
    np_p = {**p, "scale": 0, "bitmaps": [t.numpy() for t in p["bitmaps"]], "streams": [t.numpy() for t in p["streams"]]}
    q1, q2 = O.prefixes(np_p, 1024)
    assert np.array_equal(a.cpu().numpy(), q1) and np.array_equal(c.cpu().numpy(), q2)
    a2, c2 = precompute_block_offsets(p, 4096)
    q1, q2 = O.prefixes(np_p, 4096)
    assert np.array_equal(a2.cpu().numpy(), q1) and np.array_equal(c2.cpu().numpy(), q2)
    for cache in ("full", "none"):
        lin = Int8XLinear(p, bias=b, cache=cache)
        x = torch.randn(4, in_f).bfloat16().cuda()
        y = lin(x)
        ref = torch.nn.functional.linear(x, wd, b.cuda())
        assert torch.equal(y, ref)


class ToyBlock(nn.Module):
    def __init__(self, h=256, f=768):
        super().__init__()
        self.gate_proj = nn.Linear(h, f, bias=False)
        self.up_proj = nn.Linear(h, f, bias=False)
        self.down_proj = nn.Linear(f, h, bias=True)
        self.lm_head = nn.Linear(h, 64, bias=False)      # skipped by name
        self.tiny = nn.Linear(8, 8)                      # skipped by size

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


@pytest.mark.parametrize("mode", ["cached", "streaming", "graph"])
def test_engine_deploy_modes_agree(mode, tmp_path):
    from ixrun_b200.engine import GraphLinear, Int8XEngine, StreamingLinear
    from ixrun_b200.linear import Int8XLinear, iter_quantizable_linears

    torch.manual_seed(0)
    ref_model = ToyBlock().bfloat16()
    names = [n for n, _ in iter_quantizable_linears(ref_model)]
    assert names == ["gate_proj", "up_proj", "down_proj"]
    # ground truth: the same block with weights replaced by their decoded int8 values
    from ixrun_b200.kernels import decode_weight
    from ixrun_b200.quantize import int8x_quantize

    gt = ToyBlock().bfloat16()
    gt.load_state_dict(ref_model.state_dict())
    for n in names:
        lin = getattr(gt, n)
        lin.weight.data = decode_weight(int8x_quantize(lin.weight.data)).cpu()
    gt = gt.cuda()
    model = ToyBlock().bfloat16()
    model.load_state_dict(ref_model.state_dict())
    replay = None
    if mode == "cached":
        model = model.cuda()
        stats = Int8XEngine._deploy_cached(model, (3, 5, 8), verbose=False)
        assert isinstance(model.gate_proj, Int8XLinear) and stats["n_layers"] == 3
    elif mode == "streaming":
        cache = str(tmp_path / "packed.pt")
        stats = Int8XEngine._deploy_streaming(model, (3, 5, 8), verbose=False, cache_path=cache)
        assert os.path.exists(cache) and isinstance(model.down_proj, StreamingLinear)
        # second deploy loads the cache file; a wrong scheme is rejected
        m2 = ToyBlock().bfloat16()
        Int8XEngine._deploy_streaming(m2, (3, 5, 8), verbose=False, cache_path=cache)
        with pytest.raises(ValueError):
            Int8XEngine._deploy_streaming(ToyBlock().bfloat16(), (2, 5, 8), verbose=False, cache_path=cache)
        model = model.cuda()
    else:
        stats, replay = Int8XEngine._deploy_graph(model, (3, 5, 8), verbose=False)
        assert isinstance(model.up_proj, GraphLinear)
        model = model.cuda()
        for n in names:                       # buffers are only valid after a replay
            getattr(model, n)._w_buf.zero_()
        replay()
    assert stats["total_bytes"] > 0
    for shape in [(1, 1, 256), (1, 5, 256), (2, 9, 256)]:
        x = torch.randn(*shape).bfloat16().cuda()
        y, y_gt = model(x), gt(x)
        tol = 2e-2 * y_gt.float().abs().max()
        assert (y.float() - y_gt.float()).abs().max() <= tol, (mode, shape)


def test_graphed_layer_sequence_matches_eager():
    """CUDA-graph capture of a per-layer sequence of fused launches"""
    from ixrun_b200.engine import GraphedCall, StreamingLinear

    h, f = 512, 1536
    layers = [StreamingLinear(make_layer(f, h, 10)[1]), StreamingLinear(make_layer(f, h, 11)[1]),
              StreamingLinear(make_layer(h, f, 12)[1])]

    def mlp(x):
        return layers[2](torch.nn.functional.silu(layers[0](x)) * layers[1](x))

    x = torch.randn(1, h).bfloat16().cuda()
    gc = GraphedCall(mlp, x)
    for _ in range(3):
        x = torch.randn(1, h).bfloat16().cuda()
        assert torch.equal(gc(x), mlp(x))


def test_graphed_call_with_host_buffers_is_one_launch_per_call():
    """host_io=True: the copies from and to pinned host memory are part of the graph; run_host returns the result
    in host memory, equal to the eager module call on the same input."""
    from ixrun_b200.engine import GraphedCall, StreamingLinear

    lay = StreamingLinear(make_layer(768, 1024, 21)[1])
    gc = GraphedCall(lay, torch.zeros(1, 1024).bfloat16().cuda(), host_io=True)
    for i in range(3):
        x = torch.randn(1, 1024, generator=torch.Generator().manual_seed(i)).bfloat16()
        y = gc.run_host(x)
        assert not y.is_cuda and y.is_pinned()
        assert torch.equal(y, lay(x.cuda()).cpu())
    with pytest.raises(RuntimeError):
        GraphedCall(lay, torch.zeros(1, 1024).bfloat16().cuda()).run_host(x)
