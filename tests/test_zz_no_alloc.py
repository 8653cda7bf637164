"""ixb_gemv_static: the fused decode+GEMV entry point for callers that cannot
allocate device memory (its scratch is an array inside the library image).

Called through the C ABI and compared, bit for bit, with ixb_gemv on the same
inputs, for two calls in a row (the second reuses whatever the first left in
the shared array).  This file is named so that pytest collects it last.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _layer(out_f, in_f, seed):
    from ixrun_b200.packed import DevicePacked
    from ixrun_b200.synth import synthetic_packed

    return DevicePacked(synthetic_packed(out_f, in_f, seed))


def _static(dp, x, out_dtype, bias=None):
    from ixrun_b200 import _lib

    m = x.shape[0]
    y = torch.full((m, dp.out_f), float("nan"), dtype=out_dtype, device=x.device)
    rc = _lib.lib().ixb_gemv_static(C.byref(dp.struct), dp.blk_q1.data_ptr(), dp.blk_q2.data_ptr(), x.data_ptr(), m,
                                    None if bias is None else bias.data_ptr(), y.data_ptr(),
                                    1 if out_dtype == torch.float32 else 0, _lib.stream_ptr(x.device))
    _lib.check(rc)
    return y


@pytest.mark.parametrize("out_f,in_f,m", [(640, 5120, 1), (96, 2176, 3), (2048, 2048, 8)])
def test_static_scratch_matches_caller_scratch_twice(out_f, in_f, m):
    dp = _layer(out_f, in_f, seed=out_f + m)
    g = torch.Generator().manual_seed(m)
    bias = torch.randn(out_f, generator=g).bfloat16().cuda()
    for call in range(2):
        x = torch.randn(m, in_f, generator=g).bfloat16().cuda()
        for dt in (torch.float32, torch.bfloat16):
            want = dp.gemv(x, bias=bias, out_dtype=dt)
            got = _static(dp, x, dt, bias=bias)
            assert torch.equal(got, want), (call, dt)


def test_static_scratch_rejects_oversize_shapes():
    from ixrun_b200 import _lib

    L = _lib.lib()
    # a fake shape whose slots exceed the built-in array: rejected before any launch
    p = _lib.Packed()
    p.out_f, p.in_f = 1 << 20, 32
    assert L.ixb_gemv_scratch_bytes(p.out_f, p.in_f, 8) > 4 * 1024 * 1024
    rc = L.ixb_gemv_static(C.byref(p), None, None, None, 8, None, None, 0, None)
    assert rc == 4 and b"built-in array" in L.ixb_last_error()


def test_static_scratch_call_allocates_no_device_memory():
    """Free device memory (cudaMemGetInfo) and the caching allocator's counters are the same before and after calls
    of ixb_gemv_static: the entry point neither allocates nor frees."""
    dp = _layer(640, 5120, seed=5)
    x = torch.randn(2, 5120).bfloat16().cuda()
    _static(dp, x, torch.bfloat16)                       # first call on this device: symbol address looked up
    torch.cuda.synchronize()
    y = torch.empty(2, 640, dtype=torch.bfloat16, device="cuda")
    from ixrun_b200 import _lib

    L = _lib.lib()
    free0, _ = torch.cuda.mem_get_info()
    stats0 = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.memory_stats().get("num_alloc_retries", 0))
    for _ in range(3):
        _lib.check(L.ixb_gemv_static(C.byref(dp.struct), dp.blk_q1.data_ptr(), dp.blk_q2.data_ptr(), x.data_ptr(), 2, None,
                                     y.data_ptr(), 0, _lib.stream_ptr(x.device)))
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    stats1 = (torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.memory_stats().get("num_alloc_retries", 0))
    assert free1 == free0 and stats1 == stats0
    assert torch.equal(y, dp.gemv(x))
