"""One-kernel all-reduce over peer memory: the single-rank case on one GPU (the kernel talks to its own buffer;
several ranks never share a GPU) -- data path, epochs across calls, bias, fp32/bf16 output, CUDA-graph replay; the
same exchange with the sending half inside the GEMV's epilogue; and the bounded wait made to run out (a two-rank
geometry whose second rank never sends)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_allreduce_is_the_identity_call_after_call():
    from ixrun_b200.parallel import PeerAllReduce

    n = 5120
    ar = PeerAllReduce(n, "cuda")
    bias = torch.randn(1, n, device="cuda").bfloat16()
    for i in range(5):                                   # both parities of the slot buffer, growing epochs
        x = torch.randn(1, n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(i))
        assert torch.equal(ar(x, out_dtype=torch.float32), x)
        assert torch.equal(ar(x), x.bfloat16())
        assert torch.equal(ar(x, bias=bias), x.bfloat16() + bias)
    short = torch.randn(1, 1024, device="cuda")
    assert torch.equal(ar(short, out_dtype=torch.float32), short)
    assert not ar.timed_out()
    with pytest.raises(ValueError):
        ar(torch.randn(1, n + 4, device="cuda"))
    with pytest.raises(ValueError):
        ar(torch.randn(1, 6, device="cuda"))


def test_single_rank_allreduce_replays_from_a_cuda_graph():
    from ixrun_b200.parallel import PeerAllReduce

    n = 2048
    ar = PeerAllReduce(n, "cuda")
    x = torch.zeros(1, n, device="cuda")
    y = torch.empty(1, n, dtype=torch.float32, device="cuda")
    ar(x, out=y)
    torch.cuda.synchronize()
    st = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        with torch.cuda.graph(g, stream=st):
            for _ in range(3):
                ar(x, out=y)
    for i in range(4):
        x.copy_(torch.full((1, n), float(i + 1), device="cuda"))
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y, x)
    assert not ar.timed_out()


def _shard(out_f, in_f, seed):
    from ixrun_b200.p6 import P6Packed
    from oracle import ixb_oracle as O

    codes = O.laplace_codes(out_f, in_f, seed)
    return P6Packed(torch.from_numpy(codes).cuda(), torch.tensor(0.00251, dtype=torch.bfloat16), out_f, in_f)


@pytest.mark.parametrize("out_f,in_f,m", [(5120, 2176, 1), (512, 17408, 1), (1024, 4352, 4), (96, 2176, 8)])
def test_gemv_push_then_finish_equals_the_plain_gemv(out_f, in_f, m):
    """Single rank: the GEMV's epilogue stores marked words into the all-reduce buffer, the finishing kernel turns
    them into y -- the same bits as ixb_p6_gemv, call after call, mixed with plain all-reduce calls, and replayed
    from a CUDA graph."""
    from ixrun_b200.parallel import PeerAllReduce

    p6 = _shard(out_f, in_f, 5)
    n = m * out_f
    ar = PeerAllReduce(max(n, 5120), "cuda")
    bias = torch.randn(m, out_f, device="cuda").bfloat16()
    y32 = torch.empty(m, out_f, dtype=torch.float32, device="cuda")
    y16 = torch.empty(m, out_f, dtype=torch.bfloat16, device="cuda")
    for i in range(4):
        x = torch.randn(m, in_f, device="cuda", generator=torch.Generator(device="cuda").manual_seed(i)).bfloat16()
        ref = p6.gemv(x, out_dtype=torch.float32)
        assert p6.gemv_push(x, ar) == n
        assert torch.equal(ar.finish(n, y32), ref)
        p6.gemv_push(x, ar)
        assert torch.equal(ar.finish(n, y16, bias=bias), ref.bfloat16() + bias)
        # both halves in one kernel
        assert torch.equal(p6.gemv_allreduce(x, ar, out_dtype=torch.float32), ref)
        assert torch.equal(p6.gemv_allreduce(x, ar, bias=bias[0].contiguous()), ref.bfloat16() + bias[0])
        v = torch.randn(1, 1024, device="cuda")
        assert torch.equal(ar(v, out_dtype=torch.float32), v)          # a plain call in between keeps the counters in step
    x = torch.randn(m, in_f, device="cuda").bfloat16()
    st = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        p6.gemv_push(x, ar)
        ar.finish(n, y32)
        with torch.cuda.graph(g, stream=st):
            for _ in range(3):
                p6.gemv_push(x, ar)
                ar.finish(n, y32)
                p6.gemv_allreduce(x, ar, out=y32)
    for i in range(3):
        x.copy_(torch.randn(m, in_f, device="cuda").bfloat16())
        y32.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(y32, p6.gemv(x, out_dtype=torch.float32))
    assert not ar.timed_out()


def test_a_wait_that_runs_out_sets_the_error_word_and_returns():
    """Rank 0 of a two-rank geometry on one GPU: rank 1 never sends, the wait gives up after the (shortened) limit,
    the kernel returns, timed_out() is true, later calls give up at once; reset() clears it."""
    from ixrun_b200.parallel import PeerAllReduce

    n = 1024
    prev = PeerAllReduce.set_spin_limit(200)
    try:
        ar = PeerAllReduce.loopback(n, "cuda", world=2, rank=0)
        x = torch.ones(1, n, device="cuda")
        y = ar(x, out_dtype=torch.float32)
        torch.cuda.synchronize()                       # the kernel came back
        assert ar.timed_out()
        assert torch.isfinite(y).all()
        ar(x, out_dtype=torch.float32)                  # gives up after 64 polls now
        torch.cuda.synchronize()
        # the finishing kernel's wait runs out the same way
        ar2 = PeerAllReduce.loopback(n, "cuda", world=2, rank=0)
        p6 = _shard(n, 2176, 9)
        p6.gemv_push(torch.randn(1, 2176, device="cuda").bfloat16(), ar2)
        ar2.finish(n, torch.empty(1, n, dtype=torch.float32, device="cuda"))
        torch.cuda.synchronize()
        assert ar2.timed_out()
        ar2.reset()
        assert not ar2.timed_out()
        p6.gemv_allreduce(torch.randn(1, 2176, device="cuda").bfloat16(), ar2, out_dtype=torch.float32)
        torch.cuda.synchronize()
        assert ar2.timed_out()                          # ... and so does the one-kernel form's
    finally:
        PeerAllReduce.set_spin_limit(prev)
    # a single rank is unaffected
    ar1 = PeerAllReduce(n, "cuda")
    assert torch.equal(ar1(x, out_dtype=torch.float32), x) and not ar1.timed_out()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("rows,hidden", [(1, 5120), (3, 512), (1, 2048)])
def test_finishing_norm_equals_finish_then_add_rmsnorm(world, rows, hidden):
    """Every rank's sending half runs in turn on this one GPU (loopback objects sharing one buffer, each launch as its
    own rank with its own shard), then ONE finishing call adds the words up: the fused finish + residual add + RMSNorm
    kernel gives the same bits as the finishing kernel followed by the add + norm kernel, call after call."""
    from ixrun_b200.glue import add_rmsnorm, finish_add_rmsnorm
    from ixrun_b200.parallel import PeerAllReduce

    in_f = 2176
    n = rows * hidden
    ars = [PeerAllReduce.loopback(max(n, 5120), "cuda", world=world, rank=0)]
    ars += [PeerAllReduce.loopback(max(n, 5120), "cuda", world=world, rank=r, share=ars[0]) for r in range(1, world)]
    shards = [_shard(hidden, in_f, 20 + r) for r in range(world)]
    w = (1 + 0.1 * torch.randn(hidden, device="cuda")).bfloat16()
    for call in range(3):
        xs = [torch.randn(rows, in_f, device="cuda").bfloat16() for _ in range(world)]
        h0 = torch.randn(rows, hidden, device="cuda").bfloat16()
        # two kernels
        for r in range(world):
            shards[r].gemv_push(xs[r], ars[r])
        d = ars[0].finish(n, torch.empty(rows, hidden, dtype=torch.bfloat16, device="cuda"))
        ref32 = sum(shards[r].gemv(xs[r], out_dtype=torch.float32) for r in range(world))
        assert float((d.float() - ref32).abs().max()) <= 2.0 ** -7 * float(ref32.abs().max())
        h_ref = h0.clone()
        xn_ref = add_rmsnorm(h_ref, d, w, 1e-6)
        # one kernel
        for r in range(world):
            shards[r].gemv_push(xs[r], ars[r])
        h = h0.clone()
        xn = finish_add_rmsnorm(ars[0], h, w, 1e-6)
        assert torch.equal(h, h_ref) and torch.equal(xn, xn_ref)
    assert not ars[0].timed_out()
