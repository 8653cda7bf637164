"""One-kernel all-reduce over peer memory: the single-rank case on one GPU (the kernel talks to its own buffer;
several ranks never share a GPU) -- data path, epochs across calls, bias, fp32/bf16 output, CUDA-graph replay."""
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
