"""Llama-style decode loop on packed linears: graph-captured step equals the
eager step, and the packed model agrees with the same model run on decoded
bf16 weights (teacher-forced greedy tokens)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def tiny():
    from ixrun_b200.llama_runner import LlamaConfig, PackedLlama, synthetic_llama

    cfg = LlamaConfig(n_layers=2, hidden=256, intermediate=512, n_heads=4, n_kv_heads=2, head_dim=64,
                      vocab=1000, max_seq=96)
    layers, embed, head = synthetic_llama(cfg, seed=1)
    packed = PackedLlama(cfg, layers, embed, head, weights="packed")
    dense = PackedLlama(cfg, layers, embed, head, weights="decoded")
    return cfg, packed, dense


def test_graph_step_equals_eager_and_matches_decoded_weights():
    cfg, packed, dense = tiny()
    g = torch.Generator().manual_seed(0)
    prompt = torch.randint(0, cfg.vocab, (40,), generator=g)
    lp, ld = packed.prefill(prompt), dense.prefill(prompt)
    assert (lp - ld).abs().max() <= 0.05 * ld.abs().max()
    tok = ld.argmax(-1)
    # eager steps first, then the same positions again from a captured graph
    eager = []
    for i in range(8):
        eager.append(packed.step(tok, 40 + i).clone())
        tok = dense.step(tok, 40 + i).argmax(-1)
    packed.capture()
    tok = ld.argmax(-1)
    agree = 0
    dense.prefill(prompt)
    for i in range(8):
        lg = packed.step(tok, 40 + i)
        assert torch.equal(lg, eager[i]), f"graph replay differs from eager at step {i}"
        ref = dense.step(tok, 40 + i)
        agree += int(lg.argmax(-1).item() == ref.argmax(-1).item())
        assert (lg - ref).abs().max() <= 0.05 * ref.abs().max()
        tok = ref.argmax(-1)          # teacher forcing on the ground-truth model
    assert agree == 8


def test_generate_runs_and_is_deterministic():
    cfg, packed, _ = tiny()
    prompt = torch.randint(0, cfg.vocab, (20,), generator=torch.Generator().manual_seed(3))
    a = packed.generate(prompt, 12)
    packed.capture()
    b = packed.generate(prompt, 12)
    assert a.shape == (12,) and torch.equal(a, b)


def test_batched_decoder_gives_every_sequence_its_own_tokens():
    """Three prompts of different lengths decoded in lock-step (3 rows per linear through the fused GEMV, one cache and
    one position per row): every sequence gets the logits, bit for bit, and so the tokens, of its own batch-1 decode;
    eager and from the captured graph."""
    from ixrun_b200.llama_runner import BatchedGreedyDecoder

    cfg, packed, _ = tiny()
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab, (n,), generator=g) for n in (17, 40, 29)]
    alone = [packed.generate(p, 10) for p in prompts]
    dec = BatchedGreedyDecoder(packed, 3)
    toks = dec.generate(prompts, 10)
    assert torch.equal(toks, torch.stack(alone))
    dec2 = BatchedGreedyDecoder(packed, 3)
    first = dec2.prefill(prompts)
    dec2.capture()
    out, tok = [], first
    for _ in range(10):
        out.append(tok.clone())
        tok = dec2.step(tok).argmax(-1)
    assert torch.equal(torch.stack(out, dim=1), toks)


def test_batched_decoder_on_the_tensor_core_gemm():
    """Twelve sequences: the linears run on the tcgen05 GEMM (another summation order than the GEMV), so a sequence's
    logits agree with its batch-1 decode to bf16 noise instead of bit for bit."""
    from ixrun_b200.llama_runner import BatchedGreedyDecoder

    cfg, packed, _ = tiny()
    g = torch.Generator().manual_seed(6)
    prompts = [torch.randint(0, cfg.vocab, (20 + 3 * i,), generator=g) for i in range(12)]
    dec = BatchedGreedyDecoder(packed, 12)
    tok = dec.prefill(prompts)
    logits = dec.step(tok)
    for r in (0, 5, 11):
        packed.prefill(prompts[r])
        ref = packed.step(tok[r], prompts[r].numel())
        assert (logits[r] - ref[0]).abs().max() <= 0.05 * ref.abs().max()
    assert torch.isfinite(logits).all()


def test_verifier_gives_the_logits_of_the_steps_one_by_one():
    """Five tokens of one sequence in one pass (5 rows per linear, causal attention among them): the logits of every row
    are, bit for bit, those of the batch-1 steps taken one after the other; eager and from the captured graph; and the
    acceptance rule keeps exactly the prefix of a draft that greedy decoding would have produced."""
    from ixrun_b200.llama_runner import Verifier

    cfg, packed, _ = tiny()
    prompt = torch.randint(0, cfg.vocab, (30,), generator=torch.Generator().manual_seed(9))
    first = packed.prefill(prompt).argmax(-1)
    greedy = packed.generate(prompt, 8)                               # greedy[0] == first
    assert int(greedy[0]) == int(first)
    packed.prefill(prompt)
    ref = torch.cat([packed.step(greedy[i], 30 + i) for i in range(5)])     # logits after feeding greedy[0..4]
    ver = Verifier(packed, 5)
    for mode in ("eager", "graph"):
        packed.prefill(prompt)
        if mode == "graph":
            ver.capture()
            packed.prefill(prompt)
        got = ver(greedy[:5], 30)
        assert torch.equal(got, ref), mode
    # a draft whose third token is wrong: two draft tokens are confirmed, the model's own token replaces the third
    packed.prefill(prompt)
    draft = greedy[:5].clone()
    draft[3] = (draft[3] + 1) % cfg.vocab
    n, nxt = ver.accept(draft, 30)
    assert n == 2 and int(nxt) == int(greedy[3])


def test_verifier_on_the_tensor_core_gemm():
    from ixrun_b200.llama_runner import Verifier

    cfg, packed, _ = tiny()
    prompt = torch.randint(0, cfg.vocab, (25,), generator=torch.Generator().manual_seed(10))
    packed.prefill(prompt)
    toks = torch.randint(0, cfg.vocab, (12,), generator=torch.Generator().manual_seed(11))
    ref = torch.cat([packed.step(toks[i], 25 + i) for i in range(12)])
    packed.prefill(prompt)
    got = Verifier(packed, 12)(toks, 25)
    assert (got - ref).abs().max() <= 0.05 * ref.abs().max()
