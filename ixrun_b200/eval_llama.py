"""Config-3 style evaluation of the packed Llama runner on one GPU:

    python -m ixrun_b200.eval_llama [--layers 24] [--prompt 1024] [--new 256]

Random-init Llama-style decoder (hidden 2048, SwiGLU 6144, 16 Q / 8 KV heads of
128, vocab 73448), all linears packed.  Prints one JSON line with the
graph-mode ms/token of the packed model, the same for the decoded-bf16 model,
and the teacher-forced greedy-token agreement between the two.
"""
from __future__ import annotations

import argparse
import os
import json
import time

import torch

from .llama_runner import LlamaConfig, PackedLlama, synthetic_llama


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=24)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--new", type=int, default=256)
    ap.add_argument("--shared-layer-weights", action="store_true",
                    help="generate one tensor per linear type and reuse it in every layer (faster set-up)")
    ap.add_argument("--batched", default="",
                    help="comma-separated batch sizes: also time lock-step decoding of B sequences (BatchedGreedyDecoder; "
                         "B <= 8 on the fused GEMV, up to 64 on the tensor-core GEMM) and report tokens per second")
    ap.add_argument("--no-pdl", action="store_true",
                    help="launch the packed GEMVs without programmatic dependent launch")
    args = ap.parse_args()
    cfg = LlamaConfig(n_layers=args.layers, max_seq=args.prompt + args.new)
    t0 = time.time()
    layers, embed, head = synthetic_llama(cfg, seed=0, distinct_layers=not args.shared_layer_weights)
    packed_bytes = sum(p["total_bytes"] for d in layers for p in d.values())
    n_weights = sum(p["N"] for d in layers for p in d.values())
    packed = PackedLlama(cfg, layers, embed, head, weights="packed")
    dense = PackedLlama(cfg, layers, embed, head, weights="decoded")
    setup_s = time.time() - t0
    prompt = torch.randint(0, cfg.vocab, (args.prompt,), generator=torch.Generator().manual_seed(1))
    lp, ld = packed.prefill(prompt), dense.prefill(prompt)
    torch.cuda.synchronize()
    if not args.no_pdl and os.environ.get("IXB200_RESIDENT", "p6") == "p6":
        from .p6 import set_pdl

        set_pdl(True)               # every layout is complete: a GEMV may fetch weights while its predecessor finishes
    packed.capture()
    dense.capture()

    def timed(model, first_logits):
        tok = first_logits.argmax(-1)
        toks = []
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(args.new):
            toks.append(tok.clone())
            tok = model.step(tok, args.prompt + i).argmax(-1)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / args.new, torch.cat(toks)

    ms_packed, toks_packed = timed(packed, lp)
    ms_dense, toks_dense = timed(dense, ld)
    # teacher forcing: feed the ground-truth model's tokens to both, compare arg-max step by step
    packed.prefill(prompt)
    dense.prefill(prompt)
    tok = ld.argmax(-1)
    agree, ties, min_margin = 0, 0, float("inf")
    for i in range(args.new):
        a, b = packed.step(tok, args.prompt + i), dense.step(tok, args.prompt + i)
        top2 = b.topk(2).values[0]
        # a token counts as agreeing when the ground-truth model scores it as high as its own arg-max
        # (bf16 logits of a random-init model tie exactly now and then)
        same = int(float(b[0, a.argmax(-1).item()]) == float(top2[0]))
        agree += same
        ties += int(float(top2[0]) == float(top2[1]))
        if not same:
            min_margin = min(min_margin, float(top2[0] - top2[1]))
        tok = b.argmax(-1)
    batched = None
    if args.batched:
        from .llama_runner import BatchedGreedyDecoder

        batched = []
        g = torch.Generator().manual_seed(2)
        for b in (int(v) for v in args.batched.split(",")):
            dec = BatchedGreedyDecoder(packed, b)
            tok = dec.prefill([torch.randint(0, cfg.vocab, (128,), generator=g) for _ in range(b)])
            dec.capture()
            for _ in range(3):
                tok = dec.step(tok).argmax(-1)
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            steps = 32
            e0.record()
            for _ in range(steps):
                tok = dec.step(tok).argmax(-1)
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / steps
            batched.append({"sequences": b, "ms_per_step": round(ms, 4), "tokens_per_s": round(b / ms * 1e3, 1),
                            "linears": "fused GEMV" if b <= 8 else "tcgen05 GEMM"})
            del dec
            torch.cuda.empty_cache()
    print(json.dumps({
        "model": f"llama-style {args.layers}L h{cfg.hidden} ffn{cfg.intermediate} {cfg.n_heads}q/{cfg.n_kv_heads}kv vocab{cfg.vocab}",
        "packed_linears": len(layers) * 7, "packed_weights": n_weights, "packed_MB": packed_bytes / 1e6,
        "prompt": args.prompt, "new_tokens": args.new, "mode": "one CUDA graph per token step",
        "resident_layout": os.environ.get("IXB200_RESIDENT", "p6"), "programmatic_dependent_launch": not args.no_pdl,
        "ms_per_token_packed": ms_packed, "ms_per_token_decoded_bf16": ms_dense,
        "greedy_agreement_teacher_forced": agree / args.new, "steps_with_exact_top1_tie": ties,
        "free_running_prefix_match": int((toks_packed == toks_dense).long().cumprod(0).sum().item()),
        "min_top1_top2_margin_at_mismatch": None if agree == args.new else min_margin,
        "setup_s": setup_s, "batched_decode_128_token_prompts": batched,
    }), flush=True)


if __name__ == "__main__":
    main()
