"""Batch-1 decode of the 27B-class hybrid decoder (48 gated-delta-rule + 16 gated full-attention layers, hidden 5120,
SwiGLU 17408, vocabulary 151936) on packed INT8-X linears, tensor-parallel with one process per GPU.

    python -m ixrun_b200.hybrid27b [--layers 64] [--tokens 256] [--context 4096]
    python -m torch.distributed.run --nproc-per-node N ... -m ixrun_b200.hybrid27b

The whole token step -- embedding row, 64 blocks, final norm, lm_head, greedy arg-max, the token fed back and the
position advanced -- is ONE CUDA graph with no host round trip, so a decode of T tokens is T graph replays.

Per block (8 or 10 launches, on one GPU as on several); the packed linears that share an input are fused
row-wise into one resident tensor, every part keeping its own per-tensor scale (p6.P6Packed.fuse):
  gated-delta-rule layer  residual add + RMSNorm -> ONE packed GEMV for in_proj_qkv | z | a | b -> ONE kernel for the
                          causal conv1d update + SiLU and the recurrent step per value head (state fp32
                          [heads][128][128], read and written once) with the gated output norm -> out_proj
  attention layer         residual add + RMSNorm -> ONE packed GEMV for q (+ gate) | k | v -> per-head q/k RMSNorm +
                          partial RoPE + KV-cache write -> split-context grouped-query attention over the static
                          cache with the sigmoid output gate -> o_proj
  MLP                     residual add + RMSNorm -> ONE packed GEMV for gate | up -> SwiGLU -> down_proj
The reference leaves this glue to HuggingFace eager code and fla's Triton kernels (ixrun/fla_patch.py:23-72); here
it is this library's glue kernels, all of them part of the programmatic-dependent-launch chain of the GEMVs.

Tensor parallelism: in-projections, gate and up are column-parallel (heads / rows split; with more ranks than KV heads
a rank still holds one whole KV head), out_proj / o_proj / down_proj are row-parallel: their fp32 partial sums leave the
GEMV's epilogue as peer stores into every rank's exchange buffer and a 20-CTA finishing kernel adds them up in front of
the next residual add + RMSNorm kernel (the norm kernel can also take the sum itself, which saves two launches per block
but was measured slower: one CTA cannot pull every rank's words through its SM fast enough) -- one exchange per
token-mixer block and one per MLP block.  lm_head is split by vocabulary; the ranks exchange (max, index) pairs.
With --nccl the partial sums go through eager NCCL all-reduces instead (no graph; a cross-check, not a fast path).

The fused q|gate projection is stored as [all q heads | all gate heads] (a row permutation of the per-head
interleaved layout, applied when the weights are deployed).  Weights are synthetic (Laplace codes, a separate device
copy per layer); the KV caches hold `context` random positions when decoding starts.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import time
from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import glue as G
from .packed import DevicePacked
from .synth import synthetic_packed


@dataclass
class HybridConfig:
    n_layers: int = 64
    hidden: int = 5120
    ffn: int = 17408
    vocab: int = 151936
    gdn_k_heads: int = 16
    gdn_v_heads: int = 48
    gdn_dim: int = 128                 # the recurrent kernel is written for 128 x 128 head states
    conv_k: int = 4
    attn_heads: int = 24
    attn_kv_heads: int = 4
    attn_dim: int = 256
    rot_dim: int = 64
    attn_every: int = 4                # layers 3, 7, 11, ... are attention layers
    eps: float = 1e-6
    rope_theta: float = 1e7

    def is_attn(self, li: int) -> bool:
        return li % self.attn_every == self.attn_every - 1


@contextlib.contextmanager
def _stdout_to_stderr():
    """File descriptor 1 points at stderr inside the block (for output that native libraries write themselves)."""
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        yield
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


def shard_geometry(cfg: HybridConfig, world: int) -> dict:
    """Heads and rows one rank holds."""
    if cfg.gdn_k_heads % world or cfg.gdn_v_heads % world or cfg.attn_heads % world or cfg.ffn % (64 * world) \
            or cfg.vocab % world:
        raise ValueError(f"the model does not split over {world} ranks")
    hk, hv, hq = cfg.gdn_k_heads // world, cfg.gdn_v_heads // world, cfg.attn_heads // world
    hkv = max(1, cfg.attn_kv_heads // world)
    if hq % hkv:
        raise ValueError("query heads per rank must be a multiple of the KV heads per rank")
    return {"hk": hk, "hv": hv, "hq": hq, "hkv": hkv, "ffn": cfg.ffn // world, "vocab": cfg.vocab // world}


def linear_shapes(cfg: HybridConfig, world: int) -> dict:
    """(rows, cols) of one rank's shard of every packed linear, by layer kind."""
    g, h, d, da = shard_geometry(cfg, world), cfg.hidden, cfg.gdn_dim, cfg.attn_dim
    return {
        "gdn": {"in_proj_qkv": ((2 * g["hk"] + g["hv"]) * d, h), "in_proj_z": (g["hv"] * d, h), "in_proj_a": (g["hv"], h),
                "in_proj_b": (g["hv"], h), "out_proj": (h, g["hv"] * d)},
        "attn": {"q_proj": (2 * g["hq"] * da, h), "k_proj": (g["hkv"] * da, h), "v_proj": (g["hkv"] * da, h),
                 "o_proj": (h, g["hq"] * da)},
        "mlp": {"gate_proj": (g["ffn"], h), "up_proj": (g["ffn"], h), "down_proj": (h, g["ffn"])},
    }


class Hybrid27B:
    """One rank's share of the model and the state of one decoding sequence."""

    def __init__(self, cfg: HybridConfig, world: int, rank: int, dev, context: int = 4096, max_new: int = 272,
                 nccl: bool = False, seed: int = 0, lm_head: bool = True, fused_finish: bool | None = None):
        from .p6 import P6Packed

        self.cfg, self.world, self.rank, self.dev = cfg, world, rank, torch.device(dev)
        self.geo = g = shard_geometry(cfg, world)
        self.context, self.max_seq = context, context + max_new
        self.nccl = nccl and world > 1
        # second half of the exchange: the 20-CTA finishing kernel followed by the plain norm kernel (default), or inside
        # the norm kernel itself (fused_finish / IXB200_FUSED_FINISH=1).  The norm kernel is ONE CTA and has to pull every
        # rank's marked words through one SM: measured slower at every world size (2 ranks: 4.50 vs 4.38 ms/token,
        # 8 ranks: 4.11 vs 3.02), although it saves two launches per block.
        env = os.environ.get("IXB200_FUSED_FINISH")
        self.fused_finish = fused_finish if fused_finish is not None else (env == "1")
        self.ar = None
        if world > 1 and not nccl:
            from .parallel import PeerAllReduce

            self.ar = PeerAllReduce(max(cfg.hidden, 4 * world), dev)
        gen = torch.Generator(device="cpu").manual_seed(seed * 7919 + 13)      # replicated parameters: same on every rank
        bf = dict(dtype=torch.bfloat16, device=self.dev)

        def rnd(*shape, scale=1.0, shift=0.0, dtype=torch.bfloat16):
            return (torch.randn(*shape, generator=gen) * scale + shift).to(self.dev, dtype)

        shapes = linear_shapes(cfg, world)
        host = {}

        def dp(kind, name, j):
            r, c = shapes[kind][name]
            if (kind, name) not in host:
                host[(kind, name)] = synthetic_packed(r, c, seed=(seed * 64 + j) * 131 + rank)
            return DevicePacked(host[(kind, name)], self.dev)           # separate device copy per layer

        self.layers = []
        self.packed_bytes = self.resident_bytes = self.n_weights = 0
        n_attn = n_gdn = 0
        d, da = cfg.gdn_dim, cfg.attn_dim
        self.conv_ch = (2 * g["hk"] + g["hv"]) * d
        for li in range(cfg.n_layers):
            kind = "attn" if cfg.is_attn(li) else "gdn"
            names = list(shapes[kind])
            L = {"kind": kind}
            # the in-projections share their input: one resident tensor, one launch (every part keeps its scale)
            L["in"] = P6Packed.fuse([dp(kind, n, j) for j, n in enumerate(names[:-1])])
            L["out"] = P6Packed.from_packed(dp(kind, names[-1], len(names) - 1))
            L["gate_up"] = P6Packed.fuse([dp("mlp", "gate_proj", 8), dp("mlp", "up_proj", 9)])
            L["down"] = P6Packed.from_packed(dp("mlp", "down_proj", 10))
            L["ln1"], L["ln2"] = rnd(cfg.hidden, scale=0.05, shift=1.0), rnd(cfg.hidden, scale=0.05, shift=1.0)
            if kind == "attn":
                L["q_norm"], L["k_norm"] = rnd(da, scale=0.05, shift=1.0), rnd(da, scale=0.05, shift=1.0)
                L["slot"] = n_attn
                n_attn += 1
            else:
                # per-rank slices of per-head / per-channel parameters: every rank draws its own (synthetic model)
                L["conv_w"] = rnd(self.conv_ch, cfg.conv_k, scale=0.3)
                L["A_log"] = rnd(g["hv"], scale=0.5, dtype=torch.float32)
                L["dt_bias"] = rnd(g["hv"], scale=0.5, dtype=torch.float32)
                L["gn_w"] = rnd(d, scale=0.05, shift=1.0)
                L["slot"] = n_gdn
                n_gdn += 1
            self.layers.append(L)
            for v in L.values():
                if isinstance(v, P6Packed):
                    self.packed_bytes += v.total_bytes
                    self.resident_bytes += v.resident_bytes
                    self.n_weights += sum(n for _, n in v.sections) * v.in_f
        self.ln_f = rnd(cfg.hidden, scale=0.05, shift=1.0)
        self.embed = rnd(cfg.vocab, cfg.hidden, scale=0.02)
        self.lm_head = rnd(g["vocab"], cfg.hidden, scale=0.02) if lm_head else None
        # sequence state
        kv_gen = torch.Generator(device=self.dev).manual_seed(seed * 31 + 5 + rank // max(1, world // cfg.attn_kv_heads))
        self.k_cache = torch.zeros(max(n_attn, 1), self.max_seq, g["hkv"], da, **bf)
        self.v_cache = torch.zeros_like(self.k_cache)
        if n_attn and context:
            self.k_cache[:, :context] = torch.randn(n_attn, context, g["hkv"], da, device=self.dev, generator=kv_gen).bfloat16()
            self.v_cache[:, :context] = torch.randn(n_attn, context, g["hkv"], da, device=self.dev, generator=kv_gen).bfloat16()
        self.gdn_state = torch.zeros(max(n_gdn, 1), g["hv"], d, d, dtype=torch.float32, device=self.dev)
        # the conv's history is kept twice: the step at position p reads copy p & 1 and writes the other (glue.gdn_conv_step)
        self.conv_state = torch.zeros(max(n_gdn, 1), 2, self.conv_ch, cfg.conv_k - 1, **bf)
        self.cos, self.sin = G.rope_tables(self.max_seq, cfg.rot_dim, cfg.rope_theta, self.dev)
        self.attn = G.AttnDecode(g["hq"], g["hkv"], da, self.dev) if n_attn else None
        # static activations of the one-row step
        z = lambda n, dt=torch.bfloat16: torch.zeros(1, n, dtype=dt, device=self.dev)
        self.h, self.xn, self.d_out = z(cfg.hidden), z(cfg.hidden), z(cfg.hidden)
        first = {k: next((L for L in self.layers if L["kind"] == k), None) for k in ("gdn", "attn")}
        self.qkv_c, self.mix, self.att = z(self.conv_ch), z(g["hv"] * d), z(g["hq"] * da)
        if first["gdn"] is not None:                # outputs of the fused in-projections and the parts' views
            self.in_gdn = z(first["gdn"]["in"].out_f)
            self.qkv, self.z_, self.a_, self.b_ = first["gdn"]["in"].split(self.in_gdn)
        if first["attn"] is not None:
            self.in_attn = z(first["attn"]["in"].out_f)
            self.qg, self.k_, self.v_ = first["attn"]["in"].split(self.in_attn)
        self.gu = z(self.layers[0]["gate_up"].out_f)
        self.g_, self.u_ = self.layers[0]["gate_up"].split(self.gu)
        self.act = z(g["ffn"])
        self.y32 = z(cfg.hidden, torch.float32)
        self.tok = torch.zeros(1, dtype=torch.long, device=self.dev)
        self.pos32 = torch.full((1,), context, dtype=torch.int32, device=self.dev)
        self.n_done = torch.zeros(1, dtype=torch.long, device=self.dev)
        self.toks = torch.zeros(max_new, dtype=torch.long, device=self.dev)
        self.mx = torch.zeros(max(4, 2 * world), dtype=torch.float32, device=self.dev)
        self.graph = None
        self.n_allreduce = 2 * cfg.n_layers + (1 if lm_head else 0)

    # ------------------------------------------------------------------ one block
    def _row_parallel(self, lin, x):
        """Row-parallel linear.  One GPU: the bf16 result lands in self.d_out, the caller's next add + norm takes it
        from there.  Several: the fp32 partial sums leave the GEMV as peer stores; returns None, and the caller's next
        norm kernel is also the second half of the exchange (glue.finish_add_rmsnorm)."""
        if self.ar is not None:
            n = lin.gemv_push(x, self.ar)
            if self.fused_finish:
                return None
            return self.ar.finish(n, self.d_out)
        if self.nccl:
            lin.gemv(x, out=self.y32)
            dist.all_reduce(self.y32)
            self.d_out.copy_(self.y32)
        else:
            lin.gemv(x, out=self.d_out)
        return self.d_out

    def _add_norm(self, delta, w, first=False):
        if self.ar is not None and not first and self.fused_finish:
            return G.finish_add_rmsnorm(self.ar, self.h, w, self.cfg.eps, out=self.xn)
        return G.add_rmsnorm(self.h, delta, w, self.cfg.eps, out=self.xn)

    def _mixer(self, L):
        cfg, g = self.cfg, self.geo
        s = L["slot"]
        if L["kind"] == "attn":
            L["in"].gemv(self.xn, out=self.in_attn)
            nq = g["hq"] * cfg.attn_dim
            G.rope_kv(self.qg, self.k_, self.v_, self.pos32, self.k_cache[s], self.v_cache[s], self.cos, self.sin,
                      g["hq"], g["hkv"], cfg.attn_dim, rot_dim=cfg.rot_dim, q_norm=L["q_norm"], k_norm=L["k_norm"],
                      eps=cfg.eps, q_stride=2 * nq)
            self.attn(self.qg, self.k_cache[s], self.v_cache[s], self.pos32, out=self.att, gate=self.qg[nq:])
            return self._row_parallel(L["out"], self.att)
        L["in"].gemv(self.xn, out=self.in_gdn)
        G.gdn_conv_step(self.qkv, self.conv_state[s], L["conv_w"], self.pos32, self.z_, self.a_, self.b_, L["A_log"],
                        L["dt_bias"], L["gn_w"], self.gdn_state[s], g["hk"], g["hv"], cfg.eps, out=self.mix[0])
        return self._row_parallel(L["out"], self.mix)

    def _step(self):
        cfg = self.cfg
        torch.index_select(self.embed, 0, self.tok, out=self.h)
        delta, first = None, True
        for L in self.layers:
            self._add_norm(delta, L["ln1"], first)
            first = False
            delta = self._mixer(L)
            self._add_norm(delta, L["ln2"])
            L["gate_up"].gemv(self.xn, out=self.gu)
            G.swiglu(self.g_, self.u_, out=self.act[0])
            delta = self._row_parallel(L["down"], self.act)
        self._add_norm(delta, self.ln_f, first)
        if self.lm_head is not None:
            logits = F.linear(self.xn, self.lm_head).float()
            val, idx = logits.max(dim=-1)
            if self.world > 1:
                # gather (max, global index) of every rank: a sum of vectors that are zero outside the rank's own pair
                self.mx.zero_()
                self.mx[2 * self.rank: 2 * self.rank + 1] = val
                self.mx[2 * self.rank + 1: 2 * self.rank + 2] = (idx + self.rank * self.geo["vocab"]).float()
                if self.ar is not None:
                    allv = self.ar(self.mx, out_dtype=torch.float32)
                else:
                    allv = self.mx.clone()
                    dist.all_reduce(allv)
                pairs = allv[: 2 * self.world].view(self.world, 2)
                best = pairs[:, 0].argmax().view(1)
                idx = pairs[:, 1].index_select(0, best).long()          # (no host round trip: this runs inside the graph)
            self.toks.index_copy_(0, self.n_done, idx)
            self.tok.copy_(idx)
        self.n_done += 1
        self.pos32 += 1
        return self.h

    # ------------------------------------------------------------------ driving
    def reset(self, first_token: int = 1):
        """Back to the first decode position (the caches keep the context; recurrent states start from zero)."""
        self.tok.fill_(first_token)
        self.pos32.fill_(self.context)
        self.n_done.zero_()
        self.gdn_state.zero_()
        self.conv_state.zero_()

    def capture(self):
        if self.nccl:
            return                                                   # eager NCCL all-reduces stay outside graphs
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._step()
        self.graph = g

    def step(self):
        if self.graph is not None:
            self.graph.replay()
        else:
            self._step()
        return self.h


def launches_per_token(cfg: HybridConfig, world: int) -> int:
    """Kernels of this library in one token step (packed GEMVs, glue, exchange)."""
    n = 0
    for li in range(cfg.n_layers):
        n += (6 if cfg.is_attn(li) else 4) + 4 + (2 if world > 1 else 0)      # a finishing kernel per exchange
    return n + 1 + (1 if world > 1 else 0)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=256)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--nccl", action="store_true",
                    help="several GPUs: sum the partial outputs with eager NCCL all-reduces (no CUDA graph) instead of "
                         "the exchange over peer memory inside one graph per token")
    ap.add_argument("--no-pdl", action="store_true", help="launch without programmatic dependent launch")
    args = ap.parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime

        with _stdout_to_stderr():        # NCCL prints its version line to stdout; stdout is for the one JSON line
            dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
            dist.barrier()
    rec = measure(world, rank, dev, tokens=args.tokens, nccl=args.nccl, layers=args.layers, eager=args.eager,
                  pdl=not args.no_pdl, context=args.context)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure(world: int, rank: int, dev, tokens: int = 256, nccl: bool = False, layers: int = 64, eager: bool = False,
            pdl: bool = True, context: int = 4096, lm_head: bool = True) -> dict:
    """Deploy the model on this rank (the process group, if any, is already up) and time a greedy decode of `tokens`
    tokens.  Every rank must call it; the returned record is the same on every rank (max over ranks)."""
    from .p6 import set_pdl

    t0 = time.time()
    cfg = HybridConfig(n_layers=layers)
    with torch.no_grad():
        m = Hybrid27B(cfg, world, rank, dev, context=context, max_new=tokens + 16, nccl=nccl, lm_head=lm_head)
        torch.cuda.synchronize()
        prev_pdl = set_pdl(bool(pdl))                    # every layout is complete: launches may overlap their neighbours' tails
        setup = time.time() - t0
        try:
            ar_check = None
            if m.ar is not None:
                # the peer all-reduce against NCCL on one random vector (two ranks: the same bits; more: fp32 rounding)
                v = torch.randn(1, cfg.hidden, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank))
                got = m.ar(v, out_dtype=torch.float32)
                ref = v.clone()
                dist.all_reduce(ref)
                ar_check = float((got - ref).abs().max() / ref.abs().max())
                if ar_check > 1e-6 or m.ar.timed_out():
                    raise RuntimeError(f"peer all-reduce differs from NCCL: rel {ar_check}, timed out {m.ar.timed_out()}")
            mode = "eager"
            if not eager and not m.nccl:
                m.capture()
                mode = ("one CUDA graph per token step" if world == 1 else
                        "one CUDA graph per token step; partial sums pushed from the GEMV epilogue over peer memory")
            elif m.nccl:
                mode = "eager launches, NCCL all-reduces"
            m.reset()
            for _ in range(3):
                m.step()
            m.reset()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(tokens):
                m.step()
            e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1) / tokens
        finally:
            set_pdl(prev_pdl)
        toks = m.toks[:tokens].clone()
        finite = bool(torch.isfinite(m.h.float()).all().item())
        same_tokens = None
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
            if lm_head:
                ref = toks.clone()
                dist.broadcast(ref, 0)
                ok = torch.tensor([int(torch.equal(ref, toks))], device=dev)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN)
                same_tokens = bool(ok.item())
    return {
        "model": f"27B-class hybrid decoder, {layers} layers (3 gated-delta-rule : 1 gated attention), hidden {cfg.hidden}, "
                 f"ffn {cfg.ffn}, vocab {cfg.vocab}",
        "n_gpus": world, "parallelism": f"tp{world}", "mode": mode, "ms_per_token": ms,
        "tokens_decoded": tokens, "context": context, "greedy_feedback_on_device": bool(lm_head),
        "exchanges_per_token": m.n_allreduce if world > 1 else 0,
        "launches_per_token": launches_per_token(cfg, world),
        "packed_weights_per_rank": m.n_weights, "packed_GB_per_rank": m.packed_bytes / 1e9,
        "packed_GBps_per_gpu": m.packed_bytes / 1e9 / (ms * 1e-3),
        "resident_GB_per_rank": m.resident_bytes / 1e9,
        "distinct_tokens": int(toks.unique().numel()), "hidden_state_finite": finite,
        "same_tokens_on_every_rank": same_tokens, "setup_s": setup,
        "peer_allreduce_vs_nccl_rel": ar_check, "peer_allreduce_timed_out": (m.ar.timed_out() if m.ar is not None else None),
        "mixers": "gated delta rule (causal conv + recurrence) and gated softmax attention over the KV cache, this library's kernels",
    }


if __name__ == "__main__":
    main()
