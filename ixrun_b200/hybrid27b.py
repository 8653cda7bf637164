"""Tensor-parallel packed-linear stack of the 27B-class hybrid decoder
(48 gated-delta-rule + 16 full-attention layers, hidden 5120, SwiGLU 17408),
batch-1 decode step, one process per GPU.

    python -m ixrun_b200.hybrid27b [--layers 64] [--tokens 16]
    python -m torch.distributed.run --nproc-per-node N ... -m ixrun_b200.hybrid27b

What is real: every packed linear of every layer with its true shape, sharded
tensor-parallel (column-parallel in-projections / gate / up, row-parallel
out/o/down projections), fp32 partial sums and ONE all-reduce per
token-mixer block and per MLP block (2 per layer), residual adds and RMSNorms.
The whole token step is one CUDA graph.  On several GPUs the all-reduce is one
kernel of this library over peer memory (parallel.PeerAllReduce) inside that
graph; with --nccl every stretch of launches between two all-reduces is its
own graph and NCCL all-reduces are launched eagerly in between (capturing NCCL
inside one graph stalled on this pool).  What is a stand-in: the token mixers
themselves (gated delta rule recurrence, causal conv, softmax attention over
the KV cache) are replaced by an elementwise gate over the projected values, so
the reported ms/token is the packed-weight path of the model, not the full
model.  Weights are synthetic (Laplace codes); each rank generates its own
shard-sized tensors per linear type and uses a separate device copy per layer.
"""
from __future__ import annotations

import contextlib
import sys

import argparse
import json
import os
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

from .packed import DevicePacked
from .synth import synthetic_packed

HIDDEN, FFN = 5120, 17408
# (rows, cols) of the unsharded linears; "col" = column-parallel (rows split), "row" = row-parallel (cols split)
GDN = {"in_proj_qkv": (10240, HIDDEN, "col"), "in_proj_z": (6144, HIDDEN, "col"), "in_proj_a": (48, HIDDEN, "col"),
       "in_proj_b": (48, HIDDEN, "col"), "out_proj": (HIDDEN, 6144, "row")}
ATTN = {"q_proj": (12288, HIDDEN, "col"), "k_proj": (1024, HIDDEN, "col"), "v_proj": (1024, HIDDEN, "col"),
        "o_proj": (HIDDEN, 6144, "row")}
MLP = {"gate_proj": (FFN, HIDDEN, "col"), "up_proj": (FFN, HIDDEN, "col"), "down_proj": (HIDDEN, FFN, "row")}
KV_HEAD_ROWS = 256      # one KV head; with more ranks than KV heads a rank still holds a whole head



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

def shard_shape(name, rows, cols, mode, world):
    if mode == "row":
        return rows, cols // world
    r = rows // world
    if name in ("k_proj", "v_proj"):
        r = max(r, KV_HEAD_ROWS)
    return r, cols


class Stack:
    def __init__(self, n_layers: int, world: int, rank: int, dev, layout: str = "p6", nccl: bool = False):
        self.world, self.dev = world, dev
        self.ar = None
        if world > 1 and not nccl:
            from .parallel import PeerAllReduce

            self.ar = PeerAllReduce(HIDDEN, dev)        # one kernel over peer memory per row-parallel layer
        cache = {}

        def mk(name, spec, seed):
            rows, cols, mode = spec
            r, c = shard_shape(name, rows, cols, mode, world)
            key = (name, r, c)
            if key not in cache:
                cache[key] = synthetic_packed(r, c, seed=seed * 131 + rank)
            dp = DevicePacked(cache[key], dev)          # separate device copy per layer
            if layout == "p6":
                from .p6 import P6Packed

                return P6Packed.from_packed(dp)         # the streams are dropped, the re-layout stays resident
            return dp

        self.layers = []
        self.packed_bytes = 0
        self.resident_bytes = 0
        self.n_weights = 0
        for li in range(n_layers):
            kind = ATTN if li % 4 == 3 else GDN
            mix = {n: mk(n, s, i + 1) for i, (n, s) in enumerate(kind.items())}
            mlp = {n: mk(n, s, i + 11) for i, (n, s) in enumerate(MLP.items())}
            self.layers.append((kind is ATTN, mix, mlp))
            for dp in list(mix.values()) + list(mlp.values()):
                self.packed_bytes += dp.total_bytes
                self.resident_bytes += getattr(dp, "resident_bytes", dp.total_bytes)
                self.n_weights += dp.N
        self.norm_w = torch.ones(HIDDEN, dtype=torch.bfloat16, device=dev)
        self.h = torch.randn(1, HIDDEN, device=dev).bfloat16()
        self.graph = None
        self.n_allreduce = 2 * n_layers

    def _norm(self, h):
        v = h.float()
        return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * self.norm_w

    def _reduce(self, y32):
        if self.ar is not None:
            return self.ar(y32)
        if self.world > 1:
            dist.all_reduce(y32)
        return y32.to(torch.bfloat16)

    def _step(self, h):
        for is_attn, mix, mlp in self.layers:
            x = self._norm(h)
            if is_attn:
                q, k, v = mix["q_proj"].gemv(x), mix["k_proj"].gemv(x), mix["v_proj"].gemv(x)
                n_in = mix["o_proj"].in_f
                # stand-in for attention: gate the first half of q with its second half, touch k and v
                a = q[:, :n_in] * torch.sigmoid(q[:, n_in:2 * n_in].float()).to(q.dtype) + (k.sum() + v.sum()) * 0
                out = mix["o_proj"]
            else:
                qkv, z = mix["in_proj_qkv"].gemv(x), mix["in_proj_z"].gemv(x)
                a_, b_ = mix["in_proj_a"].gemv(x), mix["in_proj_b"].gemv(x)
                n_in = mix["out_proj"].in_f
                # stand-in for the gated delta rule: value slice gated by z, touch the a/b projections
                a = qkv[:, -n_in:] * F.silu(z[:, :n_in].float()).to(qkv.dtype) + (a_.sum() + b_.sum()) * 0
                out = mix["out_proj"]
            h = h + self._reduce(out.gemv(a.contiguous(), out_dtype=torch.float32))
            x = self._norm(h)
            g, u = mlp["gate_proj"].gemv(x), mlp["up_proj"].gemv(x)
            h = h + self._reduce(mlp["down_proj"].gemv((F.silu(g.float()).to(g.dtype) * u), out_dtype=torch.float32))
        return h

    # -- world > 1: the collectives stay outside CUDA graphs.  Every stretch of launches between two
    #    all-reduces becomes its own graph over the static tensors h (bf16) and y32 (fp32 partial sums).
    def _seg_mixer(self, li):
        is_attn, mix, _ = self.layers[li]
        if li > 0:
            self.h.add_(self.y32.to(torch.bfloat16))           # residual of the previous layer's MLP
        x = self._norm(self.h)
        if is_attn:
            q, k, v = mix["q_proj"].gemv(x), mix["k_proj"].gemv(x), mix["v_proj"].gemv(x)
            n_in = mix["o_proj"].in_f
            a = q[:, :n_in] * torch.sigmoid(q[:, n_in:2 * n_in].float()).to(q.dtype) + (k.sum() + v.sum()) * 0
            out = mix["o_proj"]
        else:
            qkv, z = mix["in_proj_qkv"].gemv(x), mix["in_proj_z"].gemv(x)
            a_, b_ = mix["in_proj_a"].gemv(x), mix["in_proj_b"].gemv(x)
            n_in = mix["out_proj"].in_f
            a = qkv[:, -n_in:] * F.silu(z[:, :n_in].float()).to(qkv.dtype) + (a_.sum() + b_.sum()) * 0
            out = mix["out_proj"]
        out.gemv(a.contiguous(), out=self.y32)

    def _seg_mlp(self, li):
        _, _, mlp = self.layers[li]
        self.h.add_(self.y32.to(torch.bfloat16))
        x = self._norm(self.h)
        g, u = mlp["gate_proj"].gemv(x), mlp["up_proj"].gemv(x)
        mlp["down_proj"].gemv(F.silu(g.float()).to(g.dtype) * u, out=self.y32)

    def capture(self):
        if self.world == 1 or self.ar is not None:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(2):
                    self._step(self.h)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                self.out = self._step(self.h)
            self.graph = g
            return
        self.y32 = torch.zeros(1, HIDDEN, dtype=torch.float32, device=self.dev)
        self.h0 = self.h.clone()
        segs = []
        for li in range(len(self.layers)):
            segs += [lambda li=li: self._seg_mixer(li), lambda li=li: self._seg_mlp(li)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for f in segs:
                f()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.segments = []
        for f in segs:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                f()
            self.segments.append(g)
        torch.cuda.synchronize()

    def step(self):
        if self.world > 1 and getattr(self, "segments", None):
            self.h.copy_(self.h0)
            for g in self.segments:
                g.replay()
                dist.all_reduce(self.y32)
            return self.h
        if self.graph is not None:
            self.graph.replay()
            return self.out
        return self._step(self.h)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--tokens", type=int, default=16)
    ap.add_argument("--eager", action="store_true")
    ap.add_argument("--layout", default="p6", choices=["p6", "streams"],
                    help="resident weight layout: the P6 re-layout, or the reference's streams read directly")
    ap.add_argument("--nccl", action="store_true",
                    help="several GPUs: sum the partial outputs with eager NCCL all-reduces between per-stretch graphs "
                         "instead of the one-kernel all-reduce over peer memory inside one graph per token")
    ap.add_argument("--no-pdl", action="store_true",
                    help="layout p6: launch the GEMVs without programmatic dependent launch")
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
    rec = measure(world, rank, dev, tokens=args.tokens, nccl=args.nccl, layers=args.layers, layout=args.layout,
                  eager=args.eager, pdl=not args.no_pdl)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


def measure(world: int, rank: int, dev, tokens: int = 16, nccl: bool = False, layers: int = 64, layout: str = "p6",
            eager: bool = False, pdl: bool = True) -> dict:
    """Deploy the stack on this rank (the process group, if any, is already up) and time `tokens` decode steps.
    Every rank must call it; the returned record is the same on every rank (max over ranks)."""
    t0 = time.time()
    with torch.no_grad():
        st = Stack(layers, world, rank, dev, layout=layout, nccl=nccl)
        torch.cuda.synchronize()
        if layout == "p6" and pdl:
            from .p6 import set_pdl

            set_pdl(True)                               # every layout is complete: GEMVs may overlap their neighbours' tails
        setup = time.time() - t0
        ar_check = None
        if st.ar is not None:
            # the peer all-reduce against NCCL on one random vector (two ranks: the same bits; more: fp32 rounding)
            v = torch.randn(1, HIDDEN, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank))
            got = st.ar(v, out_dtype=torch.float32)
            ref = v.clone()
            dist.all_reduce(ref)
            ar_check = float((got - ref).abs().max() / ref.abs().max())
            if ar_check > 1e-6 or st.ar.timed_out():
                raise RuntimeError(f"peer all-reduce differs from NCCL: rel {ar_check}, timed out {st.ar.timed_out()}")
        mode = "eager"
        if not eager:
            st.capture()
            mode = ("one CUDA graph per token step" if world == 1 else
                    "one CUDA graph per token step, all-reduces as one kernel each over peer memory" if st.ar is not None
                    else "one CUDA graph per stretch between all-reduces; NCCL all-reduces launched eagerly")
        for _ in range(3):
            st.step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(tokens):
            st.step()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / tokens
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return {
        "model": f"27B-class hybrid linear stack, {layers} layers (3 GDN : 1 attention), hidden {HIDDEN}, ffn {FFN}",
        "n_gpus": world, "parallelism": f"tp{world}", "mode": mode, "ms_per_token": ms,
        "all_reduces_per_token": st.n_allreduce if world > 1 else 0,
        "packed_weights_per_rank": st.n_weights, "packed_GB_per_rank": st.packed_bytes / 1e9,
        "packed_GBps_per_gpu": st.packed_bytes / 1e9 / (ms * 1e-3),
        "layout": layout, "resident_GB_per_rank": st.resident_bytes / 1e9,
        "tokens_timed": tokens, "setup_s": setup,
        "peer_allreduce_vs_nccl_rel": ar_check, "peer_allreduce_timed_out": (st.ar.timed_out() if st.ar is not None else None),
        "note": "packed-weight path only; token mixers are elementwise stand-ins",
    }


if __name__ == "__main__":
    main()
