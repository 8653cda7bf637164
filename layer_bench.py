"""Per-layer timing of the packed-weight kernels on one GPU (a measurement helper beside bench.py).

    python layer_bench.py --shape 5120x17408 --rows 1 --kernel p6 --graph --pdl
    python layer_bench.py --sweep [--graph --pdl]     # the shape / row-count sweep of the benchmark configs

For each case one JSON line: microseconds per launch (CUDA events on the
launching stream), packed-weight GB/s on the reference's byte count, and the
fraction of the measured HBM peak.  Without --graph every launch is timed alone
and an L2-sized buffer is overwritten between repetitions; with --graph the
launches sit back to back in a CUDA graph that rotates over enough copies of the
layer to keep the weights out of L2, and the graph is replayed until the timed
region is long (the number a model step sees).
Kernels: p6 / p6gemm / p6decode (resident layout: fused GEMV for 1..8 rows,
tcgen05 GEMM for up to 64 rows, decode to bf16; p6decode+dense = decode then a
dense matmul, what the GEMM replaces), gemv / gemm / decode (the reference's streams read directly), dense (bf16
matmul on decoded weights, the "cached mode" of the reference).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from ixrun_b200.p6 import P6Packed, set_pdl  # noqa: E402
from ixrun_b200.packed import DevicePacked  # noqa: E402
from ixrun_b200.synth import synthetic_packed  # noqa: E402

SWEEP_SHAPES = [(5120, 17408), (17408, 5120), (5120, 5120), (1024, 5120), (2048, 2048)]
L2_BYTES = 128 << 20


def _peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"])
    return 6650.0


def time_us(fn, reps: int, flush: torch.Tensor | None, warm: int = 3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def _line(out_f, in_f, rows, kernel, us, total_bytes, **extra):
    alg = total_bytes + 2 * in_f * rows + 2 * out_f * rows
    gbs = alg / us / 1e3
    d = {"shape": f"{out_f}x{in_f}", "rows": rows, "kernel": kernel, "us": round(us, 2), "packed_GBps": round(gbs, 1),
         "frac_of_measured_hbm_peak": round(gbs / _peak(), 4)}
    d.update(extra)
    return d


def run_case(dp: DevicePacked, total_bytes: int, kernel: str, rows: int, reps: int, flush, wdense=None, p6=None):
    out_f, in_f = dp.out_f, dp.in_f
    x = torch.randn(rows, in_f, device=dp.device).bfloat16()
    y = torch.empty(rows, out_f, dtype=torch.bfloat16, device=dp.device)
    if kernel == "gemv":
        fn = lambda: dp.gemv(x, out=y)
    elif kernel == "p6":
        fn = lambda: p6.gemv(x, out=y)
    elif kernel == "p6gemm":
        fn = lambda: p6.gemm(x, out=y)
    elif kernel == "p6decode+dense":
        w = torch.empty(out_f * in_f, dtype=torch.bfloat16, device=dp.device)
        fn = lambda: torch.nn.functional.linear(x, p6.decode(out=w))
    elif kernel == "p6decode":
        w = torch.empty(out_f * in_f, dtype=torch.bfloat16, device=dp.device)
        fn = lambda: p6.decode(out=w)
    elif kernel == "gemm":
        fn = lambda: dp.gemm(x, out=y)
    elif kernel == "decode":
        w = torch.empty(out_f * in_f, dtype=torch.bfloat16, device=dp.device)
        fn = lambda: dp.decode(out=w)
    elif kernel == "dense":
        fn = lambda: torch.nn.functional.linear(x, wdense, out=None)
    else:
        raise ValueError(kernel)
    return _line(out_f, in_f, rows, kernel, time_us(fn, reps, flush), total_bytes)


def run_graph_case(dp: DevicePacked, total_bytes: int, rows: int, first: P6Packed, pdl: bool, launches: int = 40,
                   min_ms: float = 30.0):
    """Device time per launch with the launches back to back in a CUDA graph over copies of the layer."""
    n_copies = max(2, min(24, (2 * L2_BYTES + first.resident_bytes - 1) // first.resident_bytes + 1))
    copies = [first] + [P6Packed.from_packed(dp) for _ in range(n_copies - 1)]
    x = torch.randn(rows, dp.in_f, device=dp.device).bfloat16()
    y = torch.empty(rows, dp.out_f, dtype=torch.bfloat16, device=dp.device)
    for c in copies:
        c.gemv(x, out=y)
    torch.cuda.synchronize()
    prev = set_pdl(pdl)
    try:
        st = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(st):
            with torch.cuda.graph(g, stream=st):
                for i in range(launches):
                    copies[i % n_copies].gemv(x, out=y)
            g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            g.replay()
            b.record()
            b.synchronize()
            one = a.elapsed_time(b)
            replays = max(3, int(min_ms / max(one, 1e-3)) + 1)
            a.record()
            for _ in range(replays):
                g.replay()
            b.record()
            b.synchronize()
            us = a.elapsed_time(b) * 1e3 / (replays * launches)
    finally:
        set_pdl(prev)
    return _line(dp.out_f, dp.in_f, rows, "p6 (graph, pdl)" if pdl else "p6 (graph)", us, total_bytes,
                 us_first_replay=round(one * 1e3 / launches, 2), copies=n_copies, launches_per_graph=launches,
                 replays=replays, resident_bytes=first.resident_bytes)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="5120x17408")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--kernel", default="p6", choices=["gemv", "p6", "p6gemm", "p6decode+dense", "p6decode", "gemm", "decode", "dense"])
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--pdl", action="store_true", help="with --graph: programmatic dependent launch between the launches")
    ap.add_argument("--graph", action="store_true", help="p6: time launches captured back to back in one CUDA graph")
    args = ap.parse_args()
    flush = None if args.no_flush else torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda")
    if not args.sweep:
        out_f, in_f = (int(v) for v in args.shape.split("x"))
        p = synthetic_packed(out_f, in_f, seed=1)
        dp = DevicePacked(p)
        wd = dp.decode(kind="bf16").clone() if args.kernel == "dense" else None
        p6 = P6Packed.from_packed(dp) if args.kernel.startswith("p6") else None
        if args.graph and args.kernel == "p6":
            print(json.dumps(run_graph_case(dp, p["total_bytes"], args.rows, p6, args.pdl)), flush=True)
            return
        print(json.dumps(run_case(dp, p["total_bytes"], args.kernel, args.rows, args.reps, flush, wd, p6)), flush=True)
        return
    for out_f, in_f in SWEEP_SHAPES:
        p = synthetic_packed(out_f, in_f, seed=1)
        dp = DevicePacked(p)
        p6 = P6Packed.from_packed(dp)
        big = out_f * in_f > 50e6
        for rows in ([1, 2, 4, 8] if big else [1]):
            if args.graph:
                print(json.dumps(run_graph_case(dp, p["total_bytes"], rows, p6, args.pdl)), flush=True)
            else:
                print(json.dumps(run_case(dp, p["total_bytes"], "p6", rows, args.reps, flush, None, p6)), flush=True)
        if not args.graph:
            wd = dp.decode(kind="bf16").clone()
            for k in ("gemv", "dense", "decode", "p6decode"):
                print(json.dumps(run_case(dp, p["total_bytes"], k, 1, args.reps, flush, wd, p6)), flush=True)
            del wd
        del dp, p6
        torch.cuda.empty_cache()


if __name__ == "__main__":
    main()
