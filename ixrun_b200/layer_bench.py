"""Per-layer timing of the packed-weight kernels on one GPU.

    python -m ixrun_b200.layer_bench --shape 5120x17408 --rows 1 --kernel gemv [--reps 50] [--eager-only]
    python -m ixrun_b200.layer_bench --sweep          # the shape / row-count sweep of the benchmark configs

For each case one JSON line: median microseconds (CUDA events on the launching
stream, an L2-sized buffer is overwritten between repetitions), packed-weight
GB/s on the reference's byte count, and the fraction of the measured HBM peak.
Kernels: decode (packed -> bf16), gemv (CUDA-core fused, 1..8 rows), gemm
(tensor-core fused, 1..64 rows), dense (bf16 matmul on decoded weights, the
"cached mode" of the reference).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .p5 import P5Packed
from .p6 import P6Packed
from .packed import DevicePacked
from .synth import synthetic_packed

SWEEP_SHAPES = [(5120, 17408), (17408, 5120), (5120, 5120), (1024, 5120), (2048, 2048)]


def _peak():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
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


def run_case(dp: DevicePacked, total_bytes: int, kernel: str, rows: int, reps: int, flush, wdense=None, p5=None):
    out_f, in_f = dp.out_f, dp.in_f
    x = torch.randn(rows, in_f, device=dp.device).bfloat16()
    y = torch.empty(rows, out_f, dtype=torch.bfloat16, device=dp.device)
    if kernel == "gemv":
        fn = lambda: dp.gemv(x, out=y)
    elif kernel in ("p5", "p6"):
        fn = lambda: p5.gemv(x, out=y)
    elif kernel in ("p5decode", "p6decode"):
        w = torch.empty(out_f * in_f, dtype=torch.bfloat16, device=dp.device)
        fn = lambda: p5.decode(out=w)
    elif kernel == "gemm":
        fn = lambda: dp.gemm(x, out=y)
    elif kernel == "decode":
        w = torch.empty(out_f * in_f, dtype=torch.bfloat16, device=dp.device)
        fn = lambda: dp.decode(out=w)
    elif kernel == "dense":
        fn = lambda: torch.nn.functional.linear(x, wdense, out=None)
    else:
        raise ValueError(kernel)
    us = time_us(fn, reps, flush)
    alg = total_bytes + 2 * in_f * rows + 2 * out_f * rows
    gbs = alg / us / 1e3
    return {"shape": f"{out_f}x{in_f}", "rows": rows, "kernel": kernel, "us": round(us, 2),
            "packed_GBps": round(gbs, 1), "frac_of_measured_hbm_peak": round(gbs / _peak(), 4),
            "Gelem_per_s": round(out_f * in_f / us / 1e3, 1)}


def run_graph_case(dp: DevicePacked, total_bytes: int, kernel: str, rows: int, reps: int, first, pdl=False):
    """Device time per launch with the launches back to back in a CUDA graph, over 4 copies of the layer."""
    cls = P5Packed if kernel == "p5" else P6Packed
    copies = [first] + [cls.from_packed(dp) for _ in range(3)]
    x = torch.randn(rows, dp.in_f, device=dp.device).bfloat16()
    y = torch.empty(rows, dp.out_f, dtype=torch.bfloat16, device=dp.device)
    for c in copies:
        c.gemv(x, out=y)
    torch.cuda.synchronize()
    if pdl:
        from .p6 import set_pdl
        set_pdl(True)
    n = 20
    st = torch.cuda.Stream()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        with torch.cuda.graph(g, stream=st):
            for i in range(n):
                copies[i % 4].gemv(x, out=y)
    ts = []
    for _ in range(max(reps, 5)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) * 1e3 / n)
    ts.sort()
    us = ts[len(ts) // 2]
    alg = total_bytes + 2 * dp.in_f * rows + 2 * dp.out_f * rows
    gbs = alg / us / 1e3
    if pdl:
        set_pdl(False)
    return {"shape": f"{dp.out_f}x{dp.in_f}", "rows": rows, "kernel": kernel + (" (graph, pdl)" if pdl else " (graph)"), "us": round(us, 2),
            "us_min": round(ts[0], 2), "packed_GBps": round(gbs, 1), "frac_of_measured_hbm_peak": round(gbs / _peak(), 4),
            "resident_bytes": first.resident_bytes}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="5120x17408")
    ap.add_argument("--rows", type=int, default=1)
    ap.add_argument("--kernel", default="gemv", choices=["gemv", "p5", "p5decode", "p6", "p6decode", "gemm", "decode", "dense"],
                    help="gemv/gemm/decode: kernels on the reference's streams; p5/p5decode, p6/p6decode: on the resident "
                         "P5 / P6 re-layout; "
                         "dense: bf16 matmul on decoded weights")
    ap.add_argument("--reps", type=int, default=30)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--pdl", action="store_true", help="p6 with --graph: programmatic dependent launch between the launches")
    ap.add_argument("--graph", action="store_true",
                    help="p5/p6: time 20 launches captured in one CUDA graph, rotating over 4 copies of the layer "
                         "(no host launch gaps, weights never served from L2)")
    args = ap.parse_args()
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if not args.sweep:
        out_f, in_f = (int(v) for v in args.shape.split("x"))
        p = synthetic_packed(out_f, in_f, seed=1)
        dp = DevicePacked(p)
        wd = dp.decode(kind="bf16").clone() if args.kernel == "dense" else None
        p5 = P5Packed.from_packed(dp) if args.kernel.startswith("p5") else None
        if args.kernel.startswith("p6"):
            p5 = P6Packed.from_packed(dp)
        if args.graph and args.kernel in ("p5", "p6"):
            print(json.dumps(run_graph_case(dp, p["total_bytes"], args.kernel, args.rows, args.reps, p5,
                                            pdl=args.pdl and args.kernel == "p6")), flush=True)
            return
        print(json.dumps(run_case(dp, p["total_bytes"], args.kernel, args.rows, args.reps, flush, wd, p5)), flush=True)
        return
    for out_f, in_f in SWEEP_SHAPES:
        p = synthetic_packed(out_f, in_f, seed=1)
        dp = DevicePacked(p)
        wd = dp.decode(kind="bf16").clone()
        p5 = P5Packed.from_packed(dp)
        big = out_f * in_f > 50e6
        for rows in ([1, 2, 4, 8, 16, 32, 64] if big else [1]):
            kernels = (["p5", "gemv"] if rows <= 8 else []) + (["gemm"] if rows >= 8 and in_f % 1024 == 0 else []) + ["dense"]
            for k in kernels:
                print(json.dumps(run_case(dp, p["total_bytes"], k, rows, args.reps, flush, wd, p5)), flush=True)
        print(json.dumps(run_case(dp, p["total_bytes"], "decode", 1, args.reps, flush)), flush=True)
        print(json.dumps(run_case(dp, p["total_bytes"], "p5decode", 1, args.reps, flush, None, p5)), flush=True)


if __name__ == "__main__":
    main()
