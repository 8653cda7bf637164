"""Benchmark of the INT8-X hot path: batch-1 fused decode+GEMV over the packed
down_proj tensor (5120 x 17408), reported as packed-weight GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one pass of y = W x over the whole packed tensor.  Algorithmic bytes
per step = the reference's `total_bytes` of the packed tensor + 2*in_f (x) +
2*out_f (y); rank tables and padding are not counted.  Timed steps rotate over
enough device copies of the layer (at least 256 MB per GPU, whatever the shard
size) that every step reads its weights from HBM.  The K steps are captured in
one CUDA graph, which is replayed until the timed region is at least 50 ms long;
`ms_per_step` is the device time of all replays divided by their steps.  At
N > 1 the tensor is split by columns (row-parallel linear: each rank owns
in_f/N columns of every row) and the partial outputs are summed by one kernel
over peer memory per step (NCCL with --nccl); the summed output is checked
against the unsharded layer.  Unless --no-model is given the line also carries
`model_27b`: ms per token of the tensor-parallel 27B-class hybrid decoder (real
token mixers, 4096 positions of context, greedy feedback on the device) at the
same N.

`--impl reference` times the CPU port of the reference's own layer path (decode
to bf16, then matmul) on the host cores instead.
"""
from __future__ import annotations

import contextlib

import argparse
import json
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

OUT_F, IN_F = 5120, 17408
MIN_ROTATING_BYTES = 256 << 20      # weights that the timed steps rotate over, per GPU (twice the L2)
MIN_TIMED_MS = 50.0
METRIC = "fused decode+GEMV packed-weight bandwidth (batch 1)"
UNIT = "GB/s"



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

def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, an earlier copy-bandwidth measurement on B200)"


class ClockSampler(threading.Thread):
    """Polls SM clock and throttle reasons through NVML while a region runs."""

    def __init__(self, index: int, period_s: float = 0.01):
        super().__init__(daemon=True)
        self.index, self.period, self.samples, self.reasons = index, period_s, [], set()
        self.max_mhz = None
        self._stop_evt = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _once(self):
        nv = self.nv
        self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
        try:
            r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
        except Exception:
            r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
        names = {
            "hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20,
            "hw_thermal_slowdown": 0x40, "hw_power_brake_slowdown": 0x80,
        }
        for k, bit in names.items():
            if r & bit:
                self.reasons.add(k)

    def run(self):
        if self.nv is None:
            return
        while not self._stop_evt.is_set():
            try:
                self._once()
            except Exception:
                break
            time.sleep(self.period)

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=2)
        if self.nv is not None and not self.samples:
            try:
                self._once()
            except Exception:
                pass
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def algorithmic_bytes(total_bytes: int) -> int:
    return total_bytes + 2 * IN_F + 2 * OUT_F


# ----------------------------------------------------------------- CPU arm ---
def cpu_layer_gbs(steps: int, warmup: int, seed: int = 0):
    """Oracle port of the reference's CPU layer path on the host cores."""
    from ixrun_b200.synth import laplace_codes
    from oracle import ixb_oracle as O

    # torchrun pins OMP_NUM_THREADS=1 for its ranks, and the OpenMP runtime has read it by now; the CPU arm is meant
    # to use every host core
    if os.environ.get("OMP_NUM_THREADS") == "1" and "TORCHELASTIC_RUN_ID" in os.environ:
        O.set_num_threads(os.cpu_count() or 1)

    codes = laplace_codes(OUT_F, IN_F, seed)
    sc = int(O.f32_to_bf16_bits(np.array([2.0 ** -9], dtype=np.float32))[0])
    p = O.pack_codes(codes, OUT_F, IN_F, sc)
    layer = O.LayerCPU(p)
    x = O.f32_to_bf16_bits(np.random.default_rng(1).standard_normal((1, IN_F)).astype(np.float32))
    for _ in range(warmup):
        layer(x)
    t0 = time.perf_counter()
    for _ in range(steps):
        layer(x)
    dt = (time.perf_counter() - t0) / steps
    return algorithmic_bytes(p["total_bytes"]) / dt / 1e9, dt, O.num_threads()


WORKLOAD = f"down_proj {OUT_F}x{IN_F} batch 1 fused decode+GEMV, (3,5,8) codes ~ round(Laplace(0,4.4))"


def run_reference(args):
    """The reference's CPU layer path (decode to bf16, then matmul) on all host cores: K steps after W warm-up steps,
    each one full 5120 x 17408 layer (about half a second), rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(0, args.warmup)
    if steps > 200:                          # the GPU arm's default step count would take minutes here
        steps = 20
    gbs, dt, cores = cpu_layer_gbs(steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "algorithmic_bytes_per_step": algorithmic_bytes_full(),
                   "path": "CPU port of the reference layer path: decode to bf16, then matmul, host cores"},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"{steps} full {OUT_F}x{IN_F} layers"},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


_FULL_BYTES = None


def algorithmic_bytes_full() -> int:
    global _FULL_BYTES
    if _FULL_BYTES is None:
        from ixrun_b200.quantize import pack_codes
        from ixrun_b200.synth import laplace_codes

        codes = laplace_codes(OUT_F, IN_F, seed=0)
        _FULL_BYTES = algorithmic_bytes(pack_codes(codes, torch.tensor(2.0 ** -9, dtype=torch.bfloat16), OUT_F, IN_F)["total_bytes"])
    return _FULL_BYTES


# ----------------------------------------------------------------- GPU arm ---
def run_gpu(args):
    import torch.distributed as dist

    from ixrun_b200 import _lib
    from ixrun_b200.engine import StreamingLinear
    from ixrun_b200.p6 import set_pdl
    from ixrun_b200.quantize import pack_codes
    from ixrun_b200.synth import laplace_codes

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        with _stdout_to_stderr():        # NCCL prints its version line to stdout; stdout is for the one JSON line
            dist.init_process_group("nccl", device_id=dev)
            dist.barrier()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")

    # ---- synthetic layer, column shard of this rank
    codes = laplace_codes(OUT_F, IN_F, seed=0).reshape(OUT_F, IN_F)
    scale = torch.tensor(2.0 ** -9, dtype=torch.bfloat16)
    full_packed = pack_codes(codes.reshape(-1), scale, OUT_F, IN_F) if (world > 1 and rank == 0) or world == 1 else None
    in_loc = IN_F // world
    if world > 1:
        shard = np.ascontiguousarray(codes[:, rank * in_loc:(rank + 1) * in_loc])
        packed = pack_codes(shard.reshape(-1), scale, OUT_F, in_loc)
    else:
        packed = full_packed
    alg_bytes = algorithmic_bytes_full()
    alg_bytes_rank = packed["total_bytes"] + 2 * in_loc + 2 * OUT_F
    first = StreamingLinear(packed, resident=args.layout)
    resident_bytes = first.resident_bytes
    copies = max(4, -(-MIN_ROTATING_BYTES // resident_bytes) + 1)      # the rotating set exceeds twice the L2 at every N
    layers = [first] + [StreamingLinear(packed, resident=args.layout) for _ in range(copies - 1)]
    g = torch.Generator().manual_seed(1)
    x_full = torch.randn(1, IN_F, generator=g).bfloat16()
    x_host = x_full[:, rank * in_loc:(rank + 1) * in_loc].contiguous().pin_memory()
    x = x_host.to(dev)
    y32 = torch.empty(1, OUT_F, dtype=torch.float32, device=dev)
    y16 = torch.empty(1, OUT_F, dtype=torch.bfloat16, device=dev)

    # several GPUs: the fp32 partial outputs are summed by one kernel of this library over peer memory
    # (graph-capturable); --nccl keeps the eager NCCL all-reduce
    ar = None
    ar_note = None
    if world > 1 and not args.nccl:
        from ixrun_b200.parallel import PeerAllReduce

        try:
            ar = PeerAllReduce(OUT_F, dev)
            # self-check against NCCL on one random vector per rank; on any difference beyond fp32 rounding, or a
            # wait that gave up, every rank falls back to the NCCL all-reduce together
            v = torch.randn(1, OUT_F, device=dev, generator=torch.Generator(device=dev).manual_seed(100 + rank))
            got = ar(v, out_dtype=torch.float32)
            ref = v.clone()
            dist.all_reduce(ref)
            bad = torch.tensor([float((got - ref).abs().max() > 1e-5 * ref.abs().max() or ar.timed_out())], device=dev)
        except Exception as exc:       # no symmetric memory between these GPUs: every rank fails the same way
            ar = None
            ar_note = f"disabled: {type(exc).__name__}: {exc}"[:200]
            bad = torch.tensor([1.0], device=dev)
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if bad.item() != 0:
            ar = None
            ar_note = ar_note or "disabled: the self-check against NCCL failed"

    def step(i):
        lay = layers[i % copies]
        if world > 1 and ar is not None and args.one_kernel:
            # ONE kernel: the shard GEMV stores its partial sums into every rank's buffer as its tiles finish, then
            # its warps add up all ranks' words
            lay._res.gemv_allreduce(x, ar, out=y16)
        elif world > 1 and ar is not None:
            # the GEMV's epilogue stores the partial sums into every rank's buffer; a small second kernel adds them
            ar.finish(lay._res.gemv_push(x, ar), y16)
        elif world > 1:
            lay.matvec(x, out=y32)
            dist.all_reduce(y32)
            y16.copy_(y32)
        else:
            lay.matvec(x, out=y16)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()

    # ---- the step's result against the unsharded layer (rank 0 holds it)
    tp_check = None
    if world > 1:
        y_tp = y16.float().cpu()
        if rank == 0:
            ref_layer = StreamingLinear(full_packed, resident=args.layout)
            y_ref = ref_layer.matvec(x_full.to(dev), out_dtype=torch.float32).cpu()
            tp_check = {"max_rel_err_vs_unsharded": float((y_tp - y_ref).abs().max() / y_ref.abs().max()),
                        "tolerance": "one bf16 rounding of the output (2^-8 relative to the largest element)",
                        "exchange": "peer stores from the GEMV epilogue + finishing kernel" if ar is not None else "NCCL all-reduce"}
            del ref_layer
        barrier()

    use_graph = (world == 1 or ar is not None) and not args.eager

    def capture():
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step(0)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for i in range(args.steps):
                step(i)
        gr.replay()         # untimed: the first replay uploads the graph
        torch.cuda.synchronize()
        return gr

    def timed(gr, replays, sampler=None):
        """Device time of `replays` replays of the K-step graph (or of K eager steps), max over ranks, in ms."""
        barrier()
        if sampler is not None:
            sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            if gr is not None:
                gr.replay()
            else:
                for i in range(args.steps):
                    step(i)
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def replays_for(gr):
        """Replays that make the timed region at least MIN_TIMED_MS long (the same number on every rank)."""
        one = timed(gr, 1)
        return max(1, int(MIN_TIMED_MS / max(one, 1e-3)) + 1)

    # ---- timed region: R replays of the K steps, programmatic dependent launch on (layout p6)
    pdl = args.layout == "p6" and not args.no_pdl
    launch_ms_no_pdl = None
    if pdl and use_graph and world == 1:
        # the same graph without programmatic dependent launch, for the record
        g0 = capture()
        r0 = replays_for(g0)
        launch_ms_no_pdl = timed(g0, r0) / (r0 * args.steps)
        del g0
    if pdl:
        # deployment is complete and the device idle: from here on a GEMV launch may fetch its first weight blocks
        # while the kernel ahead of it in the stream finishes (it still waits for that kernel before it reads x)
        set_pdl(True)
    graph = capture() if use_graph else None
    replays = replays_for(graph)
    launches0 = _lib.lib().ixb_launch_count()
    sampler = ClockSampler(local)
    ms = timed(graph, replays, sampler)
    clocks = sampler.stop()
    total_steps = replays * args.steps
    launches = total_steps * (2 if ar is not None and (not args.one_kernel) else 1) if graph is not None else _lib.lib().ixb_launch_count() - launches0
    ms_per_step = ms / total_steps
    value = alg_bytes / (ms_per_step * 1e-3) / 1e9
    if clocks.get("sm_mhz"):
        clocks["ms_per_step_x_mhz"] = ms_per_step * clocks["sm_mhz"]

    # ---- dominant kernel alone (rank-local shard): one launch at a time, CUDA events on the launching stream
    kt = []
    for i in range(50):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        layers[i % copies].matvec(x, out=y16)
        b.record()
        b.synchronize()
        kt.append(a.elapsed_time(b))
    kernel_ms_eager = float(np.median(kt))
    # roofline of the dominant kernel: at N = 1 a step IS one launch of it and the graph figure is its device time
    # without host gaps; at N > 1 a step also holds the all-reduce, so the eagerly launched kernel is reported
    k_ms = ms_per_step if (graph is not None and world == 1) else kernel_ms_eager
    peak, peak_src = measured_peak()
    achieved = alg_bytes_rank / (k_ms * 1e-3) / 1e9

    # ---- end to end through the module API with host buffers
    y_host = torch.empty(1, OUT_F, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(10, min(args.steps, 200))

    # single GPU: the module call sits in a CUDA graph over static buffers (engine.GraphedCall) together with the
    # H2D copy of x and the D2H copy of y, so a step is one graph launch and a stream synchronise
    graphed = None
    if world == 1 and not args.eager:
        from ixrun_b200.engine import GraphedCall

        graphed = [GraphedCall(lay, x, host_io=True) for lay in layers[:4]]

    def e2e_step(i):
        if graphed is not None:
            y_host.copy_(graphed[i % len(graphed)].run_host(x_host))
            return
        xd = x_host.to(dev, non_blocking=True)
        if world > 1 and ar is not None:
            y_host.copy_(ar.finish(layers[i % copies]._res.gemv_push(xd, ar), y16), non_blocking=True)
        elif world > 1:
            layers[i % copies].matvec(xd, out=y32)
            dist.all_reduce(y32)
            y_host.copy_(y32.to(torch.bfloat16), non_blocking=True)
        else:
            y_host.copy_(layers[i % copies](xd), non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for i in range(3):
        e2e_step(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(i)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    ar_timed_out = ar.timed_out() if ar is not None else ar_note

    # ---- the 27B-class hybrid stack at the same N (every rank takes part; rank 0 reports)
    model = None
    graph_used = graph is not None
    if not args.no_model:
        del layers, graphed, graph
        torch.cuda.empty_cache()
        from ixrun_b200 import hybrid27b

        try:
            model = hybrid27b.measure(world, rank, dev, tokens=args.model_tokens, nccl=args.nccl or (world > 1 and ar is None))
        except Exception as exc:      # reported, not hidden: the headline metric above stands on its own
            model = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {
            "workload": WORKLOAD,
            "algorithmic_bytes_per_step": alg_bytes,
            "layout": LAYOUT_TEXT[args.layout],
            "resident_bytes_per_gpu": resident_bytes,
            "l2": f"timed steps rotate over {copies} device copies of the weights ({copies * resident_bytes / 1e6:.0f} MB per GPU)",
            "parallelism": ("single GPU" if world == 1 else
                            f"tp{world}: column shards of in_f, fp32 partial outputs summed per step by " +
                            (("peer stores from the GEMV's epilogue + one finishing kernel (ixb_p6_gemv_push, ixb_allreduce_finish)" if (not args.one_kernel)
                              else "the GEMV kernel itself: peer stores from its epilogue, then its warps add all ranks' words (ixb_p6_gemv_allreduce)") if ar is not None
                             else "one NCCL all-reduce")),
            "timed_with": (f"CUDA events around {replays} replays of one graph of K launches" if graph_used
                           else f"CUDA events around {replays} x K eager steps"),
            "timed_region_ms": ms, "graph_replays": replays,
            "programmatic_dependent_launch": bool(pdl),
            "peer_allreduce_timed_out": ar_timed_out,
            "tp_check": tp_check,
        },
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": None, "peak_source": peak_src, "kernel": LAYOUT_KERNEL[args.layout],
                     "algorithmic_bytes_per_launch": alg_bytes_rank, "launch_ms": k_ms,
                     "launch_ms_no_pdl": launch_ms_no_pdl, "launch_ms_eager_median": kernel_ms_eager},
        "e2e": {"value": alg_bytes / e2e_s / 1e9, "unit": UNIT, "h2d_bytes_per_step": 2 * in_loc,
                "d2h_bytes_per_step": 2 * OUT_F, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                "call": ("engine.GraphedCall(StreamingLinear, host_io=True).run_host: one graph launch holding the H2D copy of x, "
                         "the GEMV and the D2H copy of y, then a stream synchronise" if world == 1 and not args.eager
                         else "StreamingLinear.matvec on a fresh device copy of pinned host x, y copied back")},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "model_27b": model,
    }
    if rank == 0:
        if world == 1:
            cpu_steps = 3
            gbs, dt, cores = cpu_layer_gbs(cpu_steps, 1)
            line["cpu_baseline"] = {"value": gbs, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"{cpu_steps} full {OUT_F}x{IN_F} layers, {dt * 1e3:.0f} ms each"}
        traffic = os.path.join(ROOT, "profiles", "gemv_traffic.json")
        if world == 1 and os.path.exists(traffic):
            with open(traffic) as f:
                line["roofline"]["traffic"] = json.load(f).get(line["roofline"]["kernel"], {}).get("dram_bytes_per_launch")
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


DEFAULT_LAYOUT = "p6"
LAYOUT_KERNEL = {"p6": "k_p6_mma<1>", "streams": "k_gemv<1>"}
LAYOUT_TEXT = {
    "p6": ("resident P6 re-layout of the same int8 codes (6-bit plane in mma fragment order whose fields are part of "
           "the bf16 number 1 + code/32, + a weight list for codes outside -16..31), built on the GPU at deploy time "
           "from the reference's packed streams"),
    "streams": "the reference's (3,5,8) streams read directly",
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--eager", action="store_true", help="launch the timed steps one by one instead of one CUDA graph")
    ap.add_argument("--nccl", action="store_true",
                    help="several GPUs: eager NCCL all-reduce instead of the one-kernel all-reduce over peer memory")
    ap.add_argument("--no-pdl", action="store_true",
                    help="layout p6: launch the GEMVs without programmatic dependent launch")
    ap.add_argument("--layout", default=DEFAULT_LAYOUT, choices=["p6", "streams"],
                    help="resident weight layout: the P6 re-layout, or the reference's streams read directly")
    ap.add_argument("--one-kernel", action="store_true",
                    help="several GPUs: finish the exchange inside the GEMV kernel (ixb_p6_gemv_allreduce) instead of in a "
                         "second small kernel, which measured faster because the next GEMV's prefetch overlaps it")
    ap.add_argument("--no-model", action="store_true", help="skip the model_27b sub-record (27B-class hybrid stack, ms per token)")
    ap.add_argument("--model-tokens", type=int, default=64, help="tokens decoded for the model_27b sub-record (256 is the configuration's count)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
