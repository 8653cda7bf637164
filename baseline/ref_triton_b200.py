"""Same-box baseline: the UNMODIFIED reference Triton kernels on this GPU, beside this library's kernels.

    sh baseline/install_ref.sh <reference checkout>   # once, where the reference tree is mounted
    python baseline/ref_triton_b200.py    # on the GPU box; one JSON line per shape, then a summary line

For every config-1 shape the reference's own quantiser packs the same synthetic weights, its
`ixrun.engine.StreamingLinear` runs the batch-1 forward (fused decode+GEMV Triton kernel, split-K for wide layers)
and `ixrun.triton_kernels.decode_weight_triton` decodes the tensor; this library's resident-layout GEMV runs on the
same packed dict.  Times are medians of CUDA-event timings with an L2-sized buffer overwritten between repetitions
(cold L2, launched eagerly: the reference has no graph mode for this path), so the two columns are like for like.
The outputs of the two paths are compared (relative to the largest output).
"""
from __future__ import annotations

import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
SHAPES = [(5120, 17408), (17408, 5120), (5120, 5120), (1024, 5120), (2048, 2048)]


def median_us(fn, reps, flush):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    ts.sort()
    return ts[len(ts) // 2]


def main():
    if not os.path.isdir(os.path.join(REF, "ixrun")):
        print(json.dumps({"unavailable": "baseline/_ref/ixrun is missing: run baseline/install_ref.sh <reference checkout> where the reference is mounted"}))
        return
    sys.path.insert(0, REF)
    sys.path.insert(0, ROOT)
    import ixrun.engine as ref_engine                      # the reference, unmodified
    from ixrun.quantize import int8x_quantize
    from ixrun.triton_kernels import decode_weight_triton

    from ixrun_b200.p6 import P6Packed
    from ixrun_b200.synth import codes_to_weight, laplace_codes

    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    reps = int(os.environ.get("REPS", "50"))
    out = []
    for out_f, in_f in SHAPES:
        codes = laplace_codes(out_f, in_f, 1)
        w = codes_to_weight(codes, out_f, in_f).cuda()
        packed = int8x_quantize(w)                          # the reference's packer
        lin = ref_engine.StreamingLinear(packed)
        x = torch.randn(1, in_f, device="cuda").bfloat16()
        y_ref = lin(x)
        torch.cuda.synchronize()
        fused = bool(getattr(lin, "_use_fused", False))
        us_ref = median_us(lambda: lin(x), reps, flush)
        us_dec = median_us(lambda: decode_weight_triton(packed, device="cuda"), max(5, reps // 5), flush)
        p6 = P6Packed.from_packed(packed)
        y = torch.empty(1, out_f, dtype=torch.bfloat16, device="cuda")
        us_p6 = median_us(lambda: p6.gemv(x, out=y), reps, flush)
        dense = torch.nn.functional.linear(x.float(), w.float())
        rel_ref = float((y_ref.float() - dense).abs().max() / dense.abs().max())
        rel_new = float((y.float() - dense).abs().max() / dense.abs().max())
        rel_pair = float((y.float() - y_ref.float()).abs().max() / dense.abs().max())
        rec = {"shape": f"{out_f}x{in_f}", "packed_bytes": int(packed["total_bytes"]),
               "reference_streaming_linear_us": round(us_ref, 1), "reference_used_fused_triton_gemv": fused,
               "reference_split_chunk": int(getattr(lin, "_split_chunk", 0) or 0),
               "reference_decode_weight_triton_us": round(us_dec, 1),
               "this_library_p6_gemv_us": round(us_p6, 1), "speedup": round(us_ref / us_p6, 1),
               "reference_packed_GBps": round(packed["total_bytes"] / us_ref / 1e3, 1),
               "this_library_packed_GBps": round(packed["total_bytes"] / us_p6 / 1e3, 1),
               "rel_err_reference_vs_fp32_matmul": rel_ref, "rel_err_this_library_vs_fp32_matmul": rel_new,
               "rel_diff_between_the_two": rel_pair}
        out.append(rec)
        print(json.dumps(rec), flush=True)
        del lin, p6, w, packed
        torch.cuda.empty_cache()
    import triton

    print(json.dumps({"summary": "reference Triton kernels, unmodified, same GPU, eager launches, cold L2",
                      "gpu": torch.cuda.get_device_name(0), "triton": triton.__version__, "torch": torch.__version__,
                      "reps": reps}), flush=True)


if __name__ == "__main__":
    main()
