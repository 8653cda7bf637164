"""TPAB tile format through this library: decode bit-exact against the reference's own decode (golden fixtures) and the
oracle, GEMV within fp32 rounding of the reference's matmul on the decoded weights."""
import os

import numpy as np
import pytest
import torch

from oracle import ixb_oracle as O

pytestmark = pytest.mark.gpu

CASES = ["tpab_128x256", "tpab_48x192", "tpab_64x512", "tpab_64x128"]


def as_packed(d):
    f16 = lambda a: torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.float16)
    return {"shape": (int(d["out_f"]), int(d["in_f"])), "tile_r": int(d["tile_r"]), "tile_c": 64, "T": int(d["T"]),
            "n_per": int(d["n_per"]), "bits": torch.from_numpy(d["bits"]), "scales": f16(d["scales"]),
            "goff": torch.from_numpy(d["goff"]), "gbase_bit": torch.from_numpy(d["gbase_bit"]),
            "bodies": [torch.from_numpy(d["body"])], "ol_t": torch.from_numpy(d["ol_t"]), "ol_l": torch.from_numpy(d["ol_l"]),
            "ol_val": f16(d["ol_val"])}


def bf16_bits(t):
    return t.cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


@pytest.mark.parametrize("name", CASES)
def test_tpab_decode_and_gemv_golden(golden_dir, name):
    from ixrun_b200.tpab import decode_tpab_triton, fused_gemv_tpab, prepare_gemv_stage, stage_gpu

    d = np.load(os.path.join(golden_dir, name + ".npz"))
    p = as_packed(d)
    st = stage_gpu(p)
    w = decode_tpab_triton(p, staged=st)
    assert np.array_equal(bf16_bits(w), d["decoded"])
    gs = prepare_gemv_stage(p, staged=st)
    x = torch.from_numpy(np.ascontiguousarray(d["x"]).view(np.int16)).view(torch.bfloat16).cuda()
    out_f, in_f = p["shape"]
    y32 = fused_gemv_tpab(x, gs, out_f, in_f, p["tile_r"], out_dtype=torch.float32)
    ref = d["y"]
    assert np.abs(y32.cpu().numpy() - ref).max() <= 2e-5 * np.abs(ref).max()
    y = fused_gemv_tpab(x, gs, out_f, in_f, p["tile_r"])
    assert torch.equal(y, y32.bfloat16())
    bias = torch.randn(out_f).bfloat16().cuda()
    assert torch.equal(fused_gemv_tpab(x, gs, out_f, in_f, p["tile_r"], bias=bias), y + bias)
    assert torch.equal(fused_gemv_tpab(x, gs, out_f, in_f, p["tile_r"], out_dtype=torch.float32), y32)     # reproducible


def synthetic_tpab(out_f, in_f, seed, outliers=0.01):
    """A TPAB packed dict from a seeded tensor with random widths per tile (an encoder for tests: widths are not
    searched, every tile gets scale = max / qmax in fp16 and rounded fields)."""
    rng = np.random.default_rng(seed)
    tile_r = 64
    while out_f % tile_r:
        tile_r //= 2
    t_r, t_c = out_f // tile_r, in_f // 64
    T, n_per = t_r * t_c, tile_r * 64
    w = (rng.standard_normal((out_f, in_f)) * 0.02).astype(np.float32)
    v = w.reshape(t_r, tile_r, t_c, 64).transpose(0, 2, 1, 3).reshape(T, n_per)
    is_ol = rng.random((T, n_per)) < outliers
    v = np.where(is_ol, v * 9.0, v)
    v2 = np.where(is_ol, 0.0, v)
    bits = rng.integers(2, 7, size=T).astype(np.uint8)
    qmax = (1 << (bits.astype(np.int64) - 1)) - 1
    scales = (np.abs(v2).max(axis=1) / qmax).astype(np.float16)
    q = np.clip(np.rint(v2 / np.maximum(scales.astype(np.float32), 1e-12)[:, None]), -qmax[:, None], qmax[:, None]).astype(np.int64)
    goff = np.zeros(T, dtype=np.int32)
    gbase = np.zeros(7, dtype=np.int32)
    words, cursor = [], 0
    for b in (2, 3, 4, 5, 6):
        idx = np.nonzero(bits == b)[0]
        gbase[b] = cursor
        if idx.size == 0:
            continue
        goff[idx] = np.arange(idx.size, dtype=np.int32) * n_per
        fields = (q[idx] + qmax[idx][:, None]).reshape(-1).astype(np.uint64)
        pos = np.arange(fields.size, dtype=np.uint64) * np.uint64(b)
        nw = (fields.size * b + 31) // 32
        acc = np.zeros(nw + 1, dtype=np.uint64)
        np.bitwise_or.at(acc, (pos >> np.uint64(5)).astype(np.int64), (fields << (pos & np.uint64(31))) & np.uint64(0xFFFFFFFF))
        np.bitwise_or.at(acc, (pos >> np.uint64(5)).astype(np.int64) + 1, (fields << (pos & np.uint64(31))) >> np.uint64(32))
        words.append(acc[:nw].astype(np.uint32))
        cursor += idx.size * n_per * b
    ol_t, ol_l = np.nonzero(is_ol)
    d = {"out_f": out_f, "in_f": in_f, "tile_r": tile_r, "T": T, "n_per": n_per, "bits": bits,
         "scales": scales.view(np.uint16), "goff": goff, "gbase_bit": gbase, "body": np.concatenate(words).view(np.int32),
         "ol_t": ol_t.astype(np.int32), "ol_l": ol_l.astype(np.int32), "ol_val": v[ol_t, ol_l].astype(np.float16).view(np.uint16)}
    return d


@pytest.mark.parametrize("out_f,in_f", [(5120, 1024), (48, 5120), (1024, 17408), (96, 64)])
def test_tpab_against_the_oracle_at_larger_shapes(out_f, in_f):
    from ixrun_b200.tpab import decode_tpab_triton, fused_gemv_tpab, prepare_gemv_stage, stage_gpu

    d = synthetic_tpab(out_f, in_f, seed=out_f + in_f)
    p = as_packed(d)
    st = stage_gpu(p)
    assert np.array_equal(bf16_bits(decode_tpab_triton(p, staged=st)), O.tpab_decode_bf16(d))
    xb = O.f32_to_bf16_bits(np.random.default_rng(1).standard_normal(in_f).astype(np.float32))
    ref = O.tpab_gemv_f32(d, xb)
    x = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).cuda()
    y32 = fused_gemv_tpab(x, prepare_gemv_stage(p, staged=st), out_f, in_f, p["tile_r"], out_dtype=torch.float32)
    assert np.abs(y32.cpu().numpy() - ref).max() <= 2e-5 * np.abs(ref).max()
