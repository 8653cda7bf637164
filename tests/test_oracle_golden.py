"""The CPU oracle against fixtures made by the reference's own code
(tests/golden/make_golden.py).  Everything here is bit-exact except the
matmul, which is compared at 1e-5 relative (different fp32 summation order)."""
import hashlib
import json
import os

import numpy as np
import pytest

from oracle import ixb_oracle as O

CASES = ["core_128x256", "heavy_64x1024", "allzero_8x128", "ternary_16x128",
         "laplace_32x2048", "ragged_10x96"]


def load(golden_dir, name):
    return dict(np.load(os.path.join(golden_dir, name + ".npz")))


@pytest.mark.parametrize("name", CASES)
def test_quantize_and_pack_match_reference(golden_dir, name):
    g = load(golden_dir, name)
    w = g["w_bits"]
    p = O.quantize(w)
    assert p["scale"] == int(g["scale_bits"][0])
    assert p["counts"] == [int(c) for c in g["counts"]]
    assert p["total_bytes"] == int(g["total_bytes"][0])
    codes, _ = O.quantize_bf16(w)
    assert np.array_equal(codes, g["codes"])
    for mine, ref in zip(p["bitmaps"] + p["streams"], [g["b1"], g["b2"], g["l1"], g["l2"], g["l3"]]):
        assert mine.dtype == ref.dtype and np.array_equal(mine, ref)


def ref_packed(g):
    out_f, in_f = g["w_bits"].shape
    return {"level_bits": (3, 5, 8), "out_f": out_f, "in_f": in_f, "N": out_f * in_f,
            "scale": int(g["scale_bits"][0]), "bitmaps": [g["b1"], g["b2"]],
            "streams": [g["l1"], g["l2"], g["l3"]], "counts": [int(c) for c in g["counts"]],
            "total_bytes": int(g["total_bytes"][0])}


@pytest.mark.parametrize("name", CASES)
def test_decode_matches_reference(golden_dir, name):
    g = load(golden_dir, name)
    p = ref_packed(g)
    codes = O.decode_codes(p)
    assert np.array_equal(codes, g["codes"])
    assert np.array_equal(O.decode_bf16(p), g["w_dec_bits"])
    # level-3 positions are where |code| >= 16 (compute_positions)
    assert np.array_equal(np.nonzero(np.abs(codes.astype(np.int32)) >= 16)[0], g["pos_l3"])


@pytest.mark.parametrize("name", CASES)
def test_prefix_tables_match_reference(golden_dir, name):
    g = load(golden_dir, name)
    p = ref_packed(g)
    if "blk_q1" in g:
        q1, q2 = O.prefixes(p, 1024)
        assert np.array_equal(q1, g["blk_q1"]) and np.array_equal(q2, g["blk_q2"])
    q1, q2 = O.prefixes(p, p["in_f"])
    assert np.array_equal(q1, g["row_q1"]) and np.array_equal(q2, g["row_q2"])
    if "chunk" in g:
        q1, q2 = O.prefixes(p, int(g["chunk"][0]))
        assert np.array_equal(q1, g["chunk_q1"]) and np.array_equal(q2, g["chunk_q2"])


@pytest.mark.parametrize("name", CASES)
def test_matmul_matches_reference(golden_dir, name):
    g = load(golden_dir, name)
    p = ref_packed(g)
    y = O.gemm_f32(g["codes"], p["scale"], g["x_bits"], p["out_f"], p["in_f"])
    ref = g["y_f32"]
    den = max(float(np.abs(ref).max()), 1e-30)
    assert float(np.abs(y - ref).max()) / den < 1e-5
    y2 = O.LayerCPU(p)(g["x_bits"])
    assert float(np.abs(y2 - ref).max()) / den < 1e-5


def test_bitpack_matches_reference(golden_dir):
    g = load(golden_dir, "bitpack")
    assert np.array_equal(O.pack_bits(g["v3"], 3), g["pk3"])
    assert np.array_equal(O.pack_bits(g["v5"], 5), g["pk5"])
    assert np.array_equal(O.unpack_bits(g["pk3"], 1000, 3), g["v3"])
    assert np.array_equal(O.unpack_bits(g["pk5"], 777, 5), g["v5"])


def test_full_size_tensor_hashes(golden_dir):
    """4096x4096 Laplace tensor: every stream the oracle packs hashes to what
    the reference packer produced, and the decode closes."""
    with open(os.path.join(golden_dir, "big_hashes.json")) as f:
        big = json.load(f)
    sha = lambda a: hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
    out_f, in_f = big["shape"]
    c = O.laplace_codes(out_f, in_f, seed=big["seed"])
    assert sha(c) == big["sha_codes"]
    wb = O.codes_to_weight_bits(c).reshape(out_f, in_f)
    p = O.quantize(wb)
    assert p["scale"] == big["scale_bits"] and p["counts"] == big["counts"]
    assert p["total_bytes"] == big["total_bytes"]
    for k, a in zip(["b1", "b2", "l1", "l2", "l3"], p["bitmaps"] + p["streams"]):
        assert sha(a) == big["sha_" + k], k
    assert np.array_equal(O.decode_codes(p), c)
    assert sha(O.decode_bf16(p)) == big["sha_w_dec"]
    q1, q2 = O.prefixes(p, 1024)
    assert sha(q1) == big["sha_blk_q1"] and sha(q2) == big["sha_blk_q2"]


def test_group_scale_sibling_format_golden(golden_dir):
    """The oracle's restatement of the group-scale format against the reference's own decode (fixture written by
    tests/golden/make_ixgs_golden.py from ixgs.quantize.decode_weight_scatter)."""
    d = np.load(os.path.join(golden_dir, "ixgs_48x320.npz"))
    p = {k: d[k] for k in d.files}
    got = O.ixgs_decode_bf16(p)
    assert np.array_equal(got, d["decoded"])


@pytest.mark.parametrize("name", ["tpab_128x256", "tpab_48x192", "tpab_64x512", "tpab_64x128"])
def test_tpab_tile_format_golden(golden_dir, name):
    """The oracle's restatement of the TPAB tile format against the reference's own decode and matmul (fixtures written
    by tests/golden/make_tpab_golden.py from ixrun.tpab.encode_tpab / decode_tpab_ref)."""
    d = np.load(os.path.join(golden_dir, name + ".npz"))
    p = {k: d[k] for k in d.files}
    assert np.array_equal(O.tpab_decode_bf16(p), d["decoded"])
    y = O.tpab_gemv_f32(p, d["x"])
    assert np.abs(y - d["y"]).max() <= 1e-5 * np.abs(d["y"]).max()
