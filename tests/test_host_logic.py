"""CPU-only checks of the package's host side: the quantiser/packer against the
reference fixtures, argument validation, and the C-ABI library's exports."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from ixrun_b200 import quantize as Q

CASES = ["core_128x256", "heavy_64x1024", "allzero_8x128", "ternary_16x128",
         "laplace_32x2048", "ragged_10x96"]


def bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).view(torch.bfloat16)


@pytest.mark.parametrize("name", CASES)
def test_int8x_quantize_matches_reference_fixture(golden_dir, name):
    g = dict(np.load(os.path.join(golden_dir, name + ".npz")))
    p = Q.int8x_quantize(bf16(g["w_bits"]))
    assert p["level_bits"] == (3, 5, 8)
    assert p["counts"] == [int(c) for c in g["counts"]]
    assert p["total_bytes"] == int(g["total_bytes"][0])
    assert p["scale"].dtype == torch.bfloat16 and p["scale"].dim() == 0
    assert int(p["scale"].view(torch.int16).item()) & 0xFFFF == int(g["scale_bits"][0])
    for t, k in zip(p["bitmaps"] + p["streams"], ["b1", "b2", "l1", "l2", "l3"]):
        assert t.numpy().dtype == g[k].dtype and np.array_equal(t.numpy(), g[k]), k
    assert abs(p["bits_per_weight"] - p["total_bytes"] * 8 / p["N"]) < 1e-12
    # packing the fixture's codes with the fixture's scale gives the same dict
    p2 = Q.pack_codes(g["codes"], p["scale"], p["out_f"], p["in_f"])
    for a, b in zip(p["bitmaps"] + p["streams"], p2["bitmaps"] + p2["streams"]):
        assert torch.equal(a, b)


def test_pack_fields_multi_chunk():
    """more values than one packing chunk (2**22): chunk seams stay bit-exact"""
    from oracle import ixb_oracle as O

    rng = np.random.default_rng(0)
    v = rng.integers(0, 8, size=(1 << 22) + 12345).astype(np.int32)
    assert np.array_equal(Q._pack_fields(v, 3), O.pack_bits(v, 3))
    v5 = rng.integers(0, 32, size=70001).astype(np.int32)
    assert np.array_equal(Q._pack_fields(v5, 5), O.pack_bits(v5, 5))


def test_quantize_argument_errors():
    w = torch.zeros(4, 32).bfloat16()
    with pytest.raises(ValueError):
        Q.int8x_quantize(w, (3, 5, 7))          # last level must be 8
    with pytest.raises(ValueError):
        Q.int8x_quantize(w, (2, 4, 8))          # only (3,5,8) is built
    with pytest.raises(ValueError):
        Q.int8x_quantize(torch.zeros(4).bfloat16())
    with pytest.raises(ValueError):
        Q.pack_codes(np.zeros(5, dtype=np.int8), torch.tensor(1.0), 2, 3)


def test_split_policy_matches_reference():
    from ixrun_b200.fused import _pick_split

    assert _pick_split(17408) == 2 and _pick_split(4608) == 1 and _pick_split(6144) == 2
    assert _pick_split(1536) == 1 and _pick_split(2048) == 2


def test_library_exports_every_declared_symbol():
    from ixrun_b200 import _lib, build

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = open(os.path.join(root, "include", "ixb200.h")).read()
    declared = set(re.findall(r"\b(ixb_[a-z0-9_]+)\s*\(", hdr))
    assert declared, "no declarations found"
    so = build.build()
    lib = ctypes.CDLL(so)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/ixb200.h but not exported"
    assert declared == set(_lib.SYMBOLS)
    lib.ixb_version.restype = ctypes.c_int
    assert lib.ixb_version() >= 100


def test_bad_arguments_are_reported_without_a_gpu():
    """argument validation happens before any CUDA call"""
    from ixrun_b200 import _lib

    L = _lib.lib()
    p = _lib.Packed()          # all NULL / zero
    rc = L.ixb_decode(ctypes.byref(p), None, None, None, 1, None)
    assert rc == 1 and b"shape" in L.ixb_last_error()
    assert L.ixb_gemv_scratch_bytes(0, 32, 1) == 0
    assert L.ixb_prefix_workspace_bytes(4096) >= 4 * 4 * 4


def test_no_cpu_fallback():
    if torch.cuda.is_available():
        pytest.skip("needs a box without a GPU")
    from ixrun_b200 import _lib
    from ixrun_b200.packed import DevicePacked

    p = Q.int8x_quantize(torch.randn(4, 64).bfloat16())
    with pytest.raises(_lib.IxbError):
        DevicePacked(p)


def test_ctypes_prototypes_match_the_header():
    """Every function declared in include/ixb200.h has a ctypes prototype with the same number of parameters, and the
    mirrored structs have the header's field count (an ABI drift between header, library and binding fails here, on
    the CPU)."""
    from ixrun_b200 import _lib

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    hdr = open(os.path.join(root, "include", "ixb200.h")).read()
    hdr_nc = re.sub(r"/\*.*?\*/", "", hdr, flags=re.S)                     # without comments
    L = _lib.lib()
    decls = re.findall(r"\b(?:int|size_t|int64_t|const char \*|unsigned long long)\s*\**\s*(ixb_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;", hdr_nc, flags=re.S)
    assert len(decls) >= 30
    for name, args in decls:
        args = args.strip()
        n = 0 if args in ("", "void") else len([a for a in args.split(",") if a.strip()])
        fn = getattr(L, name)
        if n == 0 and fn.argtypes is None:
            continue
        assert fn.argtypes is not None, f"{name} has no ctypes prototype"
        assert len(fn.argtypes) == n, f"{name}: header has {n} parameters, the binding {len(fn.argtypes)}"
    for struct, mirror in (("ixb_packed", _lib.Packed), ("ixb_p6", _lib.P6Struct), ("ixb_tpab", _lib.TpabStruct)):
        body = re.search(r"typedef struct " + struct + r"\s*\{(.*?)\}\s*" + struct + r"\s*;", hdr_nc, flags=re.S).group(1)
        fields = [f for f in body.split(";") if f.strip()]
        assert len(fields) == len(mirror._fields_), f"{struct}: header has {len(fields)} fields, the mirror {len(mirror._fields_)}"
