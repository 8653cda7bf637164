"""numpy/ctypes front end of the CPU oracle (``oracle/ixb_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the
benchmark's cpu-baseline / reference arm.  The shipped package never imports
it.  Parity status: pinned against fixtures generated from the reference's own
Python code (``tests/golden/make_golden.py``).

All arrays are numpy; bf16 values travel as ``uint16`` bit patterns.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "libixb_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with gcc (``make -C oracle``); returns the .so path."""
    src = os.path.join(_HERE, "ixb_oracle.c")
    stale = (not os.path.exists(_SO)) or os.path.getmtime(_SO) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        p, i64, u16 = C.c_void_p, C.c_int64, C.c_uint16
        L.ixo_num_threads.restype = C.c_int
        L.ixo_quantize_bf16.restype = u16
        L.ixo_quantize_bf16.argtypes = [p, i64, p]
        L.ixo_count_levels.argtypes = [p, i64, p]
        L.ixo_stream_words.argtypes = [i64, p, p]
        L.ixo_total_bytes.restype = i64
        L.ixo_total_bytes.argtypes = [i64, p]
        L.ixo_pack.argtypes = [p, i64, p, p, p, p, p]
        L.ixo_prefixes.argtypes = [p, p, i64, i64, i64, p, p]
        L.ixo_decode_codes.argtypes = [p, p, p, i64, p, i64, p, i64, p, p, p]
        L.ixo_codes_to_bf16.argtypes = [p, i64, u16, p]
        L.ixo_gemm_f32.argtypes = [p, u16, p, i64, i64, i64, p]
        L.ixo_layer_cpu.argtypes = [p, p, p, i64, p, i64, p, u16, p, i64, i64, i64, p, p, p, p, p]
        L.ixo_pack_bits.argtypes = [p, i64, C.c_int, p]
        L.ixo_unpack_bits.argtypes = [p, i64, i64, C.c_int, p]
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().ixo_num_threads())


def set_num_threads(n: int) -> None:
    """Threads for the OpenMP loops of the oracle (overrides an OMP_NUM_THREADS read when the runtime was loaded)."""
    lib().ixo_set_num_threads(C.c_int(int(n)))


# ------------------------------------------------------------------ bf16 ---
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# -------------------------------------------------------------- quantise ---
def quantize_bf16(w_bits: np.ndarray):
    """bf16 weight bits [out_f, in_f] -> (int8 codes flat, scale bf16 bits)."""
    w = np.ascontiguousarray(w_bits, dtype=np.uint16).reshape(-1)
    codes = np.empty(w.size, dtype=np.int8)
    sc = lib().ixo_quantize_bf16(_ptr(w), w.size, _ptr(codes))
    return codes, int(sc)


def pack_codes(codes: np.ndarray, out_f: int, in_f: int, scale_bits: int) -> dict:
    """int8 codes -> packed dict with the reference's keys (numpy arrays)."""
    codes = np.ascontiguousarray(codes, dtype=np.int8).reshape(-1)
    n = codes.size
    assert n == out_f * in_f
    counts = np.zeros(3, dtype=np.int64)
    words = np.zeros(4, dtype=np.int64)
    L = lib()
    L.ixo_count_levels(_ptr(codes), n, _ptr(counts))
    L.ixo_stream_words(n, _ptr(counts), _ptr(words))
    b1 = np.zeros(int(words[0]), dtype=np.uint32)
    b2 = np.zeros(int(words[1]), dtype=np.uint32)
    l1 = np.zeros(int(words[2]), dtype=np.uint32)
    l2 = np.zeros(int(words[3]), dtype=np.uint32)
    l3 = np.zeros(int(counts[2]), dtype=np.uint8)
    # one spare word so the C packer's straddle write never leaves the buffer
    l1p = np.zeros(l1.size + 1, dtype=np.uint32)
    l2p = np.zeros(l2.size + 1, dtype=np.uint32)
    L.ixo_pack(_ptr(codes), n, _ptr(b1), _ptr(b2), _ptr(l1p), _ptr(l2p), _ptr(l3))
    l1[:] = l1p[: l1.size]
    l2[:] = l2p[: l2.size]
    total = int(L.ixo_total_bytes(n, _ptr(counts)))
    return {
        "level_bits": (3, 5, 8),
        "out_f": out_f,
        "in_f": in_f,
        "N": n,
        "scale": scale_bits,
        "bitmaps": [b1.view(np.int32), b2.view(np.int32)],
        "streams": [l1.view(np.int32), l2.view(np.int32), l3],
        "counts": [int(c) for c in counts],
        "total_bytes": total,
        "bits_per_weight": total * 8 / n,
        "compression_vs_bf16": n * 2 / total,
    }


def quantize(w_bits: np.ndarray) -> dict:
    out_f, in_f = w_bits.shape
    codes, sc = quantize_bf16(w_bits)
    return pack_codes(codes, out_f, in_f, sc)


# ---------------------------------------------------------------- decode ---
def _streams(p: dict):
    b1, b2 = (np.ascontiguousarray(a).view(np.uint32) for a in p["bitmaps"])
    l1 = np.ascontiguousarray(p["streams"][0]).view(np.uint32)
    l2 = np.ascontiguousarray(p["streams"][1]).view(np.uint32)
    l3 = np.ascontiguousarray(p["streams"][2], dtype=np.uint8)
    # the C readers may look at one word past a stream's last value
    pad = lambda a: np.concatenate([a, np.zeros(2, dtype=a.dtype)])
    return pad(b1), pad(b2), pad(l1), pad(l2), pad(l3), l1.size, l2.size


def prefixes(p: dict, gran: int, n_units: int | None = None):
    """Exclusive (#L1, #L2) counts before flat positions u*gran."""
    n = p["N"]
    if n_units is None:
        n_units = (n + gran - 1) // gran
    b1, b2, *_ = _streams(p)
    q1 = np.zeros(n_units, dtype=np.int32)
    q2 = np.zeros(n_units, dtype=np.int32)
    lib().ixo_prefixes(_ptr(b1), _ptr(b2), n, gran, n_units, _ptr(q1), _ptr(q2))
    return q1, q2


def decode_codes(p: dict) -> np.ndarray:
    n = p["N"]
    b1, b2, l1, l2, l3, l1w, l2w = _streams(p)
    out = np.empty(n, dtype=np.int8)
    nb = (n + 1023) // 1024
    s1 = np.empty(nb, dtype=np.int32)
    s2 = np.empty(nb, dtype=np.int32)
    lib().ixo_decode_codes(_ptr(b1), _ptr(b2), _ptr(l1), l1w, _ptr(l2), l2w, _ptr(l3), n,
                           _ptr(out), _ptr(s1), _ptr(s2))
    return out


def codes_to_bf16(codes: np.ndarray, scale_bits: int) -> np.ndarray:
    codes = np.ascontiguousarray(codes, dtype=np.int8).reshape(-1)
    out = np.empty(codes.size, dtype=np.uint16)
    lib().ixo_codes_to_bf16(_ptr(codes), codes.size, scale_bits, _ptr(out))
    return out


def decode_bf16(p: dict) -> np.ndarray:
    return codes_to_bf16(decode_codes(p), p["scale"]).reshape(p["out_f"], p["in_f"])


def ixgs_decode_bf16(p: dict) -> np.ndarray:
    """Group-scale sibling format (ixgs/quantize.py:116-151): the same five streams, fields offset by -3 / -15 / -127,
    then w[e] = bf16(f32(code[e]) * f32(fp16 scale[e // group])).  `p`: the ixgs dict with numpy arrays
    (group_scales as fp16 bit patterns).  Returns bf16 bit patterns [out_f, in_f]."""
    n1, n2, n3 = (int(c) for c in p["counts"])
    n = int(p["out_f"]) * int(p["in_f"])
    main = {"N": n, "bitmaps": [np.asarray(p["b1"]), np.asarray(p["b2"])[: (n2 + n3 + 31) // 32]],
            "streams": [np.asarray(p["l1"]), np.asarray(p["l2"]), np.asarray(p["l3"])[:n3]]}
    codes = decode_codes(main).astype(np.float32)
    scales = np.asarray(p["group_scales"], dtype=np.uint16).view(np.float16).astype(np.float32)
    per_elem = np.repeat(scales, int(p["group_size"]))[:n]
    return f32_to_bf16_bits(codes * per_elem).reshape(int(p["out_f"]), int(p["in_f"]))


# ------------------------------------------------------------ TPAB tiles ----
def tpab_decode_bf16(p: dict) -> np.ndarray:
    """TPAB tile format (ixrun/tpab.py:180-203): tiles of tile_r x 64, per tile a bit width b in 2..6, an fp16 scale
    and its element offset `goff` inside the group of tiles of that width; element L of tile t is the b-bit field at
    bit gbase_bit[b] + (goff[t] + L) * b of the uint32 body, q = field - (2^(b-1) - 1), w = bf16(f32(q) * f32(scale));
    outliers (tile, element, fp16 value) replace their weights.  `p`: numpy arrays (fp16 / bf16 as bit patterns).
    Returns bf16 bit patterns [out_f, in_f]."""
    out_f, in_f, tr = int(p["out_f"]), int(p["in_f"]), int(p["tile_r"])
    n_per, t_c = tr * 64, in_f // 64
    body = np.ascontiguousarray(p["body"]).view(np.uint32).astype(np.uint64)
    body = np.concatenate([body, np.zeros(2, dtype=np.uint64)])
    bits_ = np.asarray(p["bits"]).astype(np.int64)
    scales = np.asarray(p["scales"], dtype=np.uint16).view(np.float16).astype(np.float32)
    goff = np.asarray(p["goff"]).astype(np.int64)
    gbase = np.asarray(p["gbase_bit"]).astype(np.int64)
    n_t = bits_.size
    L = np.arange(n_per, dtype=np.int64)[None, :]
    b = bits_[:, None]
    pos = gbase[bits_][:, None] + (goff[:, None] + L) * b
    word, sh = pos >> 5, (pos & 31).astype(np.uint64)
    raw = ((body[word] | (body[word + 1] << np.uint64(32))) >> sh) & ((np.uint64(1) << b.astype(np.uint64)) - np.uint64(1))
    q = raw.astype(np.int64) - ((1 << (b - 1)) - 1)
    w = f32_to_bf16_bits((q.astype(np.float32) * scales[:, None]).astype(np.float32)).reshape(n_t, n_per)
    ol_t, ol_l = np.asarray(p["ol_t"]).astype(np.int64), np.asarray(p["ol_l"]).astype(np.int64)
    ol = np.asarray(p["ol_val"], dtype=np.uint16).view(np.float16).astype(np.float32)
    w[ol_t, ol_l] = f32_to_bf16_bits(ol)
    return w.reshape(out_f // tr, t_c, tr, 64).transpose(0, 2, 1, 3).reshape(out_f, in_f)


def tpab_gemv_f32(p: dict, x_bits: np.ndarray) -> np.ndarray:
    """y = W x in float64-accumulated float32 for the decoded TPAB weights (ixrun/tpab_gemv.py:72-124)."""
    w = bf16_bits_to_f32(tpab_decode_bf16(p)).astype(np.float64)
    x = bf16_bits_to_f32(np.asarray(x_bits, dtype=np.uint16)).astype(np.float64)
    return (w @ x).astype(np.float32)


# ------------------------------------------------------------ gemv / gemm ---
def gemm_f32(codes: np.ndarray, scale_bits: int, x_bits: np.ndarray, out_f: int, in_f: int):
    """y[M, out_f] (float32) for x bf16 bits [M, in_f]."""
    codes = np.ascontiguousarray(codes, dtype=np.int8).reshape(-1)
    x = np.ascontiguousarray(x_bits, dtype=np.uint16).reshape(-1, in_f)
    y = np.empty((x.shape[0], out_f), dtype=np.float32)
    lib().ixo_gemm_f32(_ptr(codes), scale_bits, _ptr(x), x.shape[0], out_f, in_f, _ptr(y))
    return y


class LayerCPU:
    """The reference's CPU layer path (decode to bf16, then matmul) with its
    scratch buffers allocated once, for timing."""

    def __init__(self, p: dict):
        self.p = p
        self.s = _streams(p)
        n = p["N"]
        nb = (n + 1023) // 1024
        self.codes = np.empty(n, dtype=np.int8)
        self.w = np.empty(n, dtype=np.uint16)
        self.q1 = np.empty(nb, dtype=np.int32)
        self.q2 = np.empty(nb, dtype=np.int32)

    def __call__(self, x_bits: np.ndarray) -> np.ndarray:
        p = self.p
        b1, b2, l1, l2, l3, l1w, l2w = self.s
        x = np.ascontiguousarray(x_bits, dtype=np.uint16).reshape(-1, p["in_f"])
        y = np.empty((x.shape[0], p["out_f"]), dtype=np.float32)
        lib().ixo_layer_cpu(_ptr(b1), _ptr(b2), _ptr(l1), l1w, _ptr(l2), l2w, _ptr(l3),
                            p["scale"], _ptr(x), x.shape[0], p["out_f"], p["in_f"],
                            _ptr(self.codes), _ptr(self.w), _ptr(self.q1), _ptr(self.q2), _ptr(y))
        return y


# --------------------------------------------------------------- bitpack ---
def pack_bits(vals: np.ndarray, bits: int) -> np.ndarray:
    v = np.ascontiguousarray(vals, dtype=np.int32).reshape(-1)
    out = np.zeros((v.size * bits + 31) // 32 + 1, dtype=np.uint32)
    lib().ixo_pack_bits(_ptr(v), v.size, bits, _ptr(out))
    return out[:-1].view(np.int32)


def unpack_bits(packed: np.ndarray, n: int, bits: int) -> np.ndarray:
    pk = np.ascontiguousarray(packed).view(np.uint32)
    out = np.empty(n, dtype=np.int32)
    lib().ixo_unpack_bits(_ptr(pk), pk.size, n, bits, _ptr(out))
    return out


# ------------------------------------------------------- synthetic inputs ---
def laplace_codes(out_f: int, in_f: int, seed: int, b: float = 4.4) -> np.ndarray:
    """Seeded stand-in for LLM weight codes: round(Laplace(0, b)) clipped to
    +-127 with one element forced to +-127 (so the per-tensor scale is exact)."""
    rng = np.random.default_rng(seed)
    n = out_f * in_f
    c = np.clip(np.rint(rng.laplace(0.0, b, size=n)), -127, 127).astype(np.int8)
    pos = int(rng.integers(0, n))
    c[pos] = 127 if rng.integers(0, 2) else -127
    return c


def codes_to_weight_bits(codes: np.ndarray, exp2: int = -9) -> np.ndarray:
    """W = bf16(code * 2**exp2): exactly representable, so quantising W gives
    the codes back and scale == 2**exp2."""
    return f32_to_bf16_bits(codes.astype(np.float32) * np.float32(2.0 ** exp2))
