"""B200-native INT8-X weight path: (3,5,8) nested-bitmap decode, fused
decode+GEMV / small-M GEMM and the packed-linear modules built on them.

The CUDA side is one C-ABI shared library (``include/ixb200.h``) compiled for
sm_100a; this package binds it with ctypes and mirrors the reference's module
and function names so it drops in for the packed-weight path.
"""
from .quantize import DEFAULT_LEVELS, int8x_quantize, pack_codes

__version__ = "0.1.0"

__all__ = ["int8x_quantize", "pack_codes", "DEFAULT_LEVELS", "__version__"]


def __getattr__(name):
    # torch.nn-based modules are imported on first use
    if name in ("Int8XLinear", "deploy_model", "iter_quantizable_linears"):
        from . import linear

        return getattr(linear, name)
    if name in ("Int8XEngine", "StreamingLinear", "GraphLinear", "GraphedCall", "ResourceScheduler"):
        from . import engine

        return getattr(engine, name)
    if name in ("fused_gemv", "compute_row_prefixes"):
        from . import fused

        return getattr(fused, name)
    if name in ("decode_weight", "decode_weight_triton", "decode_codes", "precompute_block_offsets"):
        from . import kernels

        return getattr(kernels, name)
    if name in ("P6Packed", "set_pdl", "GemvScratch"):
        from . import p6

        return getattr(p6, name)
    if name == "PeerAllReduce":
        from . import parallel

        return parallel.PeerAllReduce
    raise AttributeError(name)
