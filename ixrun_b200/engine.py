"""Packed-linear modules and the engine front end (API of ixrun/engine.py).

Three deployment modes, as in the reference:
  cached     decode every packed weight to bf16 once, keep it resident
  streaming  keep only the packed streams resident; single-token steps (and up
             to 8 rows) run the fused decode+GEMV kernel, larger inputs decode
             into one shared bf16 buffer and call a dense matmul
  graph      per-layer bf16 buffers refreshed by one captured CUDA graph of all
             decode launches
"""
from __future__ import annotations

import gc
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from .fused import _pick_split
from .linear import _set_parent_child, iter_quantizable_linears
from .packed import DevicePacked
from .quantize import int8x_quantize

__all__ = ["Int8XEngine", "StreamingLinear", "GraphLinear", "ResourceScheduler", "GraphedCall"]

FUSED_MAX_ROWS = 8        # rows served by the CUDA-core fused kernel
TC_MAX_ROWS = 64          # rows served by the tensor-core fused kernel (when enabled)


class StreamingLinear(nn.Module):
    """Per-layer streaming linear (ixrun/engine.py:40-173).

    Attribute and buffer names follow the reference because its benchmarks and
    tests read them (`_b1 .. _l3`, `_q1/_q2`, `_scale`, `_b1_blk/_b2_blk`,
    `_use_fused`, `_split_chunk`, `_y32`).
    """

    def __init__(self, packed, bias=None, resident: str | None = None, keep_streams: bool | None = None):
        """`packed`: the reference's packed dict, or a DevicePacked already on the GPU.

        resident: "p6" (default; environment variable IXB200_RESIDENT overrides the default) re-lays the codes out
        at construction as a 6-bit plane + outlier tails and runs every input on it (up to 8 rows fused, more rows
        through its decoder and a dense matmul); "streams" keeps to the reference's (3,5,8) streams and the fused
        kernel that reads them directly.
        keep_streams: with resident="p6" the stream buffers are freed once the layout exists (the default), so a
        deployed layer holds one copy of its weights; keep_streams=True keeps them, and with them the
        reference-named buffers `_b1 .. _l3`, `_q1/_q2`, `_b1_blk/_b2_blk` that the reference's benchmarks read."""
        super().__init__()
        resident = resident or os.environ.get("IXB200_RESIDENT", "p6")
        if resident not in ("p6", "streams"):
            raise ValueError("resident must be 'p6' or 'streams'")
        if keep_streams is None:
            keep_streams = resident == "streams"
        if resident == "streams" and not keep_streams:
            raise ValueError("resident='streams' needs the streams")
        dp = packed if isinstance(packed, DevicePacked) else DevicePacked(packed)
        self.out_features = dp.out_f
        self.in_features = dp.in_f
        self.N = dp.N
        self.level_bits = (3, 5, 8)
        self.counts = dp.counts
        self.total_bytes = dp.total_bytes
        self._dp = dp
        self._use_triton = True
        # the fused kernel on the streams handles any in_f that is a multiple of 32
        self._use_fused = keep_streams and self.in_features % 32 == 0
        self._split_chunk = 0
        if keep_streams:
            for key, val in (("_b1", dp.b1), ("_b2", dp.b2), ("_l1", dp.l1), ("_l2", dp.l2), ("_l3", dp.l3),
                             ("_b1_blk", dp.blk_q1), ("_b2_blk", dp.blk_q2)):
                self.register_buffer(key, val, persistent=False)
            if self._use_fused:
                split = _pick_split(self.in_features) if self.out_features < self.in_features else 1
                gran = self.in_features
                if split > 1:
                    self._split_chunk = self.in_features // split
                    gran = self._split_chunk
                q1, q2 = dp.prefix_tables(gran, self.N // gran)
                self.register_buffer("_q1", q1, persistent=False)
                self.register_buffer("_q2", q2, persistent=False)
        self.register_buffer("_scale", dp.scale, persistent=False)
        self._y32 = None
        # 9..64 rows on the resident layout: one pass over the packed bytes on the tcgen05 tensor cores
        # (ixb_p6_gemm, in_f % 64 == 0); set _use_p6_gemm = False to take decode + dense matmul instead.
        # _use_tc: the older tensor-core kernel that reads the streams (needs them kept, in_f % 1024 == 0); off.
        self._use_p6_gemm = True
        self._use_tc = False
        if bias is not None:
            self.register_buffer("_bias", bias.detach().clone().to(dp.device), persistent=False)
            self._bias_bf16 = self._bias.to(torch.bfloat16)
        else:
            self._bias = None
            self._bias_bf16 = None
        self._w_buf = None
        self._res = None                         # the resident re-layout
        if resident == "p6":
            from .p6 import P6Packed

            self._res = P6Packed.from_packed(dp)
            if not keep_streams:
                self._dp = None                  # the streams (and their rank tables) are released with it

    @classmethod
    def from_weight(cls, weight: torch.Tensor, bias=None, **kw):
        """Quantise and pack a bf16 weight on the GPU (no CPU pass over the tensor)."""
        from .gpu_pack import quantize_pack_gpu

        return cls(quantize_pack_gpu(weight.detach().to("cuda", torch.bfloat16)), bias=bias, **kw)

    @property
    def resident_bytes(self) -> int:
        """Bytes of weight data this layer keeps on the device."""
        n = self._res.resident_bytes if self._res is not None else 0
        if self._dp is not None:
            n += self.total_bytes
        return n

    def matvec(self, x, out=None, out_dtype=torch.bfloat16):
        """y[M, out_f] for 1..8 bf16 rows on the resident layout, without bias (used by the runners and bench)."""
        if self._res is not None:
            return self._res.gemv(x, out=out, out_dtype=out_dtype)
        return self._dp.gemv(x, out=out, out_dtype=out_dtype)

    def _set_shared_buf(self, w_buf):
        self._w_buf = w_buf

    def _decode(self):
        """Decode the packed weight into the shared buffer -> bf16 [out, in]."""
        if self._w_buf is None:
            raise RuntimeError("no decode buffer set (call _set_shared_buf)")
        src = self._res if self._res is not None else self._dp       # the decoder of the resident layout is the faster of the two
        return src.decode(out=self._w_buf[: self.N], kind="bf16")

    def forward(self, x):
        rows = x.numel() // self.in_features
        if self._res is not None and x.dtype == torch.bfloat16 and 1 <= rows <= FUSED_MAX_ROWS \
                and x.shape[-1] == self.in_features:
            y = self._res.gemv(x.reshape(rows, self.in_features), bias=self._bias_bf16)
            return y.view(x.shape[:-1] + (self.out_features,))
        if self._res is not None and self._use_p6_gemm and x.dtype == torch.bfloat16 and rows <= TC_MAX_ROWS \
                and self.in_features % 64 == 0 and x.shape[-1] == self.in_features:
            y = self._res.gemm(x.reshape(rows, self.in_features), bias=self._bias_bf16)
            return y.view(x.shape[:-1] + (self.out_features,))
        if self._use_fused and x.dtype == torch.bfloat16 and 1 <= rows <= FUSED_MAX_ROWS \
                and x.shape[-1] == self.in_features:
            y = self._dp.gemv(x.reshape(rows, self.in_features), bias=self._bias_bf16)
            return y.view(x.shape[:-1] + (self.out_features,))
        if self._use_tc and self._dp is not None and x.dtype == torch.bfloat16 and rows <= TC_MAX_ROWS \
                and self.in_features % 1024 == 0 and x.shape[-1] == self.in_features:
            y = self._dp.gemm(x.reshape(rows, self.in_features), bias=self._bias_bf16)
            return y.view(x.shape[:-1] + (self.out_features,))
        w = self._decode()
        bias = self._bias.to(x.dtype) if self._bias is not None else None
        return F.linear(x, w if w.dtype == x.dtype else w.to(x.dtype), bias)


class GraphLinear(nn.Module):
    """Matmul-only layer; its weight buffer is refreshed by the engine's graph
    replay (ixrun/engine.py:179-196)."""

    def __init__(self, packed: dict, bias=None, decode_buf=None):
        super().__init__()
        self.out_features = packed["out_f"]
        self.in_features = packed["in_f"]
        self.N = packed["N"]
        self._w_buf = decode_buf
        if bias is not None:
            self.register_buffer("_bias", bias.detach().clone().cuda())
        else:
            self._bias = None

    def forward(self, x):
        w = self._w_buf[: self.N].view(self.out_features, self.in_features)
        bias = self._bias.to(x.dtype) if self._bias is not None else None
        return F.linear(x, w, bias)


class GraphedCall:
    """Capture a fixed sequence of launches (e.g. the packed linears of one
    decoder block) in a CUDA graph over static buffers.

    `fn(*static_inputs)` must allocate nothing new between calls that matters
    to the caller: its outputs are kept as static tensors and overwritten by
    every replay.  Call the object with new inputs of the same shapes.
    """

    def __init__(self, fn, *example_inputs, warmup: int = 2, host_io: bool = False):
        """host_io=True also captures the copies between pinned host buffers and the static device tensors, so
        that `run_host` is ONE graph launch per call: host-to-device copy of the inputs, the launches, device-to-host
        copy of the (single tensor) result."""
        self.static_in = [t.clone() for t in example_inputs]
        self.host_in = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in example_inputs] if host_io else None
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(max(warmup, 1)):
                out = fn(*self.static_in)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory() if host_io else None
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            if host_io:
                for dst, src in zip(self.static_in, self.host_in):
                    dst.copy_(src, non_blocking=True)
            self.static_out = fn(*self.static_in)
            if host_io:
                self.host_out.copy_(self.static_out, non_blocking=True)

    def __call__(self, *inputs):
        for dst, src in zip(self.static_in, inputs):
            dst.copy_(src)
        self.graph.replay()
        return self.static_out

    def run_host(self, *host_inputs):
        """Inputs from host memory, result in pinned host memory, valid on return (needs host_io=True)."""
        if self.host_in is None:
            raise RuntimeError("GraphedCall was built without host_io=True")
        for dst, src in zip(self.host_in, host_inputs):
            dst.copy_(src)                        # host memcpy into the pinned staging buffer the graph reads
        self.graph.replay()
        torch.cuda.current_stream().synchronize()
        return self.host_out


class ResourceScheduler:
    """Memory estimates and mode recommendation (ixrun/engine.py:202-235)."""

    @staticmethod
    @torch.no_grad()
    def estimate(model: nn.Module, level_bits=(3, 5, 8)) -> dict:
        bf16_bytes = packed_bytes = n_elems = max_layer = 0
        for _, mod in iter_quantizable_linears(model):
            w = mod.weight.data
            packed_bytes += int8x_quantize(w, level_bits)["total_bytes"]
            bf16_bytes += w.numel() * 2
            n_elems += w.numel()
            max_layer = max(max_layer, w.numel())
        return {
            "bf16_weight_MB": bf16_bytes / 1e6,
            "packed_storage_MB": packed_bytes / 1e6,
            "compression": bf16_bytes / max(packed_bytes, 1),
            "max_layer_elems": max_layer,
            "shared_decode_buf_MB": max_layer * 2 / 1e6,
            "n_elems": n_elems,
        }

    @staticmethod
    def recommend(model: nn.Module, gpu_budget_GB: float, level_bits=(3, 5, 8)) -> str:
        est = ResourceScheduler.estimate(model, level_bits)
        return "cached" if est["bf16_weight_MB"] + 1500 <= gpu_budget_GB * 1000 else "streaming"


class Int8XEngine:
    """High-level engine: load, deploy, generate (ixrun/engine.py:241-516)."""

    def __init__(self, model, tokenizer, stats=None, graph_replay=None):
        self.model = model
        self.tokenizer = tokenizer
        self.stats = stats or {}
        self._graph_replay = graph_replay
        self.model.eval()

    # ------------------------------------------------------------- loading --
    @classmethod
    def from_pretrained(cls, model_path: str, mode: str = "cached", level_bits=(3, 5, 8),
                        dtype=torch.bfloat16, verbose: bool = True, cache_path: str | None = None):
        from transformers import AutoModelForCausalLM, AutoTokenizer

        if mode not in ("cached", "streaming", "graph"):
            raise ValueError("mode must be 'cached', 'streaming' or 'graph'")
        tokenizer = AutoTokenizer.from_pretrained(model_path, trust_remote_code=True)
        if tokenizer.pad_token is None:
            tokenizer.pad_token = tokenizer.eos_token
        model = AutoModelForCausalLM.from_pretrained(model_path, dtype=dtype, low_cpu_mem_usage=True)
        big = mode in ("streaming", "graph")
        if not big:
            model = model.cuda()
        if mode == "streaming":
            stats = cls._deploy_streaming(model, level_bits, verbose=verbose, cache_path=cache_path)
        elif mode == "graph":
            stats, replay = cls._deploy_graph(model, level_bits, verbose=verbose)
            eng = cls(model, tokenizer, stats, graph_replay=replay)
            eng._finalize_device()
            return eng
        else:
            stats = cls._deploy_cached(model, level_bits, verbose=verbose)
        eng = cls(model, tokenizer, stats)
        if big:
            eng._finalize_device()
        return eng

    # -------------------------------------------------------------- deploy --
    @staticmethod
    def _deploy_cached(model, level_bits, verbose=True):
        from .linear import deploy_model

        return deploy_model(model, level_bits=level_bits, cache="full", verbose=verbose)

    @staticmethod
    def _load_or_quantize(model, level_bits, verbose, cache_path):
        """[(name, packed, bias)] from the packed-weight cache file if it exists,
        else quantised now (and saved).  File layout as in ixrun/engine.py:356-383."""
        if cache_path is not None and os.path.exists(cache_path):
            blob = torch.load(cache_path, map_location="cpu", weights_only=False)
            if tuple(blob["level_bits"]) != tuple(level_bits):
                raise ValueError(f"cache was built with level_bits={blob['level_bits']}, "
                                 f"requested {tuple(level_bits)}; delete the cache or change level_bits")
            layer_data = blob["layers"]
            have = {n for n, _ in model.named_modules()}
            missing = [n for n, _, _ in layer_data if n not in have]
            if missing:
                raise ValueError(f"cache/model mismatch: {len(missing)} unknown layers")
            if verbose:
                print(f"[engine][cache] {len(layer_data)} layers loaded from {cache_path}", flush=True)
            return layer_data
        layer_data = []
        for name, mod in iter_quantizable_linears(model):
            bias = mod.bias.data if mod.bias is not None else None
            layer_data.append((name, int8x_quantize(mod.weight.data, level_bits), bias))
        if cache_path is not None:
            torch.save({"level_bits": tuple(level_bits), "layers": layer_data}, cache_path)
            if verbose:
                print(f"[engine][cache] packed weights saved to {cache_path}", flush=True)
        return layer_data

    @staticmethod
    @torch.no_grad()
    def _deploy_streaming(model, level_bits, verbose=True, cache_path=None):
        max_n = total_bytes = 0
        layers = []
        if cache_path is None:
            # no cache file wanted: quantise and pack every layer on the GPU, one at a time
            if tuple(sorted(level_bits)) != (3, 5, 8):
                raise ValueError(f"only the (3, 5, 8) scheme is supported, got {tuple(level_bits)}")
            for name, mod in list(iter_quantizable_linears(model)):
                sl = StreamingLinear.from_weight(mod.weight.data, bias=mod.bias.data if mod.bias is not None else None)
                layers.append((name, sl))
                total_bytes += sl.total_bytes
                max_n = max(max_n, sl.N)
        else:
            for name, p, bias in Int8XEngine._load_or_quantize(model, level_bits, verbose, cache_path):
                layers.append((name, StreamingLinear(p, bias=bias)))
                total_bytes += p["total_bytes"]
                max_n = max(max_n, p["N"])
        shared_w = torch.empty(max(max_n, 1), dtype=torch.bfloat16, device="cuda")
        for name, sl in layers:
            sl._set_shared_buf(shared_w)
            _set_parent_child(model, name, sl)
        gc.collect()
        torch.cuda.empty_cache()
        shared_mb = shared_w.numel() * 2 / 1e6
        if verbose:
            print(f"[engine][streaming] {len(layers)} layers | packed GPU-resident={total_bytes / 1e6:.0f}MB | "
                  f"shared decode buf={shared_mb:.1f}MB", flush=True)
        return {"mode": "streaming", "n_layers": len(layers), "total_bytes": total_bytes,
                "resident_bytes": sum(sl.resident_bytes for _, sl in layers), "shared_gpu_MB": shared_mb}

    @staticmethod
    @torch.no_grad()
    def _deploy_graph(model, level_bits, verbose=True):
        targets = list(iter_quantizable_linears(model))
        total_params = sum(m.weight.numel() for _, m in targets)
        if total_params * 2 > torch.cuda.get_device_properties(0).total_memory * 0.9:
            raise RuntimeError(f"graph mode needs {total_params * 2 / 1e9:.1f}GB of per-layer decode "
                               f"buffers — too large for this GPU; use mode='streaming'")
        total_bytes = 0
        specs = []
        for name, mod in targets:
            p = int8x_quantize(mod.weight.data, level_bits)
            sl = StreamingLinear(p, bias=mod.bias.data if mod.bias is not None else None)
            buf = torch.empty(p["N"], dtype=torch.bfloat16, device="cuda")
            sl._set_shared_buf(buf)
            specs.append((name, sl, buf))
            total_bytes += p["total_bytes"]

        def decode_all():
            for _, sl, _ in specs:
                sl._decode()

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            decode_all()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            decode_all()
        torch.cuda.synchronize()
        for name, sl, buf in specs:
            gl = GraphLinear({"out_f": sl.out_features, "in_f": sl.in_features, "N": sl.N},
                             bias=sl._bias, decode_buf=buf)
            _set_parent_child(model, name, gl)

        def replay(_keep_alive=specs, _graph=graph):
            _graph.replay()

        if verbose:
            print(f"[engine][graph] {len(specs)} layers | packed={total_bytes / 1e6:.0f}MB | "
                  f"decode=graph.replay()", flush=True)
        return {"mode": "graph", "n_layers": len(specs), "total_bytes": total_bytes}, replay

    # ----------------------------------------------------------- inference --
    def _finalize_device(self):
        for _, mod in self.model.named_modules():
            for p in mod.parameters(recurse=False):
                if p.data.device.type != "cuda":
                    p.data = p.data.cuda()
            for bname, b in list(mod.named_buffers(recurse=False)):
                if b.device.type != "cuda":
                    setattr(mod, bname, b.cuda())
        gc.collect()
        torch.cuda.empty_cache()
        self.model.eval()

    def _pre_forward(self):
        if self._graph_replay is not None:
            self._graph_replay()

    @torch.no_grad()
    def generate(self, prompt, max_new_tokens: int = 64, **kw):
        self._pre_forward()
        enc = self.tokenizer(prompt, return_tensors="pt").to("cuda")
        out = self.model.generate(**enc, max_new_tokens=max_new_tokens, do_sample=kw.pop("do_sample", False), **kw)
        return self.tokenizer.decode(out[0, enc["input_ids"].shape[1]:], skip_special_tokens=True)

    def stream(self, prompt, **kw):
        yield self.generate(prompt, **kw)
