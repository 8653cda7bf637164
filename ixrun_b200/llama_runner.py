"""Batch-1 decode loop for a Llama-style decoder whose linears are packed
INT8-X layers, with the whole token step captured in one CUDA graph.

The reference drives HuggingFace `generate()` around its packed modules
(ixrun/generate.py:39-70, ixrun/engine.py:510-516) and records that whole-model
graph capture was not possible with HF's dynamic KV cache.  This runner keeps a
static KV cache and position tensors so that one token step is a fixed launch
sequence: per layer RMSNorm -> q/k/v packed GEMVs -> RoPE -> cache write ->
attention over the static cache -> o_proj GEMV -> RMSNorm -> gate/up GEMVs ->
SwiGLU -> down GEMV.  The packed linears run the fused decode+GEMV kernel; with
`glue="kernels"` the work between them is this library's glue kernels (residual
add + RMSNorm, RoPE + cache write, split-context attention, SwiGLU) and q|k|v
and gate|up are one fused packed tensor each: 10 launches per layer, all taking
part in programmatic dependent launch; with
`glue="eager"` it is plain torch.  Prefill (many rows) always takes the torch path.

`weights="packed"` uses StreamingLinear (fused kernels); `weights="decoded"`
builds the same model with the packed weights decoded to bf16 and dense
matmuls -- with eager glue the ground truth for greedy-token agreement.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .engine import StreamingLinear
from .packed import DevicePacked


@dataclass
class LlamaConfig:
    n_layers: int = 24
    hidden: int = 2048
    intermediate: int = 6144
    n_heads: int = 16
    n_kv_heads: int = 8
    head_dim: int = 128
    vocab: int = 73448
    rope_theta: float = 10000.0
    rms_eps: float = 1e-5
    max_seq: int = 1280


LINEARS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


def linear_shapes(cfg: LlamaConfig) -> dict:
    h, hd = cfg.hidden, cfg.head_dim
    return {
        "q_proj": (cfg.n_heads * hd, h), "k_proj": (cfg.n_kv_heads * hd, h), "v_proj": (cfg.n_kv_heads * hd, h),
        "o_proj": (h, cfg.n_heads * hd), "gate_proj": (cfg.intermediate, h), "up_proj": (cfg.intermediate, h),
        "down_proj": (h, cfg.intermediate),
    }


class _DenseLinear(torch.nn.Module):
    """bf16 weight decoded once from a packed dict (ground-truth path)."""

    def __init__(self, packed: dict):
        super().__init__()
        self.weight = DevicePacked(packed).decode(kind="bf16")

    def forward(self, x):
        return F.linear(x, self.weight)


def _rms(x, w, eps):
    v = x.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


class FusedPackedLinear(torch.nn.Module):
    """Several packed linears that share their input (q|k|v, gate|up) as ONE resident tensor and one launch; every
    part keeps its own per-tensor scale (p6.P6Packed.fuse).  forward returns the parts' outputs."""

    def __init__(self, packed_parts: list):
        super().__init__()
        from .p6 import P6Packed

        self.res = P6Packed.fuse(packed_parts)
        self.in_features = self.res.in_f
        self._w_buf = None

    def _set_shared_buf(self, buf):
        self._w_buf = buf

    def forward(self, x):
        rows = x.numel() // self.in_features
        x2 = x.reshape(rows, self.in_features)
        if rows <= 8:
            y = self.res.gemv(x2)
        else:                                   # prefill: decode into the shared buffer, dense matmul
            y = F.linear(x2, self.res.decode(out=self._w_buf[: self.res.N], kind="bf16"))
        return [y[:, a:a + n] for a, n in self.res.sections]


class PackedLlama(torch.nn.Module):
    def __init__(self, cfg: LlamaConfig, packed_layers: list, embed: torch.Tensor, lm_head: torch.Tensor,
                 norms: list | None = None, weights: str = "packed", device="cuda", glue: str | None = None):
        """packed_layers[i][name] = packed dict of layer i's linear `name`;
        embed [vocab, hidden] and lm_head [vocab, hidden] stay bf16.
        glue: "kernels" (default for packed weights) or "eager" (default for decoded weights)."""
        super().__init__()
        if weights not in ("packed", "decoded"):
            raise ValueError("weights must be 'packed' or 'decoded'")
        glue = glue or ("kernels" if weights == "packed" else "eager")
        if glue not in ("kernels", "eager"):
            raise ValueError("glue must be 'kernels' or 'eager'")
        self.cfg, self.glue, self.weights = cfg, glue, weights
        dev = torch.device(device)
        mk = StreamingLinear if weights == "packed" else _DenseLinear
        self.layers = torch.nn.ModuleList()
        max_n = 0
        for li in range(cfg.n_layers):
            pl = packed_layers[li]
            if weights == "packed":
                # linears that share their input are one resident tensor and one launch
                mods = torch.nn.ModuleDict({"qkv": FusedPackedLinear([pl["q_proj"], pl["k_proj"], pl["v_proj"]]),
                                            "o_proj": mk(pl["o_proj"]),
                                            "gate_up": FusedPackedLinear([pl["gate_proj"], pl["up_proj"]]),
                                            "down_proj": mk(pl["down_proj"])})
                max_n = max([max_n, pl["o_proj"]["N"], pl["down_proj"]["N"], mods["qkv"].res.N, mods["gate_up"].res.N])
            else:
                mods = torch.nn.ModuleDict({n: mk(pl[n]) for n in LINEARS})
            self.layers.append(mods)
        if weights == "packed":
            # one shared decode buffer for inputs of more than 8 rows (prefill), like the streaming engine
            self._shared = torch.empty(max_n, dtype=torch.bfloat16, device=dev)
            for mods in self.layers:
                for m in mods.values():
                    m._set_shared_buf(self._shared)
        ones = torch.ones(cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.ln1 = [ones.clone() if norms is None else norms[i][0].to(dev) for i in range(cfg.n_layers)]
        self.ln2 = [ones.clone() if norms is None else norms[i][1].to(dev) for i in range(cfg.n_layers)]
        self.ln_f = ones.clone()
        self.embed = embed.to(dev, torch.bfloat16)
        self.lm_head = lm_head.to(dev, torch.bfloat16)
        half = cfg.head_dim // 2
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float32) / half))
        ang = torch.arange(cfg.max_seq, dtype=torch.float32)[:, None] * inv[None, :]
        self.cos = ang.cos().to(dev)
        self.sin = ang.sin().to(dev)
        self.k_cache = torch.zeros(cfg.n_layers, cfg.max_seq, cfg.n_kv_heads, cfg.head_dim, dtype=torch.bfloat16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.key_pos = torch.arange(cfg.max_seq, device=dev)
        # static inputs / outputs of the captured step
        self.tok = torch.zeros(1, dtype=torch.long, device=dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.pos32 = torch.zeros(1, dtype=torch.int32, device=dev)
        self.logits = None
        self.graph = None
        if glue == "kernels":
            from .glue import AttnDecode

            bf = dict(dtype=torch.bfloat16, device=dev)
            qd, kd = cfg.n_heads * cfg.head_dim, cfg.n_kv_heads * cfg.head_dim
            # static activations of the one-row step
            self._h = torch.zeros(1, cfg.hidden, **bf)
            self._xn = torch.zeros(1, cfg.hidden, **bf)
            if weights == "packed":                                # outputs of the fused linears and the parts' views
                self._qkv = torch.zeros(1, self.layers[0]["qkv"].res.out_f, **bf)
                self._q, self._k, self._v = self.layers[0]["qkv"].res.split(self._qkv)
                self._gu = torch.zeros(1, self.layers[0]["gate_up"].res.out_f, **bf)
                self._g, self._u = self.layers[0]["gate_up"].res.split(self._gu)
            else:
                self._q, self._k, self._v = torch.zeros(qd, **bf), torch.zeros(kd, **bf), torch.zeros(kd, **bf)
                self._g, self._u = torch.zeros(cfg.intermediate, **bf), torch.zeros(cfg.intermediate, **bf)
            self._a = torch.zeros(1, qd, **bf)
            self._d = torch.zeros(1, cfg.hidden, **bf)             # output of o_proj / down_proj: the next residual
            self._act = torch.zeros(1, cfg.intermediate, **bf)
            self._attn = AttnDecode(cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, dev)

    # ------------------------------------------------------------------ core
    def _rope(self, x, pos):
        """x [T, heads, head_dim], pos [T] (rotate-half convention)"""
        c = self.cos.index_select(0, pos)[:, None, :]
        s = self.sin.index_select(0, pos)[:, None, :]
        x1, x2 = x.float().chunk(2, dim=-1)
        return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)

    def _block(self, li, h, pos):
        """h [T, hidden], pos [T] absolute positions (T = 1 in the decode step)"""
        cfg, m = self.cfg, self.layers[li]
        t = h.shape[0]
        x = _rms(h, self.ln1[li], cfg.rms_eps)
        q, k, v = m["qkv"](x) if self.weights == "packed" else (m["q_proj"](x), m["k_proj"](x), m["v_proj"](x))
        q = q.reshape(t, cfg.n_heads, cfg.head_dim)
        k = k.reshape(t, cfg.n_kv_heads, cfg.head_dim)
        v = v.reshape(t, cfg.n_kv_heads, cfg.head_dim)
        q, k = self._rope(q, pos), self._rope(k, pos)
        self.k_cache[li].index_copy_(0, pos, k)
        self.v_cache[li].index_copy_(0, pos, v)
        # attention of the T new queries over the whole static cache, masked to keys <= query position
        rep = cfg.n_heads // cfg.n_kv_heads
        kk = self.k_cache[li].repeat_interleave(rep, dim=1).transpose(0, 1)      # [heads, S, d]
        vv = self.v_cache[li].repeat_interleave(rep, dim=1).transpose(0, 1)
        mask = self.key_pos[None, :] <= pos[:, None]                               # [T, S]
        a = F.scaled_dot_product_attention(q.transpose(0, 1), kk, vv, attn_mask=mask[None])
        a = a.transpose(0, 1).reshape(t, cfg.n_heads * cfg.head_dim)
        h = h + m["o_proj"](a)
        x = _rms(h, self.ln2[li], cfg.rms_eps)
        g, u = m["gate_up"](x) if self.weights == "packed" else (m["gate_proj"](x), m["up_proj"](x))
        return h + m["down_proj"](F.silu(g) * u)

    def _lin(self, li, name, x, out):
        m = self.layers[li][name]
        if self.weights == "packed":
            return m._res.gemv(x, out=out) if m._res is not None else out.copy_(m(x))
        return torch.matmul(x, m.weight.t(), out=out.view(1, -1))

    def _qkv_step(self, li):
        if self.weights == "packed":
            return self.layers[li]["qkv"].res.gemv(self._xn, out=self._qkv)
        for n, o in (("q_proj", self._q), ("k_proj", self._k), ("v_proj", self._v)):
            self._lin(li, n, self._xn, o)

    def _gate_up_step(self, li):
        if self.weights == "packed":
            return self.layers[li]["gate_up"].res.gemv(self._xn, out=self._gu)
        self._lin(li, "gate_proj", self._xn, self._g)
        self._lin(li, "up_proj", self._xn, self._u)

    def _step_kernels(self):
        """One row at position self.pos32 (device) through all layers on the glue kernels; static buffers only."""
        from . import glue as G

        cfg = self.cfg
        torch.index_select(self.embed, 0, self.tok, out=self._h)
        delta = None
        for li in range(cfg.n_layers):
            G.add_rmsnorm(self._h, delta, self.ln1[li], cfg.rms_eps, out=self._xn)
            self._qkv_step(li)
            G.rope_kv(self._q, self._k, self._v, self.pos32, self.k_cache[li], self.v_cache[li], self.cos, self.sin,
                      cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
            self._attn(self._q, self.k_cache[li], self.v_cache[li], self.pos32, out=self._a)
            self._lin(li, "o_proj", self._a, self._d)
            G.add_rmsnorm(self._h, self._d, self.ln2[li], cfg.rms_eps, out=self._xn)
            self._gate_up_step(li)
            G.swiglu(self._g, self._u, out=self._act[0])
            self._lin(li, "down_proj", self._act, self._d)
            delta = self._d
        G.add_rmsnorm(self._h, delta, self.ln_f, cfg.rms_eps, out=self._xn)
        return F.linear(self._xn, self.lm_head).float()

    def _forward(self, tok, pos):
        if self.glue == "kernels" and tok.numel() == 1 and tok.data_ptr() == self.tok.data_ptr():
            return self._step_kernels()
        h = self.embed.index_select(0, tok)
        for li in range(self.cfg.n_layers):
            h = self._block(li, h, pos)
        h = _rms(h[-1:], self.ln_f, self.cfg.rms_eps)
        return F.linear(h, self.lm_head).float()

    # ------------------------------------------------------------------- API
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor, chunk: int = 256) -> torch.Tensor:
        """Run the prompt through the model (many rows per linear: decode +
        dense matmul path); returns the logits of the last prompt token."""
        logits = None
        for s in range(0, ids.numel(), chunk):
            part = ids[s:s + chunk].to(self.tok.device)
            pos = torch.arange(s, s + part.numel(), device=part.device)
            logits = self._forward(part, pos)
        return logits

    @torch.no_grad()
    def capture(self):
        """Capture one token step (static tok/pos in, static logits out)."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._forward(self.tok, self.pos)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self._forward(self.tok, self.pos)
        return self

    @torch.no_grad()
    def step(self, tok: torch.Tensor, pos: int) -> torch.Tensor:
        """One decode step at absolute position `pos`; returns logits [1, vocab]
        (a static tensor when the step is graph-captured)."""
        self.tok.copy_(tok.reshape(1))
        self.pos.fill_(pos)
        self.pos32.fill_(pos)
        if self.graph is not None:
            self.graph.replay()
            return self.logits
        return self._forward(self.tok, self.pos)

    @torch.no_grad()
    def generate(self, prompt_ids: torch.Tensor, n_new: int) -> torch.Tensor:
        """Greedy decode of n_new tokens after the prompt."""
        logits = self.prefill(prompt_ids)
        out = []
        pos = prompt_ids.numel()
        tok = logits.argmax(-1)
        for _ in range(n_new):
            out.append(tok.clone())
            logits = self.step(tok, pos)
            tok = logits.argmax(-1)
            pos += 1
        return torch.cat(out)


class Verifier:
    """T new tokens of ONE sequence in one pass (the verification forward of speculative decoding,
    ixrun/mtp.py:198-280: the draft's tokens go through the model together and the longest prefix that the model's own
    arg-max confirms is kept).  Every packed linear sees T rows (fused GEMV for T <= 8, tensor-core GEMM up to 64), the
    keys and values of the T positions are written into the sequence's cache, and query r attends up to position
    pos0 + r.  Runs on the model's own cache: a rejected tail is simply overwritten by the next call."""

    def __init__(self, model: PackedLlama, rows: int):
        from .glue import AttnDecode

        if model.weights != "packed" or model.glue != "kernels":
            raise ValueError("the verifier runs on packed weights and the glue kernels")
        if not 1 <= rows <= 64:
            raise ValueError("1..64 rows")
        self.m, self.t = model, int(rows)
        cfg, dev = model.cfg, model.embed.device
        bf = dict(dtype=torch.bfloat16, device=dev)
        t = self.t
        first = model.layers[0]
        self._h, self._xn, self._d = (torch.zeros(t, cfg.hidden, **bf) for _ in range(3))
        self._qkv = torch.zeros(t, first["qkv"].res.out_f, **bf)
        self._q, self._k, self._v = (self._qkv[:, a:a + n] for a, n in first["qkv"].res.sections)
        self._gu = torch.zeros(t, first["gate_up"].res.out_f, **bf)
        self._g, self._u = (self._gu[:, a:a + n] for a, n in first["gate_up"].res.sections)
        self._a = torch.zeros(t, cfg.n_heads * cfg.head_dim, **bf)
        self._act = torch.zeros(t, cfg.intermediate, **bf)
        self._attn = AttnDecode(cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, dev, splits=model._attn.splits, batch=t)
        self.tok = torch.zeros(t, dtype=torch.long, device=dev)
        self.pos0 = torch.zeros(1, dtype=torch.int32, device=dev)                 # position of the first row
        self.pos_rows = torch.zeros(t, dtype=torch.int32, device=dev)             # pos0 + r
        self._ramp = torch.arange(t, dtype=torch.int32, device=dev)
        self.logits = None
        self.graph = None

    def _lin(self, res, x, out):
        return res.gemv(x, out=out) if self.t <= 8 else res.gemm(x, out=out)

    def _forward(self):
        from . import glue as G

        m, cfg = self.m, self.m.cfg
        torch.add(self._ramp, self.pos0, out=self.pos_rows)
        torch.index_select(m.embed, 0, self.tok, out=self._h)
        delta = None
        for li in range(cfg.n_layers):
            L = m.layers[li]
            G.add_rmsnorm(self._h, delta, m.ln1[li], cfg.rms_eps, out=self._xn)
            self._lin(L["qkv"].res, self._xn, self._qkv)
            G.rope_kv(self._q, self._k, self._v, self.pos0, m.k_cache[li], m.v_cache[li], m.cos, m.sin,
                      cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)              # rows = consecutive positions pos0 + r
            self._attn(self._q, m.k_cache[li], m.v_cache[li], self.pos_rows, out=self._a, q_stride=self._qkv.shape[1],
                       shared_cache=True)
            self._lin(L["o_proj"]._res, self._a, self._d)
            G.add_rmsnorm(self._h, self._d, m.ln2[li], cfg.rms_eps, out=self._xn)
            self._lin(L["gate_up"].res, self._xn, self._gu)
            G.swiglu(self._g, self._u, out=self._act)
            self._lin(L["down_proj"]._res, self._act, self._d)
            delta = self._d
        G.add_rmsnorm(self._h, delta, m.ln_f, cfg.rms_eps, out=self._xn)
        return F.linear(self._xn, m.lm_head).float()

    @torch.no_grad()
    def capture(self):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._forward()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self._forward()
        return self

    @torch.no_grad()
    def __call__(self, tokens: torch.Tensor, pos0: int) -> torch.Tensor:
        """tokens [T] at positions pos0 .. pos0 + T - 1; returns logits [T, vocab] (row r = the model's prediction for
        position pos0 + r + 1)."""
        self.tok.copy_(tokens.reshape(self.t))
        self.pos0.fill_(pos0)
        if self.graph is not None:
            self.graph.replay()
            return self.logits
        return self._forward()

    @torch.no_grad()
    def accept(self, tokens: torch.Tensor, pos0: int):
        """tokens[0] is the last confirmed token, tokens[1:] a draft of what follows.  Returns (number of draft tokens the
        model's greedy arg-max confirms, the model's own next token after the confirmed prefix)."""
        pred = self(tokens, pos0).argmax(-1)                          # pred[r]: greedy token for position pos0 + r + 1
        ok = (pred[:-1] == tokens[1:].to(pred.device)).long().cumprod(0)
        n = int(ok.sum().item())
        return n, pred[n]


class BatchedGreedyDecoder:
    """B sequences decoded in lock-step on a packed model: the decode loop of the reference's batched generator
    (ixrun/batching.py:88-234: per-row greedy arg-max, sequences of different lengths, one KV cache per row) without its
    request queue and tokenizer.  Every packed linear sees B rows per step -- the fused GEMV for B <= 8, the tensor-core
    GEMM on the resident layout up to 64 -- and the glue kernels take one row per sequence (its own position, its own
    cache).  One step is one CUDA graph."""

    def __init__(self, model: PackedLlama, batch: int):
        from .glue import AttnDecode

        if model.weights != "packed" or model.glue != "kernels":
            raise ValueError("the batched decoder runs on packed weights and the glue kernels")
        if not 1 <= batch <= 64:
            raise ValueError("1..64 sequences")
        self.m, self.b = model, int(batch)
        cfg, dev = model.cfg, model.embed.device
        bf = dict(dtype=torch.bfloat16, device=dev)
        b = self.b
        self.k_cache = torch.zeros(cfg.n_layers, b, cfg.max_seq, cfg.n_kv_heads, cfg.head_dim, **bf)
        self.v_cache = torch.zeros_like(self.k_cache)
        qd = cfg.n_heads * cfg.head_dim
        first = model.layers[0]
        self._h, self._xn, self._d = (torch.zeros(b, cfg.hidden, **bf) for _ in range(3))
        self._qkv = torch.zeros(b, first["qkv"].res.out_f, **bf)
        self._q, self._k, self._v = (self._qkv[:, a:a + n] for a, n in first["qkv"].res.sections)
        self._gu = torch.zeros(b, first["gate_up"].res.out_f, **bf)
        self._g, self._u = (self._gu[:, a:a + n] for a, n in first["gate_up"].res.sections)
        self._a = torch.zeros(b, qd, **bf)
        self._act = torch.zeros(b, cfg.intermediate, **bf)
        # the same context splits as the one-sequence step: a sequence then gets the same bits alone or in a batch
        self._attn = AttnDecode(cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, dev, splits=model._attn.splits, batch=b)
        self.tok = torch.zeros(b, dtype=torch.long, device=dev)
        self.pos32 = torch.zeros(b, dtype=torch.int32, device=dev)
        self.logits = None
        self.graph = None

    def _lin(self, res, x, out):
        return res.gemv(x, out=out) if self.b <= 8 else res.gemm(x, out=out)

    def _step_kernels(self):
        from . import glue as G

        m, cfg = self.m, self.m.cfg
        torch.index_select(m.embed, 0, self.tok, out=self._h)
        delta = None
        for li in range(cfg.n_layers):
            L = m.layers[li]
            G.add_rmsnorm(self._h, delta, m.ln1[li], cfg.rms_eps, out=self._xn)
            self._lin(L["qkv"].res, self._xn, self._qkv)
            G.rope_kv(self._q, self._k, self._v, self.pos32, self.k_cache[li], self.v_cache[li], m.cos, m.sin,
                      cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, batched=True)
            self._attn(self._q, self.k_cache[li], self.v_cache[li], self.pos32, out=self._a, q_stride=self._qkv.shape[1])
            self._lin(L["o_proj"]._res, self._a, self._d)
            G.add_rmsnorm(self._h, self._d, m.ln2[li], cfg.rms_eps, out=self._xn)
            self._lin(L["gate_up"].res, self._xn, self._gu)
            G.swiglu(self._g, self._u, out=self._act)
            self._lin(L["down_proj"]._res, self._act, self._d)
            delta = self._d
        G.add_rmsnorm(self._h, delta, m.ln_f, cfg.rms_eps, out=self._xn)
        return F.linear(self._xn, m.lm_head).float()

    @torch.no_grad()
    def prefill(self, prompts: list) -> torch.Tensor:
        """Run every prompt through the model (the many-row path), keep its keys and values in the row's own cache;
        returns the first generated token of every sequence [B]."""
        if len(prompts) != self.b:
            raise ValueError(f"{self.b} prompts expected")
        first = []
        for r, ids in enumerate(prompts):
            logits = self.m.prefill(ids)
            n = ids.numel()
            self.k_cache[:, r, :n] = self.m.k_cache[:, :n]
            self.v_cache[:, r, :n] = self.m.v_cache[:, :n]
            self.pos32[r] = n
            first.append(logits.argmax(-1))
        return torch.cat(first)

    @torch.no_grad()
    def capture(self):
        saved = self.pos32.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                self._step_kernels()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.logits = self._step_kernels()
        self.pos32.copy_(saved)
        return self

    @torch.no_grad()
    def step(self, tokens: torch.Tensor) -> torch.Tensor:
        """Feed one token per sequence (at the sequences' current positions); returns logits [B, vocab]."""
        self.tok.copy_(tokens.reshape(self.b))
        if self.graph is not None:
            self.graph.replay()
            out = self.logits
        else:
            out = self._step_kernels()
        self.pos32 += 1
        return out

    @torch.no_grad()
    def generate(self, prompts: list, n_new: int) -> torch.Tensor:
        """Greedy decode of n_new tokens for every prompt; returns [B, n_new]."""
        tok = self.prefill(prompts)
        out = []
        for _ in range(n_new):
            out.append(tok.clone())
            tok = self.step(tok).argmax(-1)
        return torch.stack(out, dim=1)


def synthetic_llama(cfg: LlamaConfig, seed: int = 0, distinct_layers: bool = True):
    """Random-init weights of the config: Laplace codes for every linear (one
    tensor per linear type and layer when distinct_layers, else one per type
    shared by all layers), N(0, 0.02) embeddings and head."""
    from .synth import synthetic_packed

    shapes = linear_shapes(cfg)
    layers = []
    cache = {}
    for li in range(cfg.n_layers):
        d = {}
        for j, n in enumerate(LINEARS):
            key = (li if distinct_layers else 0, n)
            if key not in cache:
                cache[key] = synthetic_packed(*shapes[n], seed=seed * 1000003 + key[0] * 16 + j)
            d[n] = cache[key]
        layers.append(d)
    g = torch.Generator().manual_seed(seed + 17)
    embed = (torch.randn(cfg.vocab, cfg.hidden, generator=g) * 0.02).bfloat16()
    head = (torch.randn(cfg.vocab, cfg.hidden, generator=g) * 0.02).bfloat16()
    return layers, embed, head
