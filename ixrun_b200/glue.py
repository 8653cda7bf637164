"""Per-token glue kernels of a decode step (see ``csrc/ixb_glue.cuh``): thin wrappers over the C ABI.

The reference leaves this work to HuggingFace eager code and to fla's Triton
kernels (ixrun/fla_patch.py:23-72).  Every function is one launch (attention:
two) on the current stream, allocates nothing when its outputs are passed in,
and can be captured in a CUDA graph: positions are device tensors.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["gdn_conv_step", "add_rmsnorm", "finish_add_rmsnorm", "swiglu", "rope_kv", "AttnDecode", "conv_update", "gdn_step", "rope_tables"]


def _st(t):
    return _lib.stream_ptr(t.device)


def _bf16(*ts):
    for t in ts:
        if t is not None and (t.dtype != torch.bfloat16 or not t.is_contiguous() or not t.is_cuda):
            raise ValueError("glue kernels take contiguous bf16 CUDA tensors")


def add_rmsnorm(h: torch.Tensor, delta: torch.Tensor | None, w: torch.Tensor, eps: float, out: torch.Tensor | None = None):
    """h [rows, hidden] += delta (in place; None: no add); returns rmsnorm(h) * w."""
    _bf16(h, delta, w)
    rows, hidden = h.reshape(-1, h.shape[-1]).shape
    if out is None:
        out = torch.empty_like(h)
    with torch.cuda.device(h.device):
        _lib.check(_lib.lib().ixb_add_rmsnorm(h.data_ptr(), None if delta is None else delta.data_ptr(), w.data_ptr(),
                                              float(eps), out.data_ptr(), rows, hidden, _st(h)))
    return out


def finish_add_rmsnorm(ar, h: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor | None = None):
    """Second half of a row-parallel exchange (after ``P6Packed.gemv_push(x, ar)``) fused with the residual add and the
    RMSNorm that follow it: h [rows, hidden] += bf16(sum over the ranks' partial sums); returns rmsnorm(h) * w.
    The same bits as ``ar.finish`` into a bf16 vector followed by ``add_rmsnorm``."""
    _bf16(h, w)
    rows, hidden = h.reshape(-1, h.shape[-1]).shape
    if out is None:
        out = torch.empty_like(h)
    with torch.cuda.device(h.device):
        _lib.check(_lib.lib().ixb_allreduce_finish_add_rmsnorm(ar._ptrs, ar.rank, ar.world, ar.n_max, h.data_ptr(), w.data_ptr(),
                                                               float(eps), out.data_ptr(), rows, hidden, _st(h)))
    return out


def _rows_view(t: torch.Tensor, what: str):
    """(rows, cols, row pitch) of a bf16 CUDA tensor that is a matrix with unit column stride (a column slice of a wider
    contiguous matrix is fine), or a vector."""
    if t.dtype != torch.bfloat16 or not t.is_cuda:
        raise ValueError(f"{what}: bf16 CUDA tensor expected")
    if t.dim() == 1:
        t = t.unsqueeze(0)
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{what}: a [rows, cols] tensor with contiguous columns expected")
    return t.shape[0], t.shape[1], t.stride(0) if t.shape[0] > 1 else t.shape[1]


def swiglu(g: torch.Tensor, u: torch.Tensor, out: torch.Tensor | None = None):
    """silu(g) * u; g and u: vectors, or [rows, cols] matrices that may be column slices of one wider matrix (the two
    halves of a fused gate|up output); out: contiguous [rows, cols]."""
    rows, cols, pitch = _rows_view(g, "g")
    if _rows_view(u, "u") != (rows, cols, pitch):
        raise ValueError("g and u must have the same shape and row pitch")
    if out is None:
        out = torch.empty(g.shape, dtype=torch.bfloat16, device=g.device)
    _bf16(out)
    with torch.cuda.device(g.device):
        _lib.check(_lib.lib().ixb_swiglu(g.data_ptr(), u.data_ptr(), out.data_ptr(), rows, cols, pitch, _st(g)))
    return out


def rope_tables(max_seq: int, rot_dim: int, theta: float, device):
    """fp32 cos / sin [max_seq][rot_dim / 2] of the rotate-half convention (the tables the eager path builds)."""
    half = rot_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, half, dtype=torch.float32) / half))
    ang = torch.arange(max_seq, dtype=torch.float32)[:, None] * inv[None, :]
    return ang.cos().to(device).contiguous(), ang.sin().to(device).contiguous()


def rope_kv(q, k, v, pos, k_cache, v_cache, cos, sin, hq: int, hkv: int, head_dim: int, rot_dim: int | None = None,
            q_norm=None, k_norm=None, eps: float = 1e-6, q_stride: int | None = None, batched: bool = False):
    """q [rows, >= hq*head_dim] rotated in place; k, v [rows, hkv*head_dim] (column slices allowed) into the caches.
    batched=False: one sequence, caches [max_seq, hkv, head_dim], the rows are positions pos[0] + row (pos: int32 device
    tensor of one element).  batched=True: row r is the newest token of sequence r: caches [rows, max_seq, hkv, head_dim],
    pos int32 [rows]."""
    _bf16(k_cache, v_cache, q_norm, k_norm)
    if pos.dtype != torch.int32 or not pos.is_cuda:
        raise ValueError("pos must be an int32 CUDA tensor")
    rows, kcols, kv_pitch = _rows_view(k, "k")
    if _rows_view(v, "v") != (rows, kcols, kv_pitch) or kcols != hkv * head_dim:
        raise ValueError("k and v must be [rows, hkv*head_dim] with the same row pitch")
    if q_stride is None:
        q_stride = _rows_view(q, "q")[2]
    max_seq = k_cache.shape[-3]
    batch_stride = max_seq * hkv * head_dim if batched else 0
    if batched and (k_cache.dim() != 4 or k_cache.shape[0] < rows or pos.numel() < rows):
        raise ValueError("batched caches are [rows, max_seq, hkv, head_dim] with one position per row")
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().ixb_rope_kv(q.data_ptr(), k.data_ptr(), v.data_ptr(), pos.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), None if q_norm is None else q_norm.data_ptr(),
                                          None if k_norm is None else k_norm.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                          rows, hq, hkv, head_dim, rot_dim or head_dim, float(eps), q_stride, max_seq,
                                          kv_pitch, batch_stride, _st(q)))
    return q


class AttnDecode:
    """Single-query grouped-query attention over static KV caches, for one sequence or a batch of them; owns the scratch
    of the context splits."""

    def __init__(self, hq: int, hkv: int, head_dim: int, device, splits: int | None = None, batch: int = 1):
        self.hq, self.hkv, self.d, self.batch = hq, hkv, head_dim, int(batch)
        if splits is None:
            # one CTA looks after all query heads of a KV head (group sizes 2, 3, 4, 6, 8; else one head per CTA):
            # as many context splits as give about one CTA per SM
            sms = torch.cuda.get_device_properties(device).multi_processor_count
            rep = hq // hkv
            groups = hq // rep if rep in (2, 3, 4, 6, 8) else hq
            splits = max(1, min(256, sms // (groups * self.batch)))
        self.splits = int(splits)
        self.scratch = torch.empty(self.batch * _lib.lib().ixb_attn_scratch_bytes(hq, head_dim, self.splits), dtype=torch.uint8,
                                   device=device)

    def __call__(self, q, k_cache, v_cache, pos, out=None, gate=None, gate_stride: int | None = None, scale: float | None = None,
                 q_stride: int | None = None, gate_row_stride: int = 0, shared_cache: bool = False):
        """One sequence: q [hq*head_dim] (contiguous heads), caches [max_seq, hkv, head_dim], pos int32 [1] = index of
        the newest key; returns out [hq*head_dim] (optionally gated by sigmoid(gate[head*gate_stride + d])).
        A batch (constructed with batch = B): q [B, >= hq*head_dim] (row pitch q_stride, default its own), caches
        [B, max_seq, hkv, head_dim], pos int32 [B]; returns out [B, hq*head_dim].  shared_cache=True: the B queries
        are B positions of ONE sequence (caches [max_seq, hkv, head_dim], pos[r] = index of the newest key query r may
        see): causal attention of a short run of new tokens, as in the verification step of speculative decoding."""
        _bf16(k_cache, v_cache)
        b = self.batch
        if b > 1:
            if q_stride is None:
                q_stride = _rows_view(q, "q")[2]
            if pos.numel() < b or (not shared_cache and (k_cache.dim() != 4 or k_cache.shape[0] < b)):
                raise ValueError("batched caches are [B, max_seq, hkv, head_dim] with one position per sequence")
        batch_stride = k_cache.shape[-3] * self.hkv * self.d if b > 1 and not shared_cache else 0
        if out is None:
            out = torch.empty((b, self.hq * self.d) if b > 1 else (self.hq * self.d,), dtype=torch.bfloat16, device=q.device)
        with torch.cuda.device(q.device):
            _lib.check(_lib.lib().ixb_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), pos.data_ptr(),
                                                  None if gate is None else gate.data_ptr(),
                                                  gate_stride if gate_stride is not None else self.d, out.data_ptr(),
                                                  self.scratch.data_ptr(), self.scratch.numel(), self.hq, self.hkv, self.d,
                                                  self.splits, float(scale if scale is not None else self.d ** -0.5), b,
                                                  q_stride or 0, batch_stride, gate_row_stride, _st(q)))
        return out


def conv_update(x, state, w, bias=None, out=None):
    """x [C]; state [C, K-1] (updated in place); w [C, K]; returns silu(conv) [C]."""
    _bf16(x, state, w, bias)
    if out is None:
        out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        _lib.check(_lib.lib().ixb_conv_update(x.data_ptr(), state.data_ptr(), w.data_ptr(),
                                              None if bias is None else bias.data_ptr(), out.data_ptr(), x.numel(),
                                              w.shape[-1], _st(x)))
    return out


def gdn_step(qkv, z, a, b, A_log, dt_bias, norm_w, state, hk: int, hv: int, eps: float = 1e-6, out=None):
    """One gated-delta-rule step for all value heads; state fp32 [hv, 128, 128] updated in place; returns [hv*128]."""
    _bf16(qkv, z, a, b, norm_w)
    if state.dtype != torch.float32 or A_log.dtype != torch.float32 or dt_bias.dtype != torch.float32:
        raise ValueError("state, A_log and dt_bias are fp32")
    if out is None:
        out = torch.empty(hv * 128, dtype=torch.bfloat16, device=qkv.device)
    with torch.cuda.device(qkv.device):
        _lib.check(_lib.lib().ixb_gdn_step(qkv.data_ptr(), z.data_ptr(), a.data_ptr(), b.data_ptr(), A_log.data_ptr(),
                                           dt_bias.data_ptr(), norm_w.data_ptr(), state.data_ptr(), out.data_ptr(), hk, hv,
                                           float(eps), _st(qkv)))
    return out


def gdn_conv_step(qkv_raw, conv_state, conv_w, pos, z, a, b, A_log, dt_bias, norm_w, state, hk: int, hv: int,
                  eps: float = 1e-6, out=None):
    """``conv_update`` (kernel size 4, no bias) + ``gdn_step`` in one launch.  conv_state: bf16 [2, C, 3] with
    C = (2 hk + hv) * 128 -- the step at position pos[0] reads copy pos[0] & 1 and writes the other one, so pos (int32
    device tensor) must advance by one per step."""
    _bf16(qkv_raw, conv_state, conv_w, z, a, b, norm_w)
    if conv_state.shape != (2, (2 * hk + hv) * 128, 3) or conv_w.shape[-1] != 4:
        raise ValueError("conv_state must be [2, (2 hk + hv) * 128, 3] and the kernel size 4")
    if state.dtype != torch.float32 or A_log.dtype != torch.float32 or dt_bias.dtype != torch.float32 or pos.dtype != torch.int32:
        raise ValueError("state, A_log and dt_bias are fp32, pos int32")
    if out is None:
        out = torch.empty(hv * 128, dtype=torch.bfloat16, device=qkv_raw.device)
    with torch.cuda.device(qkv_raw.device):
        _lib.check(_lib.lib().ixb_gdn_conv_step(qkv_raw.data_ptr(), conv_state.data_ptr(), conv_w.data_ptr(), pos.data_ptr(),
                                                z.data_ptr(), a.data_ptr(), b.data_ptr(), A_log.data_ptr(), dt_bias.data_ptr(),
                                                norm_w.data_ptr(), state.data_ptr(), out.data_ptr(), hk, hv, float(eps),
                                                _st(qkv_raw)))
    return out
