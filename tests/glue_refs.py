"""Plain torch fp32 restatements of the per-token glue operations (test infrastructure, shared by the glue and the
hybrid-model tests).  Values that the eager reference path holds in bf16 tensors are rounded to bf16 at the same
places."""
import torch
import torch.nn.functional as F


def rms_ref(x_bf16, w, eps):
    v = x_bf16.float()
    return (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16) * w


def rope_ref(x, cos, sin, pos, rot):
    """x [T, H, D] fp32, rotate-half over the first `rot` dimensions; pos [T] long"""
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :]
    xr, rest = x[..., :rot], x[..., rot:]
    x1, x2 = xr.chunk(2, dim=-1)
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)


def conv_ref(x, state, w, bias=None):
    """x [C] bf16, state [C, K-1] bf16 (oldest first), w [C, K]; returns (y bf16 [C], new state)"""
    full = torch.cat([state.float(), x.float()[:, None]], dim=1)
    acc = (full * w.float()).sum(-1)
    if bias is not None:
        acc = acc + bias.float()
    return F.silu(acc).to(torch.bfloat16), full[:, 1:].to(torch.bfloat16)


def gdn_ref(qkv, z, a, b, A_log, dt_bias, norm_w, S, hk, hv, eps):
    """One gated-delta-rule step + gated RMSNorm (the published recurrence); S fp32 [hv, 128, 128]."""
    dk = dv = 128
    q = qkv[: hk * dk].float().view(hk, dk)
    k = qkv[hk * dk: 2 * hk * dk].float().view(hk, dk)
    v = qkv[2 * hk * dk:].float().view(hv, dv)
    q = q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    rep = hv // hk
    q, k = q.repeat_interleave(rep, 0), k.repeat_interleave(rep, 0)
    g = torch.exp(-A_log.exp() * F.softplus(a.float() + dt_bias))
    beta = torch.sigmoid(b.float())
    S = S * g[:, None, None]
    kv = torch.einsum("hij,hi->hj", S, k)
    delta = (v - kv) * beta[:, None]
    S = S + k[:, :, None] * delta[:, None, :]
    o = torch.einsum("hij,hi->hj", S, q).to(torch.bfloat16).float()
    o = (o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16) * norm_w
    out = o * F.silu(z.float().view(hv, dv)).to(torch.bfloat16)
    return out.reshape(-1), S


def attn_ref(q, k_cache, v_cache, n_ctx, gate=None):
    """q [hq, D] bf16; caches [S, hkv, D]; positions 0 .. n_ctx - 1; returns bf16 [hq * D]"""
    hq, d = q.shape
    rep = hq // k_cache.shape[1]
    kk = k_cache[:n_ctx].float().repeat_interleave(rep, dim=1).transpose(0, 1)
    vv = v_cache[:n_ctx].float().repeat_interleave(rep, dim=1).transpose(0, 1)
    att = torch.softmax(q.float()[:, None, :] @ kk.transpose(1, 2) * d ** -0.5, dim=-1) @ vv
    o = att.reshape(hq * d).to(torch.bfloat16)
    if gate is not None:
        o = o * torch.sigmoid(gate.float()).to(torch.bfloat16)
    return o
