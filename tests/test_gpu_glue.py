"""Per-token glue kernels against plain torch fp32 references of the same operations (tolerance 1e-3 of the largest
output unless the output itself is a bf16 tensor, where one bf16 rounding, 2^-8, is allowed)."""

import pytest
import torch
import torch.nn.functional as F

from glue_refs import gdn_ref, rope_ref

pytestmark = pytest.mark.gpu

BF16_ULP = 2.0 ** -8


def close(got, ref, tol):
    err = float((got.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-20))
    assert err <= tol, err


@pytest.mark.parametrize("rows,hidden", [(1, 5120), (1, 2048), (3, 640), (8, 5120)])
def test_add_rmsnorm(rows, hidden):
    from ixrun_b200.glue import add_rmsnorm

    h = torch.randn(rows, hidden, device="cuda").bfloat16()
    d = torch.randn(rows, hidden, device="cuda").bfloat16()
    w = (1 + 0.1 * torch.randn(hidden, device="cuda")).bfloat16()
    for delta in (d, None):
        h0 = h.clone()
        hr = (h0 + delta) if delta is not None else h0             # bf16 add, as the eager residual
        v = hr.float()
        ref = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + 1e-5)).to(torch.bfloat16) * w
        hh = h.clone()
        xn = add_rmsnorm(hh, delta, w, 1e-5)
        assert torch.equal(hh, hr)
        close(xn, ref, BF16_ULP)


def test_swiglu():
    from ixrun_b200.glue import swiglu

    g = torch.randn(17408, device="cuda").bfloat16() * 3
    u = torch.randn(17408, device="cuda").bfloat16()
    close(swiglu(g, u), F.silu(g) * u, BF16_ULP)


@pytest.mark.parametrize("hq,hkv,d,rot,norm", [(16, 8, 128, 128, False), (24, 4, 256, 64, True), (3, 1, 256, 256, False)])
def test_rope_kv_and_attention(hq, hkv, d, rot, norm):
    from ixrun_b200.glue import AttnDecode, rope_kv, rope_tables

    dev, max_seq, ctx = "cuda", 512, 300
    cos, sin = rope_tables(max_seq, rot, 10000.0, dev)
    kc = torch.randn(max_seq, hkv, d, device=dev).bfloat16()
    vc = torch.randn(max_seq, hkv, d, device=dev).bfloat16()
    kc0, vc0 = kc.clone(), vc.clone()
    qg = torch.randn(1, 2 * hq * d, device=dev).bfloat16()          # [q | gate], as a gated attention's projection
    k = torch.randn(1, hkv * d, device=dev).bfloat16()
    v = torch.randn(1, hkv * d, device=dev).bfloat16()
    qn = (1 + 0.1 * torch.randn(d, device=dev)).bfloat16() if norm else None
    kn = (1 + 0.1 * torch.randn(d, device=dev)).bfloat16() if norm else None
    pos = torch.tensor([ctx], dtype=torch.int32, device=dev)

    def hnorm(x, w):
        if w is None:
            return x.float()
        f = x.float()
        return ((f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + 1e-6)).to(torch.bfloat16) * w).float()

    q_ref = rope_ref(hnorm(qg[:, :hq * d].view(1, hq, d), qn), cos, sin, pos.long(), rot).to(torch.bfloat16)
    k_ref = rope_ref(hnorm(k.view(1, hkv, d), kn), cos, sin, pos.long(), rot).to(torch.bfloat16)
    q = qg.clone()
    rope_kv(q, k, v, pos, kc, vc, cos, sin, hq, hkv, d, rot_dim=rot, q_norm=qn, k_norm=kn, q_stride=2 * hq * d)
    close(q[:, :hq * d].view(1, hq, d), q_ref, BF16_ULP)
    assert torch.equal(q[:, hq * d:], qg[:, hq * d:])               # the gate half is untouched
    close(kc[ctx], k_ref[0], BF16_ULP)
    assert torch.equal(vc[ctx], v.view(hkv, d))
    mask = torch.ones(max_seq, dtype=torch.bool, device=dev)
    mask[ctx] = False
    assert torch.equal(kc[mask], kc0[mask]) and torch.equal(vc[mask], vc0[mask])

    # attention of the rotated query over positions 0 .. ctx, with and without the sigmoid gate
    rep = hq // hkv
    qq = q[:, :hq * d].view(hq, 1, d).float()
    kk = kc[: ctx + 1].float().repeat_interleave(rep, dim=1).transpose(0, 1)      # [hq, S, d]
    vv = vc[: ctx + 1].float().repeat_interleave(rep, dim=1).transpose(0, 1)
    att = torch.softmax(qq @ kk.transpose(1, 2) * d ** -0.5, dim=-1) @ vv         # [hq, 1, d]
    ref = att.view(hq * d)
    for splits in (1, 7, None):
        ad = AttnDecode(hq, hkv, d, dev, splits=splits)
        out = ad(q[0, :hq * d].contiguous(), kc, vc, pos)
        close(out, ref, BF16_ULP)
    gate = q[0, hq * d:].contiguous()
    out = AttnDecode(hq, hkv, d, dev)(q[0, :hq * d].contiguous(), kc, vc, pos, gate=gate)
    close(out, (ref.to(torch.bfloat16) * torch.sigmoid(gate.float()).to(torch.bfloat16)).float(), 2 * BF16_ULP)
    # a context of one position
    p0 = torch.zeros(1, dtype=torch.int32, device=dev)
    out = AttnDecode(hq, hkv, d, dev)(q[0, :hq * d].contiguous(), kc, vc, p0)
    close(out, vc[0].float().repeat_interleave(rep, dim=0).reshape(-1), BF16_ULP)


def test_conv_update():
    from ixrun_b200.glue import conv_update

    c, k = 10240, 4
    w = torch.randn(c, k, device="cuda").bfloat16()
    bias = torch.randn(c, device="cuda").bfloat16()
    state = torch.randn(c, k - 1, device="cuda").bfloat16()
    hist = state.clone()
    for step in range(5):
        x = torch.randn(c, device="cuda").bfloat16()
        full = torch.cat([hist.float(), x.float()[:, None]], dim=1)                 # [C, K]
        ref = F.silu((full * w.float()).sum(-1) + bias.float())
        y = conv_update(x, state, w, bias if step % 2 == 0 else None)
        if step % 2:
            ref = F.silu((full * w.float()).sum(-1))
        close(y, ref, BF16_ULP)
        hist = full[:, 1:].to(torch.bfloat16)
        assert torch.equal(state, hist)


@pytest.mark.parametrize("hk,hv", [(16, 48), (2, 6), (1, 1)])
def test_gdn_step(hk, hv):
    from ixrun_b200.glue import gdn_step

    dev = "cuda"
    S = torch.randn(hv, 128, 128, device=dev) * 0.1
    A_log = torch.randn(hv, device=dev) * 0.5
    dt_bias = torch.randn(hv, device=dev) * 0.5
    norm_w = (1 + 0.1 * torch.randn(128, device=dev)).bfloat16()
    S_gpu = S.clone()
    for step in range(3):
        qkv = torch.randn(2 * hk * 128 + hv * 128, device=dev).bfloat16()
        z = torch.randn(hv * 128, device=dev).bfloat16()
        a = torch.randn(hv, device=dev).bfloat16()
        b = torch.randn(hv, device=dev).bfloat16()
        ref, S = gdn_ref(qkv, z, a, b, A_log, dt_bias, norm_w, S, hk, hv, 1e-6)
        out = gdn_step(qkv, z, a, b, A_log, dt_bias, norm_w, S_gpu, hk, hv, 1e-6)
        close(S_gpu, S, 1e-4)
        close(out, ref, 2 * BF16_ULP)


@pytest.mark.parametrize("hk,hv", [(16, 48), (2, 6), (1, 1)])
def test_gdn_conv_step_equals_conv_then_gdn(hk, hv):
    """The fused kernel (conv history kept twice, read copy pos & 1, write the other) gives the bits of the conv
    kernel followed by the recurrent kernel, step after step."""
    from ixrun_b200.glue import conv_update, gdn_conv_step, gdn_step

    dev = "cuda"
    C = (2 * hk + hv) * 128
    conv_w = (torch.randn(C, 4, device=dev) * 0.3).bfloat16()
    A_log = torch.randn(hv, device=dev) * 0.5
    dt_bias = torch.randn(hv, device=dev) * 0.5
    norm_w = (1 + 0.1 * torch.randn(128, device=dev)).bfloat16()
    S_a = torch.randn(hv, 128, 128, device=dev) * 0.1
    S_b = S_a.clone()
    hist = torch.randn(C, 3, device=dev).bfloat16()
    start = 5                                              # an odd first position: the first step reads copy 1
    state2 = torch.zeros(2, C, 3, dtype=torch.bfloat16, device=dev)
    state2[start & 1] = hist
    pos = torch.tensor([start], dtype=torch.int32, device=dev)
    for step in range(4):
        qkv = torch.randn(C, device=dev).bfloat16()
        z = torch.randn(hv * 128, device=dev).bfloat16()
        a = torch.randn(hv, device=dev).bfloat16()
        b = torch.randn(hv, device=dev).bfloat16()
        ref = gdn_step(conv_update(qkv, hist, conv_w), z, a, b, A_log, dt_bias, norm_w, S_a, hk, hv, 1e-6)
        out = gdn_conv_step(qkv, state2, conv_w, pos, z, a, b, A_log, dt_bias, norm_w, S_b, hk, hv, 1e-6)
        assert torch.equal(out, ref) and torch.equal(S_a, S_b)
        pos += 1
        assert torch.equal(state2[int(pos.item()) & 1], hist)
