"""The hybrid decoder's token step on the glue kernels against a plain torch restatement of the same step on the
decoded weights (a small configuration with every kind of layer), eager and from the captured graph."""
import pytest
import torch
import torch.nn.functional as F

from glue_refs import attn_ref, conv_ref, gdn_ref, rms_ref, rope_ref

pytestmark = pytest.mark.gpu


def small():
    from ixrun_b200.hybrid27b import Hybrid27B, HybridConfig

    cfg = HybridConfig(n_layers=4, hidden=512, ffn=1024, vocab=2000, gdn_k_heads=2, gdn_v_heads=4, attn_heads=4,
                       attn_kv_heads=2, attn_dim=256, rot_dim=64)
    return cfg, Hybrid27B(cfg, 1, 0, "cuda", context=40, max_new=16)


def lin(p6, x):
    w = p6.decode(kind="bf16").float()
    return (x.float() @ w.t()).to(torch.bfloat16)


class RefState:
    def __init__(self, m):
        self.k, self.v = m.k_cache.clone(), m.v_cache.clone()
        self.S, self.conv = m.gdn_state.clone(), m.conv_state[:, 0].clone()     # (the model keeps the history twice)


def ref_step(m, st, tok, pos):
    cfg, g = m.cfg, m.geo
    h = m.embed[tok].clone()                                          # [1, hidden] bf16
    for L in m.layers:
        x = rms_ref(h, L["ln1"], cfg.eps)
        s = L["slot"]
        proj = lin(L["in"], x)[0]
        parts = [proj[a:a + n] for a, n in L["in"].sections]
        if L["kind"] == "attn":
            nq, d = g["hq"] * cfg.attn_dim, cfg.attn_dim
            qg, k, v = parts
            p = torch.tensor([pos], device=h.device)
            q = rope_ref(rms_ref(qg[:nq].view(1, g["hq"], d), L["q_norm"], cfg.eps).float(), m.cos, m.sin, p, cfg.rot_dim)
            kk = rope_ref(rms_ref(k.view(1, g["hkv"], d), L["k_norm"], cfg.eps).float(), m.cos, m.sin, p, cfg.rot_dim)
            st.k[s, pos] = kk[0].to(torch.bfloat16)
            st.v[s, pos] = v.view(g["hkv"], d)
            a = attn_ref(q[0].to(torch.bfloat16), st.k[s], st.v[s], pos + 1, gate=qg[nq:])
        else:
            qkv, z, a_, b_ = parts
            qc, st.conv[s] = conv_ref(qkv, st.conv[s], L["conv_w"])
            a, st.S[s] = gdn_ref(qc, z, a_, b_, L["A_log"], L["dt_bias"], L["gn_w"], st.S[s], g["hk"], g["hv"], cfg.eps)
        h = h + lin(L["out"], a[None])
        x = rms_ref(h, L["ln2"], cfg.eps)
        gu = lin(L["gate_up"], x)[0]
        gate, up = [gu[a0:a0 + n] for a0, n in L["gate_up"].sections]
        act = F.silu(gate.float()).to(torch.bfloat16) * up
        h = h + lin(L["down"], act[None])
    xn = rms_ref(h, m.ln_f, cfg.eps)
    return h, F.linear(xn, m.lm_head).float()


def test_token_step_matches_the_torch_restatement_eager_and_captured():
    cfg, m = small()
    with torch.no_grad():
        st = RefState(m)
        m.reset(first_token=7)
        tok, pos = 7, m.context
        got_h, got_tok = [], []
        for i in range(4):
            h_ref, logits_ref = ref_step(m, st, torch.tensor([tok], device="cuda"), pos)
            m.step()
            # the step's h is the residual stream before the last add; compare the normed final state instead
            xn_ref = rms_ref(h_ref, m.ln_f, cfg.eps)
            err = float((m.xn.float() - xn_ref.float()).abs().max() / xn_ref.float().abs().max())
            assert err <= 3e-2, (i, err)                               # a chain of bf16 roundings over 4 blocks
            top = int(m.toks[i].item())
            # the kernel path's token must be (one of) the restatement's best within bf16 noise of the logits
            assert float(logits_ref[0, top]) >= float(logits_ref.max()) - 3e-2 * float(logits_ref.abs().max())
            got_h.append(m.xn.clone())
            got_tok.append(top)
            tok, pos = top, pos + 1
        assert torch.isfinite(m.xn.float()).all()
        # the same decode again from the captured graph: identical bits
        m.k_cache[:, m.context:] = 0
        m.v_cache[:, m.context:] = 0
        m.capture()
        m.reset(first_token=7)
        for i in range(4):
            m.step()
            assert torch.equal(m.xn, got_h[i]), i
            assert int(m.toks[i].item()) == got_tok[i]
