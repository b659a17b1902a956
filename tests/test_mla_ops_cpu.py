"""CPU checks of the latent-attention entry points: the in-place rotary tail and the fallbacks of
``mla_attention`` agree with the concatenating formulation they replace, values and gradients."""
import torch

from hyper_parallel_b200 import ops
from hyper_parallel_b200.ops import mla_attention as mla


def _cat_formulation(q, kv, k_rope, dn, dr, dv, seq_len, theta):
    """The model code before the cat-free operator: split, rotate, concatenate, expand."""
    T, nh, _ = q.shape
    B = T // seq_len
    q_nope, q_rope = q.split([dn, dr], dim=-1)
    q_rope = ops.apply_rope(q_rope.contiguous(), seq_len, theta)
    k_nope, v = kv.split([dn, dv], dim=-1)
    qh = torch.cat([q_nope, q_rope], dim=-1).view(B, seq_len, nh, dn + dr)
    kh = torch.cat([k_nope, k_rope.view(T, 1, dr).expand(T, nh, dr)], dim=-1).view(B, seq_len, nh, dn + dr)
    return ops.attention.causal_attention(qh, kh, v.reshape(B, seq_len, nh, dv))


def test_rope_tail_and_fallback_match_cat_formulation():
    torch.manual_seed(0)
    B, S, nh, dn, dr, dv = 2, 24, 3, 16, 8, 12
    T = B * S
    q0 = torch.randn(T, nh, dn + dr, dtype=torch.float64)
    kv0 = torch.randn(T, nh, dn + dv, dtype=torch.float64)
    kr0 = torch.randn(T, dr, dtype=torch.float64)
    go = torch.randn(B, S, nh, dv, dtype=torch.float64)

    qa, kva, kra = [t.clone().requires_grad_() for t in (q0, kv0, kr0)]
    ref = _cat_formulation(qa, kva, kra, dn, dr, dv, S, 10000.0)
    ref.backward(go)

    qb, kvb, krb = [t.clone().requires_grad_() for t in (q0, kv0, kr0)]
    qr = mla.rope_tail_(qb * 1.0, dr, S, 10000.0)            # in place on a non-leaf, as in the model
    out = mla.mla_attention(qr.view(B, S, nh, dn + dr), kvb.view(B, S, nh, dn + dv), krb.view(B, S, dr), dn, dv)
    out.backward(go)

    assert torch.allclose(out, ref, atol=1e-9)
    for a, b in ((qa, qb), (kva, kvb), (kra, krb)):
        assert torch.allclose(a.grad, b.grad, atol=1e-9)


def test_reference_mode_matches_fallback(monkeypatch):
    torch.manual_seed(1)
    B, S, nh, dn, dr, dv = 1, 17, 2, 8, 4, 8
    q = torch.randn(B, S, nh, dn + dr)
    kv = torch.randn(B, S, nh, dn + dv)
    kr = torch.randn(B, S, dr)
    a = mla.mla_attention(q, kv, kr, dn, dv)
    monkeypatch.setenv("HPB_MLA", "ref")
    b = mla.mla_attention(q, kv, kr, dn, dv)
    assert torch.allclose(a, b, atol=1e-5)
    full = mla.mla_attention(q, kv, kr, dn, dv, causal=False)
    assert not torch.allclose(full, b, atol=1e-3)            # the mask matters


def test_embedding_cpu_fallback_matches_torch():
    torch.manual_seed(2)
    w = torch.randn(50, 16, requires_grad=True)
    tok = torch.randint(0, 50, (3, 7))
    out = ops.embedding(tok, w)
    assert torch.equal(out, torch.nn.functional.embedding(tok, w))
    out.sum().backward()
    assert w.grad.abs().sum() > 0
