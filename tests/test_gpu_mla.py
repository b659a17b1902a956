"""GPU numerics of the multi-head latent attention kernels (192-wide q/k, 128-wide v) and of the
strided in-place RoPE against plain fp32 PyTorch."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def _inputs(B, S, H, seed, sharp=1.0):
    torch.manual_seed(seed)
    q = torch.randn(B, S, H, 192, device=_dev(), dtype=torch.bfloat16) * sharp
    kv = torch.randn(B, S, H, 256, device=_dev(), dtype=torch.bfloat16)
    kr = torch.randn(B, S, 64, device=_dev(), dtype=torch.bfloat16)
    return q, kv, kr


def _oracle(q, kv, kr, causal):
    """fp32 attention and its log-sum-exp."""
    B, S, H, _ = q.shape
    qf = q.float().transpose(1, 2)
    kn = kv[..., :128].float().transpose(1, 2)
    v = kv[..., 128:].float().transpose(1, 2)
    s = (qf[..., :128] @ kn.transpose(-1, -2) + qf[..., 128:] @ kr.float().view(B, 1, S, 64).transpose(-1, -2))
    s = s / math.sqrt(192)
    if causal:
        s = s.masked_fill(~torch.ones(S, S, dtype=torch.bool, device=q.device).tril(), float("-inf"))
    return (torch.softmax(s, -1) @ v).transpose(1, 2), torch.logsumexp(s, -1)


@pytest.mark.parametrize("B,S,H,causal", [(1, 128, 1, True), (1, 256, 2, True), (2, 1024, 3, True),
                                          (1, 384, 2, False), (1, 200, 2, True), (1, 333, 1, False)])
def test_mla_forward(B, S, H, causal):
    from hyper_parallel_b200.ops import mla_attention as mla
    from hyper_parallel_b200.ops import native
    q, kv, kr = _inputs(B, S, H, 21, sharp=3.0)        # sharper softmax: exercises the rescale path
    out, lse = mla.mla_forward(q, kv, kr, causal=causal)
    native.check_status()
    ref, ref_lse = _oracle(q, kv, kr, causal)
    assert _rel_err(out, ref) < 1.5e-2
    assert torch.allclose(lse, ref_lse, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("B,S,H,causal", [(1, 128, 1, True), (1, 256, 2, True), (2, 1024, 3, True),
                                          (1, 384, 2, False), (1, 200, 2, True)])
def test_mla_backward(B, S, H, causal):
    from hyper_parallel_b200.ops import mla_attention as mla
    from hyper_parallel_b200.ops import native
    q, kv, kr = _inputs(B, S, H, 22)
    do = torch.randn(B, S, H, 128, device=_dev(), dtype=torch.bfloat16)
    out, lse = mla.mla_forward(q, kv, kr, causal=causal)
    dq, dkv, dkr = mla.mla_backward(q, kv, kr, out, lse, do, causal=causal)
    native.check_status()
    qf, kvf, krf = [t.float().requires_grad_() for t in (q, kv, kr)]
    ref, _ = _oracle(qf, kvf, krf, causal)
    rq, rkv, rkr = torch.autograd.grad(ref, (qf, kvf, krf), do.float())
    assert _rel_err(dkv[..., 128:], rkv[..., 128:]) < 2e-2        # dV
    assert _rel_err(dkv[..., :128], rkv[..., :128]) < 2e-2        # dK nope
    assert _rel_err(dkr, rkr) < 2e-2                              # dK rope, summed over heads
    assert _rel_err(dq[..., :128], rq[..., :128]) < 2e-2
    assert _rel_err(dq[..., 128:], rq[..., 128:]) < 2e-2


def test_mla_autograd_from_strided_projection_views():
    """q / kv as views of wider projection outputs (token stride larger than the row), k_rope as the
    tail of the down-projection: the op reads them in place and its gradients match the oracle."""
    from hyper_parallel_b200.ops import mla_attention as mla
    from hyper_parallel_b200.ops import native
    torch.manual_seed(23)
    B, S, H = 2, 256, 2
    qbuf = torch.randn(B, S, H * 192 + 64, device=_dev(), dtype=torch.bfloat16)
    kva = torch.randn(B, S, 512 + 64, device=_dev(), dtype=torch.bfloat16)
    kv = torch.randn(B, S, H, 256, device=_dev(), dtype=torch.bfloat16).requires_grad_()
    qbuf.requires_grad_()
    kva.requires_grad_()
    q = qbuf[..., :H * 192].view(B, S, H, 192)
    kr = kva[..., 512:]
    o = mla.mla_attention(q, kv, kr)
    do = torch.randn_like(o)
    o.backward(do)
    native.check_status()
    qf, kvf, kaf = [t.detach().float().requires_grad_() for t in (qbuf, kv, kva)]
    ref, _ = _oracle(qf[..., :H * 192].view(B, S, H, 192), kvf, kaf[..., 512:], True)
    ref.backward(do.float())
    assert _rel_err(o, ref) < 1.5e-2
    assert _rel_err(qbuf.grad, qf.grad) < 2e-2
    assert _rel_err(kv.grad, kvf.grad) < 2e-2
    assert _rel_err(kva.grad, kaf.grad) < 2e-2


def test_rope_tail_in_place_matches_reference():
    from hyper_parallel_b200.ops import functional as Fn
    from hyper_parallel_b200.ops import mla_attention as mla
    torch.manual_seed(24)
    T, NH, S = 512, 4, 128
    x = torch.randn(T, NH, 192, device=_dev(), dtype=torch.bfloat16)
    ref = x.clone().float()
    ref[..., 128:] = Fn._rope_ref(x[..., 128:].float(), S, 10000.0)
    xa = x.clone().requires_grad_()
    y = mla.rope_tail_(xa * 1.0, 64, S, 10000.0)
    assert _rel_err(y, ref) < 1e-2
    assert torch.equal(y[..., :128], x[..., :128])
    g = torch.randn_like(y)
    y.backward(g)
    gref = g.clone().float()
    gref[..., 128:] = Fn._rope_ref(g[..., 128:].float(), S, 10000.0, None, True)
    assert _rel_err(xa.grad, gref) < 1e-2


def test_deepseek_block_uses_mla_kernels():
    """A DeepSeek-V3 attention block with the real head widths runs on the MLA kernels and agrees with
    the fp32 reference path of the same module."""
    import os
    from hyper_parallel_b200.models.deepseek_v3 import MLA, DeepSeekV3Config
    from hyper_parallel_b200.ops import mla_attention as mla
    from hyper_parallel_b200.ops import native
    torch.manual_seed(25)
    cfg = DeepSeekV3Config.tiny()
    cfg.hidden_size, cfg.num_heads = 256, 2
    cfg.q_lora_rank, cfg.kv_lora_rank = 128, 128
    cfg.qk_nope_head_dim, cfg.qk_rope_head_dim, cfg.v_head_dim = 128, 64, 128
    m = MLA(cfg, device=_dev(), dtype=torch.bfloat16)
    m.reset_parameters()
    with torch.no_grad():
        for w in (m.wq_a, m.wq_b, m.wkv_a, m.wkv_b, m.wo):
            w.normal_(0.0, 0.06)
    B, S = 2, 256
    x = torch.randn(B * S, cfg.hidden_size, device=_dev(), dtype=torch.bfloat16)
    calls = []
    orig = mla._MLAAttention.apply
    outs = {}
    try:
        mla._MLAAttention.apply = lambda *a: (calls.append(1), orig(*a))[1]
        for mode in ("hpb", "ref"):
            os.environ["HPB_MLA"] = mode
            xa = x.clone().requires_grad_()
            for w in m.parameters():
                w.grad = None
            y = m(xa, B, S)
            y.float().square().mean().backward()
            outs[mode] = [y.detach(), xa.grad] + [w.grad.clone() for w in m.parameters()]
    finally:
        mla._MLAAttention.apply = orig
        os.environ.pop("HPB_MLA", None)
    native.check_status()
    assert len(calls) == 1
    for a, b in zip(outs["hpb"], outs["ref"]):
        assert _rel_err(a, b) < 4e-2
