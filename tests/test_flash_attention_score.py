"""``flash_attention_score``: single-device semantics against an explicit-mask oracle, and the
distributed rule (DP / MP / SP over the five layouts and sparse modes, packed sequences, error
paths) against the single-device operator.  Case list after the reference's
``tests/torch/shard/ops/parallel_op_flash_attention_score.py``."""
import math

import pytest
import torch

from dist_utils import run_distributed

B, S, N, NKV, D = 2, 16, 4, 2, 8
SCALE = 1.0 / math.sqrt(D)


def _qkv(seed=0, s=S, skv=None):
    g = torch.Generator().manual_seed(seed)
    skv = skv or s
    return (torch.randn(B, s, N, D, generator=g), torch.randn(B, skv, NKV, D, generator=g),
            torch.randn(B, skv, NKV, D, generator=g))


def _oracle(q, k, v, keep):
    kk = k.repeat_interleave(N // NKV, 2)
    vv = v.repeat_interleave(N // NKV, 2)
    s = torch.einsum("bqnd,bknd->bnqk", q, kk) * SCALE
    s = s.masked_fill(~keep, float("-inf"))
    return torch.einsum("bnqk,bknd->bqnd", torch.softmax(s, -1), vv)


def _as(t, fmt):
    if fmt == "BSND":
        return t
    if fmt == "BNSD":
        return t.transpose(1, 2).contiguous()
    if fmt == "BSH":
        return t.reshape(t.shape[0], t.shape[1], -1)
    if fmt == "SBH":
        return t.reshape(t.shape[0], t.shape[1], -1).transpose(0, 1).contiguous()
    raise AssertionError(fmt)


def test_layouts_and_sparse_modes_single_device():
    from hyper_parallel_b200.ops.flash_attention_score import flash_attention_score as fas
    q, k, v = _qkv(skv=24)
    sq, skv = S, 24
    i = torch.arange(sq)[:, None]
    j = torch.arange(skv)[None, :]
    d = skv - sq
    user_mask = torch.rand(sq, skv, generator=torch.Generator().manual_seed(4)) < 0.3
    user_mask[:, 0] = False
    cases = [
        (dict(sparse_mode=0), torch.ones(sq, skv, dtype=torch.bool)),
        (dict(sparse_mode=0, pre_tockens=3, next_tockens=2), ((i - j) <= 3) & ((j - i) <= 2)),
        (dict(sparse_mode=0, atten_mask=user_mask), ~user_mask),
        (dict(sparse_mode=1, atten_mask=user_mask, pre_tockens=1, next_tockens=1), ~user_mask),
        (dict(sparse_mode=2), j <= i),
        (dict(sparse_mode=3), j <= i + d),
        (dict(sparse_mode=4, pre_tockens=5, next_tockens=1), ((j - i - d) >= -5) & ((j - i - d) <= 1)),
    ]
    for kw, keep in cases:
        ref = _oracle(q, k, v, keep)
        for fmt in ("BSND", "BNSD", "BSH", "SBH"):
            out, smax, ssum, placeholder = fas(_as(q, fmt), _as(k, fmt), _as(v, fmt), N, fmt, scale=SCALE, **kw)
            assert torch.allclose(out, _as(ref, fmt), atol=1e-5), (kw.get("sparse_mode"), fmt)
            assert smax.shape == (B, N, sq, 8) and ssum.shape == (B, N, sq, 8) and placeholder.numel() == 0
    # the statistics reproduce the log-sum-exp of the scores
    out, smax, ssum, _ = fas(q, k, v, N, "BSND", scale=SCALE, sparse_mode=3)
    kk = k.repeat_interleave(N // NKV, 2)
    s = (torch.einsum("bqnd,bknd->bnqk", q, kk) * SCALE).masked_fill(~(j <= i + d), float("-inf"))
    assert torch.allclose(smax[..., 0] + ssum[..., 0].log(), torch.logsumexp(s, -1), atol=1e-5)
    # pse is added before the scale
    pse = torch.randn(B, N, sq, skv, generator=torch.Generator().manual_seed(8))
    out, *_ = fas(q, k, v, N, "BSND", pse=pse, scale=SCALE)
    s = (torch.einsum("bqnd,bknd->bnqk", q, kk) + pse) * SCALE
    assert torch.allclose(out, torch.einsum("bnqk,bknd->bqnd", torch.softmax(s, -1),
                                            v.repeat_interleave(N // NKV, 2)), atol=1e-5)
    # gradients flow through every layout
    qg = _as(q, "BSH").clone().requires_grad_()
    fas(qg, _as(k, "BSH"), _as(v, "BSH"), N, "BSH", scale=SCALE, sparse_mode=2)[0].sum().backward()
    assert qg.grad is not None and torch.isfinite(qg.grad).all()
    with pytest.raises(ValueError):
        fas(q, k, v, N, "BHSD")
    with pytest.raises(ValueError):
        fas(q, k, v, N, "BSND", sparse_mode=1)
    with pytest.raises(ValueError):
        fas(q, k, v, N, "BSND", sparse_mode=7)


def test_packed_sequences_single_device():
    from hyper_parallel_b200.ops.flash_attention_score import flash_attention_score as fas
    g = torch.Generator().manual_seed(2)
    lens = [5, 9, 2]
    t = sum(lens)
    q, k, v = torch.randn(t, N, D, generator=g), torch.randn(t, NKV, D, generator=g), torch.randn(t, NKV, D, generator=g)
    ends = [5, 14, 16]
    out, smax, ssum, _ = fas(q, k, v, N, "TND", scale=SCALE, sparse_mode=3, actual_seq_qlen=ends,
                             actual_seq_kvlen=ends)
    a = 0
    for b in ends:
        n = b - a
        i = torch.arange(n)[:, None]
        j = torch.arange(n)[None, :]
        kk = k[a:b].repeat_interleave(N // NKV, 1)
        vv = v[a:b].repeat_interleave(N // NKV, 1)
        s = (torch.einsum("qnd,knd->nqk", q[a:b], kk) * SCALE).masked_fill(~(j <= i), float("-inf"))
        assert torch.allclose(out[a:b], torch.einsum("nqk,knd->qnd", torch.softmax(s, -1), vv), atol=1e-5)
        a = b
    assert smax.shape == (t, N, 8) and ssum.shape == (t, N, 8)
    with pytest.raises(ValueError):
        fas(q, k, v, N, "TND", scale=SCALE)
    with pytest.raises(ValueError):
        fas(q, k, v, N, "TND", actual_seq_qlen=[5, 3], actual_seq_kvlen=[5, 16])


def test_shard_parameter_rewrites():
    """The rewritten (mode, pre, next) of a query shard selects the same pairs as the global mask."""
    from hyper_parallel_b200.core.shard.ops.parallel_flash_attention_score import (shard_mask_params,
                                                                                    shard_packed_lengths)
    from hyper_parallel_b200.ops.flash_attention_score import keep_mask
    n, local_q = 4, 4
    for skv in (16, 24):
        sq = n * local_q
        for mode, pre, nxt in [(0, 2147483647, 2147483647), (0, 5, 3), (2, 0, 0), (3, 0, 0), (4, 6, 2), (4, 2147483647, 0)]:
            whole = keep_mask(sq, skv, mode, pre, nxt, None, "cpu")
            if whole is None:
                whole = torch.ones(sq, skv, dtype=torch.bool)
            for r in range(n):
                m2, p2, n2 = shard_mask_params(mode, pre, nxt, r, n, local_q, skv)
                part = keep_mask(local_q, skv, m2, p2, n2, None, "cpu")
                if part is None:
                    part = torch.ones(local_q, skv, dtype=torch.bool)
                assert torch.equal(part.expand(local_q, skv), whole[r * local_q:(r + 1) * local_q]), (skv, mode, r)
    # packed lengths: three sequences of 6, 7 and 3 tokens over 4 ranks of 4 rows
    q_ends = kv_ends = [6, 13, 16]
    got = [shard_packed_lengths(q_ends, kv_ends, r, 4, 16, False) for r in range(4)]
    assert got[0] == ([4, 4, 4], [4, 4, 4])          # rows 0-3 of sequence 0: its first 4 keys, nothing else
    assert got[1] == ([2, 4, 4], [6, 8, 8])          # rows 4-5 end sequence 0; rows 6-7 open sequence 1 (2 keys)
    assert got[3] == ([0, 1, 4], [6, 13, 16])
    assert shard_packed_lengths([4, 8, 12, 16], [4, 8, 12, 16], 2, 4, 4, True) == ([0, 0, 4, 4], [0, 0, 4, 4])


def _dist_worker(rank, world):
    from hyper_parallel_b200 import Layout, distribute_tensor
    from hyper_parallel_b200.ops.flash_attention_score import flash_attention_score as fas, npu_fusion_attention
    lay = Layout((2, 2), ("dp", "sp"), list(range(4)))

    def d(t, *spec):
        return distribute_tensor(t.clone(), lay(*spec))

    q, k, v = _qkv(seed=7)
    specs = {
        # layout: (batch-sharded spec, head-sharded spec, (query seq-sharded spec, kv spec))
        "BSND": (("dp", "None", "None", "None"), ("None", "None", "sp", "None"),
                 (("dp", "sp", "None", "None"), ("dp", "None", "None", "None"))),
        "BNSD": (("dp", "None", "None", "None"), ("None", "sp", "None", "None"),
                 (("dp", "None", "sp", "None"), ("dp", "None", "None", "None"))),
        "BSH": (("dp", "None", "None"), ("None", "None", "sp"),
                (("dp", "sp", "None"), ("dp", "None", "None"))),
        "SBH": (("None", "dp", "None"), ("None", "None", "sp"),
                (("sp", "dp", "None"), ("None", "dp", "None"))),
    }
    modes = [dict(sparse_mode=0), dict(sparse_mode=0, pre_tockens=5, next_tockens=2), dict(sparse_mode=2),
             dict(sparse_mode=3), dict(sparse_mode=4, pre_tockens=6, next_tockens=1)]
    for fmt, (dp_spec, mp_spec, (sp_q, sp_kv)) in specs.items():
        qf, kf, vf = _as(q, fmt), _as(k, fmt), _as(v, fmt)
        for kw in modes:
            want, want_max, want_sum, _ = fas(qf, kf, vf, N, fmt, scale=SCALE, **kw)
            for tag, qs, ks in (("dp", dp_spec, dp_spec), ("mp", mp_spec, mp_spec), ("sp", sp_q, sp_kv)):
                out, smax, ssum, placeholder = fas(d(qf, *qs), d(kf, *ks), d(vf, *ks), N, fmt, scale=SCALE, **kw)
                assert torch.allclose(out.full_tensor(), want, atol=1e-5), (fmt, kw, tag)
                lse = smax.full_tensor()[..., 0] + ssum.full_tensor()[..., 0].log()
                assert torch.allclose(lse, want_max[..., 0] + want_sum[..., 0].log(), atol=1e-5), (fmt, kw, tag)
                assert out.layout.dim_axes == d(qf, *qs).layout.dim_axes
                assert placeholder.to_local().numel() == 0

    # an explicit mask of the global shape is narrowed to the shard's query rows
    mask = torch.rand(S, S, generator=torch.Generator().manual_seed(9)) < 0.25
    mask[:, 0] = False
    want = fas(q, k, v, N, "BSND", atten_mask=mask, scale=SCALE, sparse_mode=1)[0]
    out = npu_fusion_attention(d(q, "dp", "sp", "None", "None"), d(k, "dp", "None", "None", "None"),
                               d(v, "dp", "None", "None", "None"), N, "BSND", atten_mask=mask, scale=SCALE,
                               sparse_mode=1)[0]
    assert torch.allclose(out.full_tensor(), want, atol=1e-5)

    # backward through the sequence-parallel rule
    qd = d(q, "dp", "sp", "None", "None").requires_grad_()
    kd = d(k, "dp", "None", "None", "None").requires_grad_()
    out = fas(qd, kd, d(v, "dp", "None", "None", "None"), N, "BSND", scale=SCALE, sparse_mode=2)[0]
    out.to_local().sum().backward()
    q0 = q.clone().requires_grad_()
    fas(q0, k, v, N, "BSND", scale=SCALE, sparse_mode=2)[0].sum().backward()
    assert torch.allclose(qd.grad, q0.grad.chunk(2, 0)[rank // 2].chunk(2, 1)[rank % 2], atol=1e-5)

    # packed sequences: whole sequences per rank (DP over tokens), and context parallel
    g = torch.Generator().manual_seed(11)
    t = 16
    qt, kt, vt = (torch.randn(t, N, D, generator=g), torch.randn(t, NKV, D, generator=g),
                  torch.randn(t, NKV, D, generator=g))
    flat = Layout((4,), ("cp",), list(range(4)))
    ends = [4, 8, 12, 16]
    want = fas(qt, kt, vt, N, "TND", scale=SCALE, sparse_mode=3, actual_seq_qlen=ends, actual_seq_kvlen=ends)[0]
    sh = lambda x: distribute_tensor(x.clone(), flat("cp", "None", "None"))
    rep = lambda x: distribute_tensor(x.clone(), flat("None", "None", "None"))
    out = fas(sh(qt), sh(kt), sh(vt), N, "TND", scale=SCALE, sparse_mode=3, actual_seq_qlen=ends,
              actual_seq_kvlen=ends)[0]
    assert torch.allclose(out.full_tensor(), want, atol=1e-5)
    ends = [6, 13, 16]
    want = fas(qt, kt, vt, N, "TND", scale=SCALE, sparse_mode=3, actual_seq_qlen=ends, actual_seq_kvlen=ends)[0]
    out, smax, _, _ = fas(sh(qt), rep(kt), rep(vt), N, "TND", scale=SCALE, sparse_mode=3, actual_seq_qlen=ends,
                          actual_seq_kvlen=ends)
    assert torch.allclose(out.full_tensor(), want, atol=1e-5)
    assert smax.to_local().shape == (4, N, 8)

    # error paths
    with pytest.raises(NotImplementedError):      # key/value sequence sharded: ring attention
        fas(d(q, "dp", "sp", "None", "None"), d(k, "dp", "sp", "None", "None"), d(v, "dp", "sp", "None", "None"),
            N, "BSND", scale=SCALE)
    with pytest.raises(ValueError):               # key and value sharded differently
        fas(d(q, "dp", "None", "None", "None"), d(k, "dp", "None", "None", "None"),
            d(v, "None", "None", "None", "None"), N, "BSND", scale=SCALE)
    with pytest.raises(ValueError):               # batch sharding differs between query and key
        fas(d(q, "dp", "None", "None", "None"), d(k, "None", "None", "None", "None"),
            d(v, "None", "None", "None", "None"), N, "BSND", scale=SCALE)
    with pytest.raises(ValueError):               # unknown layout string
        fas(d(q, "dp", "None", "None", "None"), d(k, "dp", "None", "None", "None"),
            d(v, "dp", "None", "None", "None"), N, "BHSD", scale=SCALE)
    with pytest.raises(ValueError):               # context parallel needs right-down causal
        fas(sh(qt), rep(kt), rep(vt), N, "TND", scale=SCALE, sparse_mode=2, actual_seq_qlen=ends,
            actual_seq_kvlen=ends)
    with pytest.raises(ValueError):               # 3 local heads cannot be derived from head_num=5
        fas(d(q, "None", "None", "sp", "None"), d(k, "None", "None", "sp", "None"),
            d(v, "None", "None", "sp", "None"), 5, "BSND", scale=SCALE)


def test_distributed_rule_matches_single_device():
    run_distributed(_dist_worker, 4)
