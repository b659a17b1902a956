"""``flash_attention_score`` on DTensors, one pytest id per case of the reference's catalogue
(``tests/torch/shard/ops/parallel_op_flash_attention_score.py:135-1390``): DP / MP / SP and their 2-D
and 3-D combinations over the five layouts, the sparse modes under sequence and data parallelism,
packed (TND) sequences with DP, MP and context parallelism, the error paths, and the cross checks
against ``scaled_dot_product_attention``.

All cases run inside ONE launch of 8 gloo ranks on a (dp=2, sp=2, mp=2) mesh (a module-scoped
fixture); every case compares the distributed result with the single-device operator on the same
inputs and records its own pass / failure, which the parametrised test then reports.
"""
import json
import math
import os
import traceback

import pytest
import torch

from dist_utils import run_distributed

B, S, N, NKV, D = 4, 16, 4, 2, 8
SCALE = 1.0 / math.sqrt(D)
WORLD = 8


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


class _Ctx:
    """Inputs and helpers shared by the cases of one rank."""

    def __init__(self, rank):
        from hyper_parallel_b200 import Layout, distribute_tensor
        from hyper_parallel_b200.ops.flash_attention_score import flash_attention_score
        self.rank = rank
        self.fas = flash_attention_score
        self.lay = Layout((2, 2, 2), ("dp", "sp", "mp"), list(range(WORLD)))
        self.flat = Layout((WORLD,), ("cp",), list(range(WORLD)))
        self.dt = distribute_tensor
        g = torch.Generator().manual_seed(3)
        self.q = torch.randn(B, S, N, D, generator=g)
        self.k = torch.randn(B, S, NKV, D, generator=g)
        self.v = torch.randn(B, S, NKV, D, generator=g)

    def d(self, t, *spec):
        return self.dt(t.clone(), self.lay(*spec))

    def check(self, fmt, q_spec, kv_spec, q=None, k=None, v=None, head_num=N, **kw):
        """Distributed call with the given shardings against the single-device call."""
        q, k, v = [_as(t, fmt) for t in (self.q if q is None else q, self.k if k is None else k,
                                         self.v if v is None else v)]
        kw.setdefault("scale", SCALE)
        want, wmax, wsum, _ = self.fas(q, k, v, head_num, fmt, **kw)
        out, smax, ssum, _ = self.fas(self.d(q, *q_spec), self.d(k, *kv_spec), self.d(v, *kv_spec), head_num, fmt, **kw)
        assert torch.allclose(out.full_tensor(), want, atol=1e-5)
        lse = smax.full_tensor()[..., 0] + ssum.full_tensor()[..., 0].log()
        assert torch.allclose(lse, wmax[..., 0] + wsum[..., 0].log(), atol=1e-5)
        assert out.layout.dim_axes == self.d(q, *q_spec).layout.dim_axes
        return out


R3, R4 = ("None",) * 3, ("None",) * 4
CASES = {}


def case(fn):
    CASES[fn.__name__] = fn
    return fn


# ---- BSH ---------------------------------------------------------------------------------------
@case
def bsh_replicate(c):
    c.check("BSH", R3, R3)


@case
def bsh_dp(c):
    c.check("BSH", ("dp", "None", "None"), ("dp", "None", "None"))


@case
def bsh_mp(c):
    c.check("BSH", ("None", "None", "mp"), ("None", "None", "mp"))


@case
def bsh_sp(c):
    c.check("BSH", ("None", "sp", "None"), R3)


@case
def bsh_dp_mp_2d(c):
    c.check("BSH", ("dp", "None", "mp"), ("dp", "None", "mp"))


@case
def bsh_sp_mp_2d(c):
    c.check("BSH", ("None", "sp", "mp"), ("None", "None", "mp"))


@case
def bsh_dp_sp_mp_3d(c):
    c.check("BSH", ("dp", "sp", "mp"), ("dp", "None", "mp"), sparse_mode=2)


# ---- other layouts -----------------------------------------------------------------------------
@case
def bnsd_dp_mp(c):
    c.check("BNSD", ("dp", "mp", "None", "None"), ("dp", "mp", "None", "None"))


@case
def bnsd_sp(c):
    c.check("BNSD", ("None", "None", "sp", "None"), R4)


@case
def bnsd_sp_correctness(c):
    c.check("BNSD", ("dp", "None", "sp", "None"), ("dp", "None", "None", "None"), sparse_mode=3)


@case
def sbh_dp(c):
    c.check("SBH", ("None", "dp", "None"), ("None", "dp", "None"))


@case
def sbh_sp_mp(c):
    c.check("SBH", ("sp", "None", "mp"), ("None", "None", "mp"), sparse_mode=2)


@case
def bsnd_dp_mp(c):
    c.check("BSND", ("dp", "None", "mp", "None"), ("dp", "None", "mp", "None"))


@case
def bsnd_dp_sp_mp_3d(c):
    c.check("BSND", ("dp", "sp", "mp", "None"), ("dp", "None", "mp", "None"), sparse_mode=3)


# ---- sparse modes under sequence / data parallelism ------------------------------------------------
@case
def sp_sparse_mode_0(c):
    c.check("BSH", ("None", "sp", "None"), R3, sparse_mode=0)


@case
def sp_sparse_mode_0_band(c):
    c.check("BSH", ("None", "sp", "None"), R3, sparse_mode=0, pre_tockens=5, next_tockens=2)


@case
def sp_sparse_mode_2(c):
    c.check("BSH", ("None", "sp", "None"), R3, sparse_mode=2)


@case
def sp_sparse_mode_3(c):
    c.check("BSH", ("None", "sp", "None"), R3, sparse_mode=3)


@case
def sp_sparse_mode_4(c):
    c.check("BSH", ("None", "sp", "None"), R3, sparse_mode=4, pre_tockens=6, next_tockens=1)


@case
def sp_sparse_mode_2_with_2way_split(c):
    c.check("BSND", ("dp", "sp", "None", "None"), ("dp", "None", "None", "None"), sparse_mode=2)


@case
def sp_sparse_mode_3_with_2way_split(c):
    c.check("BSND", ("dp", "sp", "None", "None"), ("dp", "None", "None", "None"), sparse_mode=3)


@case
def dp_sparse_mode_1(c):
    mask = torch.rand(S, S, generator=torch.Generator().manual_seed(9)) < 0.25
    mask[:, 0] = False
    c.check("BSH", ("dp", "None", "None"), ("dp", "None", "None"), sparse_mode=1, atten_mask=mask)


@case
def sp_sparse_mode_1_mask_is_narrowed(c):
    mask = torch.rand(S, S, generator=torch.Generator().manual_seed(10)) < 0.25
    mask[:, 0] = False
    c.check("BSND", ("dp", "sp", "None", "None"), ("dp", "None", "None", "None"), sparse_mode=1, atten_mask=mask)


@case
def dp_sparse_mode_4(c):
    c.check("BSH", ("dp", "None", "None"), ("dp", "None", "None"), sparse_mode=4, pre_tockens=4, next_tockens=0)


# ---- options ------------------------------------------------------------------------------------
@case
def bsh_custom_scale(c):
    c.check("BSH", ("dp", "None", "mp"), ("dp", "None", "mp"), scale=0.37)


@case
def bsh_dropout(c):
    # keep_prob < 1 draws a mask: only shapes and layout can be compared
    q, k, v = [_as(t, "BSH") for t in (c.q, c.k, c.v)]
    spec = ("dp", "None", "None")
    out = c.fas(c.d(q, *spec), c.d(k, *spec), c.d(v, *spec), N, "BSH", scale=SCALE, keep_prob=0.9)[0]
    assert out.full_tensor().shape == q.shape and torch.isfinite(out.full_tensor()).all()


@case
def bsh_long_sequence_sp(c):
    g = torch.Generator().manual_seed(21)
    q, k, v = (torch.randn(2, 64, N, D, generator=g), torch.randn(2, 64, NKV, D, generator=g),
               torch.randn(2, 64, NKV, D, generator=g))
    c.check("BSH", ("None", "sp", "None"), R3, q=q, k=k, v=v, sparse_mode=2)


@case
def bsh_large_batch_dp(c):
    g = torch.Generator().manual_seed(22)
    q, k, v = (torch.randn(16, 8, N, D, generator=g), torch.randn(16, 8, NKV, D, generator=g),
               torch.randn(16, 8, NKV, D, generator=g))
    c.check("BSH", ("dp", "None", "None"), ("dp", "None", "None"), q=q, k=k, v=v)


@case
def bsh_redistribute_then_attention(c):
    q, k, v = [_as(t, "BSH") for t in (c.q, c.k, c.v)]
    want = c.fas(q, k, v, N, "BSH", scale=SCALE, sparse_mode=2)[0]
    qd = c.d(q, "dp", "None", "None").redistribute(c.lay("dp", "sp", "None"))
    out = c.fas(qd, c.d(k, "dp", "None", "None"), c.d(v, "dp", "None", "None"), N, "BSH", scale=SCALE, sparse_mode=2)[0]
    assert torch.allclose(out.full_tensor(), want, atol=1e-5)


@case
def sp_backward_matches_single_device(c):
    qd = c.d(c.q, "dp", "sp", "None", "None").requires_grad_()
    kd = c.d(c.k, "dp", "None", "None", "None").requires_grad_()
    out = c.fas(qd, kd, c.d(c.v, "dp", "None", "None", "None"), N, "BSND", scale=SCALE, sparse_mode=2)[0]
    out.to_local().sum().backward()
    q0 = c.q.clone().requires_grad_()
    c.fas(q0, c.k, c.v, N, "BSND", scale=SCALE, sparse_mode=2)[0].sum().backward()
    dp, sp = c.rank // 4, (c.rank // 2) % 2
    assert torch.allclose(qd.grad, q0.grad.chunk(2, 0)[dp].chunk(2, 1)[sp], atol=1e-5)


# ---- cross validation against scaled_dot_product_attention ----------------------------------------------
def _sdpa(q, k, v, causal):
    kk = k.repeat_interleave(N // NKV, 2).transpose(1, 2)
    vv = v.repeat_interleave(N // NKV, 2).transpose(1, 2)
    return torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), kk, vv, is_causal=causal,
                                                            scale=SCALE).transpose(1, 2)


@case
def fa_vs_sdpa_cross_validation(c):
    for mode, causal in ((0, False), (2, True)):
        got = c.fas(c.q, c.k, c.v, N, "BSND", scale=SCALE, sparse_mode=mode)[0]
        assert torch.allclose(got, _sdpa(c.q, c.k, c.v, causal), atol=1e-5)


@case
def fa_vs_sdpa_distributed_cross_validation(c):
    out = c.check("BSND", ("dp", "sp", "mp", "None"), ("dp", "None", "mp", "None"), sparse_mode=2)
    assert torch.allclose(out.full_tensor(), _sdpa(c.q, c.k, c.v, True), atol=1e-5)


# ---- packed sequences (TND) -------------------------------------------------------------------------
def _tnd(seed=11, t=32):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(t, N, D, generator=g), torch.randn(t, NKV, D, generator=g), torch.randn(t, NKV, D, generator=g))


def _tnd_check(c, q_spec, kv_spec, ends, mode=3, lay=None):
    qt, kt, vt = _tnd()
    lay = lay or c.lay
    want = c.fas(qt, kt, vt, N, "TND", scale=SCALE, sparse_mode=mode, actual_seq_qlen=ends, actual_seq_kvlen=ends)[0]
    sh = lambda x, spec: c.dt(x.clone(), lay(*spec))
    out = c.fas(sh(qt, q_spec), sh(kt, kv_spec), sh(vt, kv_spec), N, "TND", scale=SCALE, sparse_mode=mode,
                actual_seq_qlen=ends, actual_seq_kvlen=ends)[0]
    assert torch.allclose(out.full_tensor(), want, atol=1e-5)


@case
def tnd_dp(c):
    _tnd_check(c, ("dp", "None", "None"), ("dp", "None", "None"), [8, 16, 24, 32])      # whole sequences per rank


@case
def tnd_mp(c):
    _tnd_check(c, ("None", "mp", "None"), ("None", "mp", "None"), [5, 19, 32])


@case
def tnd_dp_mp(c):
    _tnd_check(c, ("dp", "mp", "None"), ("dp", "mp", "None"), [16, 32])


@case
def tnd_dp_correctness(c):
    _tnd_check(c, ("cp", "None", "None"), ("cp", "None", "None"), [4, 8, 12, 16, 20, 24, 28, 32], lay=c.flat)


@case
def tnd_cp(c):
    _tnd_check(c, ("cp", "None", "None"), ("None", "None", "None"), [6, 13, 32], lay=c.flat)


@case
def tnd_dp_kv_sharded(c):
    _tnd_check(c, ("dp", "None", "None"), ("dp", "None", "None"), [16, 32], mode=2)


# ---- error paths --------------------------------------------------------------------------------------
def _raises(exc, fn):
    try:
        fn()
    except exc:
        return
    raise AssertionError(f"expected {exc.__name__}")


@case
def error_kv_strategy_mismatch(c):
    _raises(ValueError, lambda: c.fas(c.d(c.q, "dp", *R3), c.d(c.k, "dp", *R3), c.d(c.v, *R4), N, "BSND", scale=SCALE))


@case
def error_head_num_not_divisible(c):
    spec = ("None", "None", "mp", "None")
    _raises(ValueError, lambda: c.fas(c.d(c.q, *spec), c.d(c.k, *spec), c.d(c.v, *spec), 5, "BSND", scale=SCALE))


@case
def error_kv_seq_sharding_blocked(c):
    spec = ("dp", "sp", "None", "None")
    _raises(NotImplementedError, lambda: c.fas(c.d(c.q, *spec), c.d(c.k, *spec), c.d(c.v, *spec), N, "BSND", scale=SCALE))


@case
def error_bnsd_kv_seq_sharding_blocked(c):
    q, k, v = [_as(t, "BNSD") for t in (c.q, c.k, c.v)]
    spec = ("None", "None", "sp", "None")
    _raises(NotImplementedError, lambda: c.fas(c.d(q, *spec), c.d(k, *spec), c.d(v, *spec), N, "BNSD", scale=SCALE))


@case
def error_sparse_mode_1_no_mask(c):
    spec = ("dp", "None", "None", "None")
    _raises(ValueError, lambda: c.fas(c.d(c.q, *spec), c.d(c.k, *spec), c.d(c.v, *spec), N, "BSND", scale=SCALE,
                                      sparse_mode=1))


@case
def error_tnd_sp_without_actual_seq_len(c):
    qt, kt, vt = _tnd()
    sh = lambda x: c.dt(x.clone(), c.flat("cp", "None", "None"))
    rep = lambda x: c.dt(x.clone(), c.flat("None", "None", "None"))
    _raises(ValueError, lambda: c.fas(sh(qt), rep(kt), rep(vt), N, "TND", scale=SCALE, sparse_mode=3))


@case
def error_batch_sharding_mismatch(c):
    _raises(ValueError, lambda: c.fas(c.d(c.q, "dp", *R3), c.d(c.k, *R4), c.d(c.v, *R4), N, "BSND", scale=SCALE))


@case
def error_hidden_sharding_mismatch(c):
    q, k, v = [_as(t, "BSH") for t in (c.q, c.k, c.v)]
    _raises(ValueError, lambda: c.fas(c.d(q, "None", "None", "mp"), c.d(k, *R3), c.d(v, *R3), N, "BSH", scale=SCALE))


@case
def error_dim_sharding_mismatch(c):
    spec = ("None", "None", "None", "mp")
    _raises(ValueError, lambda: c.fas(c.d(c.q, *spec), c.d(c.k, *spec), c.d(c.v, *spec), N, "BSND", scale=SCALE))


@case
def error_tnd_cp_wrong_sparse_mode(c):
    qt, kt, vt = _tnd()
    sh = lambda x: c.dt(x.clone(), c.flat("cp", "None", "None"))
    rep = lambda x: c.dt(x.clone(), c.flat("None", "None", "None"))
    ends = [6, 13, 32]
    _raises(ValueError, lambda: c.fas(sh(qt), rep(kt), rep(vt), N, "TND", scale=SCALE, sparse_mode=2,
                                      actual_seq_qlen=ends, actual_seq_kvlen=ends))


@case
def error_tnd_cp_qk_global_t_mismatch(c):
    qt, kt, vt = _tnd()
    sh = lambda x: c.dt(x.clone(), c.flat("cp", "None", "None"))
    rep = lambda x: c.dt(x.clone(), c.flat("None", "None", "None"))
    _raises(ValueError, lambda: c.fas(sh(qt), rep(kt[:24]), rep(vt[:24]), N, "TND", scale=SCALE, sparse_mode=3,
                                      actual_seq_qlen=[6, 13, 32], actual_seq_kvlen=[6, 13, 24]))


@case
def error_unknown_layout(c):
    spec = ("dp", "None", "None", "None")
    _raises(ValueError, lambda: c.fas(c.d(c.q, *spec), c.d(c.k, *spec), c.d(c.v, *spec), N, "BHSD", scale=SCALE))


# ---- one launch for all cases ---------------------------------------------------------------------------------
def _worker(rank, world, out_dir):
    ctx = _Ctx(rank)
    results = {}
    for name, fn in CASES.items():
        try:
            fn(ctx)
            results[name] = ""
        except Exception:  # noqa: BLE001  (recorded per case, reported by the parametrised test)
            results[name] = traceback.format_exc()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(results, f)


@pytest.fixture(scope="module")
def results(tmp_path_factory):
    out = tmp_path_factory.mktemp("fas_cases")
    run_distributed(_worker, WORLD, str(out), timeout=600.0)
    merged = {name: [] for name in CASES}
    for r in range(WORLD):
        with open(out / f"rank{r}.json") as f:
            for name, err in json.load(f).items():
                if err:
                    merged[name].append(f"rank {r}:\n{err}")
    return merged


@pytest.mark.parametrize("name", list(CASES))
def test_case(results, name):
    assert not results[name], "\n".join(results[name][:2])
