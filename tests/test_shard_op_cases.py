"""Distributed-operator rules, one pytest id per case, all cases in ONE launch of 4 gloo ranks on a
(dp=2, mp=2) mesh: every case runs an operator on DTensors and compares the gathered result with the
same operator on the full tensors.  Case list after the reference's per-operator files
``tests/torch/shard/ops/parallel_op_*.py`` (all / cat / cumsum / elementwise / embedding / expand / isin
/ layernorm / linear / masked_scatter / max / multinomial / new_ones / pad / prod / repeat_interleave /
reshape_view / scaled_dot_product_attention / scatter / softmax / sort / split / squeeze / topk /
transpose_permute / unbind)."""
import json
import os
import traceback

import pytest
import torch
import torch.nn.functional as F

from dist_utils import run_distributed

WORLD = 4
CASES = {}


def case(fn):
    CASES[fn.__name__] = fn
    return fn


class _Ctx:
    def __init__(self, rank):
        import hyper_parallel_b200 as hp
        from hyper_parallel_b200 import Layout, distribute_tensor
        self.hp = hp
        self.rank = rank
        self.lay = Layout((2, 2), ("dp", "mp"), list(range(WORLD)))
        self.dt = distribute_tensor
        g = torch.Generator().manual_seed(11)
        self.X = torch.randn(8, 12, generator=g)
        self.Y = torch.randn(8, 12, generator=g)
        self.W = torch.randn(16, 12, generator=g)
        self.W2 = torch.randn(12, 6, generator=g)
        self.B3 = torch.randn(4, 8, 12, generator=g)
        self.IDX = torch.randint(0, 16, (8, 5), generator=g)
        self.EMB = torch.randn(16, 12, generator=g)
        self.Q = torch.randn(2, 4, 8, 6, generator=g)
        self.K = torch.randn(2, 4, 8, 6, generator=g)
        self.V = torch.randn(2, 4, 8, 6, generator=g)

    def d(self, t, *spec):
        return self.dt(t.clone(), self.lay(*spec))

    def full(self, o):
        if isinstance(o, self.hp.DTensor):
            if o.layout.is_partial():
                o = o.reduce_partial()
            return o.full_tensor()
        return o

    def same(self, got, ref, atol=1e-5):
        got = self.full(got)
        assert got.shape == ref.shape, (tuple(got.shape), tuple(ref.shape))
        if ref.dtype.is_floating_point:
            assert torch.allclose(got.float(), ref.float(), atol=atol, rtol=1e-5)
        else:
            assert torch.equal(got, ref)


def _raises(exc, fn):
    try:
        fn()
    except exc:
        return
    raise AssertionError(f"expected {exc}")


# ---- matmul / linear -----------------------------------------------------------------------------
@case
def matmul_column_parallel(c):
    c.same(torch.matmul(c.d(c.X, "dp", "None"), c.d(c.W2, "None", "mp")), c.X @ c.W2)


@case
def matmul_row_parallel_partial(c):
    out = torch.matmul(c.d(c.X, "dp", "mp"), c.d(c.W2, "mp", "None"))
    assert out.layout.is_partial()
    c.same(out, c.X @ c.W2)


@case
def linear_column_parallel(c):
    c.same(F.linear(c.d(c.X, "dp", "None"), c.d(c.W, "mp", "None")), F.linear(c.X, c.W))


@case
def linear_row_parallel_partial(c):
    c.same(F.linear(c.d(c.X, "dp", "mp"), c.d(c.W, "None", "mp")), F.linear(c.X, c.W))


@case
def linear_with_bias_on_partial_output(c):
    b = torch.arange(16.0)
    c.same(F.linear(c.d(c.X, "dp", "mp"), c.d(c.W, "None", "mp"), c.d(b, "None")), F.linear(c.X, c.W, b))


@case
def bmm_batch_sharded(c):
    a, b = c.B3, c.B3.transpose(1, 2).contiguous()
    c.same(torch.bmm(c.d(a, "dp", "None", "None"), c.d(b, "dp", "None", "None")), torch.bmm(a, b))


# ---- elementwise ------------------------------------------------------------------------------------
@case
def elementwise_add_same_layout(c):
    c.same(c.d(c.X, "dp", "mp") + c.d(c.Y, "dp", "mp"), c.X + c.Y)


@case
def elementwise_broadcast_row(c):
    c.same(c.d(c.X, "dp", "None") * c.d(c.Y[0], "None"), c.X * c.Y[0])


@case
def elementwise_scalar_chain(c):
    c.same((c.d(c.X, "dp", "mp") * 2.0 - 1.0) / 3.0, (c.X * 2.0 - 1.0) / 3.0)


@case
def elementwise_unary_chain(c):
    c.same(torch.tanh(F.gelu(c.d(c.X, "dp", "mp"))).abs().sqrt(), torch.tanh(F.gelu(c.X)).abs().sqrt())


@case
def elementwise_where(c):
    x, y = c.d(c.X, "dp", "mp"), c.d(c.Y, "dp", "mp")
    c.same(torch.where(x > 0, x, y), torch.where(c.X > 0, c.X, c.Y))


@case
def elementwise_masked_fill(c):
    c.same(c.d(c.X, "dp", "mp").masked_fill(c.d(c.Y, "dp", "mp") > 0, -1.0), c.X.masked_fill(c.Y > 0, -1.0))


@case
def elementwise_clamp_pow_exp(c):
    c.same(torch.exp(c.d(c.X, "dp", "mp").clamp(-1, 1)).pow(2), torch.exp(c.X.clamp(-1, 1)).pow(2))


@case
def elementwise_comparison_and_logical(c):
    x, y = c.d(c.X, "dp", "mp"), c.d(c.Y, "dp", "mp")
    c.same((x > y) & (x > 0), (c.X > c.Y) & (c.X > 0))


# ---- reductions -----------------------------------------------------------------------------------------
@case
def sum_over_sharded_dim(c):
    c.same(c.d(c.X, "dp", "mp").sum(1), c.X.sum(1))


@case
def sum_keepdim_over_unsharded_dim(c):
    c.same(c.d(c.X, "dp", "None").sum(1, keepdim=True), c.X.sum(1, keepdim=True))


@case
def mean_all(c):
    c.same(c.d(c.X, "dp", "mp").mean(), c.X.mean())


@case
def amax_over_sharded_dim(c):
    c.same(c.d(c.X, "dp", "mp").amax(1), c.X.amax(1))


@case
def max_dim_values_and_indices(c):
    got = c.d(c.X, "dp", "None").max(1)
    ref = c.X.max(1)
    c.same(got.values, ref.values)
    c.same(got.indices, ref.indices)


@case
def max_over_sharded_dim_partial_values_global_indices(c):
    """The values stay Partial(max) on the mesh axis of the reduced dim; the indices are global."""
    for op in ("max", "min"):
        got = getattr(c.d(c.X, "dp", "mp"), op)(0)
        ref = getattr(c.X, op)(0)
        vals, idx = got
        assert vals.layout.is_partial() and not idx.layout.is_partial()
        assert tuple(vals.layout.alias_tensor_map) == ("mp",)
        c.same(vals, ref.values)
        c.same(idx, ref.indices)
    tie = torch.zeros(8, 4)
    tie[2] = tie[6] = 5.0                                   # the winner appears in both shards: first one counts
    _, idx = c.d(tie, "dp", "None").max(0, keepdim=True)
    c.same(idx, tie.max(0, keepdim=True).indices)


@case
def max_of_two_tensors_is_elementwise(c):
    c.same(torch.max(c.d(c.X, "dp", "mp"), c.d(c.Y, "dp", "mp")), torch.max(c.X, c.Y))
    c.same(torch.min(c.d(c.X, "dp", "None"), c.d(c.Y, "dp", "None")), torch.min(c.X, c.Y))


@case
def sum_and_mean_of_a_pending_sum_stay_pending(c):
    """The product of a row-parallel matmul is Partial(sum); sum and mean are linear and keep it."""
    prod = torch.matmul(c.d(c.X, "dp", "mp"), c.d(c.W2, "mp", "None"))
    assert prod.layout.is_partial()
    ref = c.X @ c.W2
    s = prod.sum()
    assert s.layout.is_partial()
    c.same(s, ref.sum(), atol=1e-4)
    c.same(prod.sum(1), ref.sum(1), atol=1e-4)
    c.same(prod.mean(0, keepdim=True), ref.mean(0, keepdim=True), atol=1e-5)
    _raises(ValueError, lambda: prod.prod())
    _raises(ValueError, lambda: prod.amax(0))


@case
def max_all(c):
    c.same(c.d(c.X, "dp", "mp").max(), c.X.max())


@case
def min_all(c):
    c.same(c.d(c.X, "dp", "mp").min(), c.X.min())


@case
def max_elementwise_two_tensors(c):
    c.same(torch.maximum(c.d(c.X, "dp", "mp"), c.d(c.Y, "dp", "mp")), torch.maximum(c.X, c.Y))


@case
def prod_over_unsharded_dim(c):
    x = c.X[:, :4] * 0.5 + 1.0
    c.same(c.d(x.contiguous(), "dp", "None").prod(1), x.prod(1))


@case
def prod_all(c):
    x = (c.X[:2, :3] * 0.1 + 1.0).contiguous()
    c.same(c.d(x, "None", "None").prod(), x.prod())


@case
def all_and_any(c):
    m = c.X > -3
    c.same(c.d(m, "dp", "mp").all(), m.all())
    c.same(c.d(c.X > 2.5, "dp", "mp").any(), (c.X > 2.5).any())


@case
def all_over_dim(c):
    m = c.X > 0
    c.same(c.d(m, "dp", "None").all(1), m.all(1))


# ---- normalisation / softmax / losses ----------------------------------------------------------------------
@case
def softmax_over_unsharded_dim(c):
    c.same(torch.softmax(c.d(c.X, "dp", "None"), -1), torch.softmax(c.X, -1))


@case
def log_softmax_over_unsharded_dim(c):
    c.same(F.log_softmax(c.d(c.X, "dp", "None"), -1), F.log_softmax(c.X, -1))


@case
def softmax_over_sharded_dim_raises(c):
    _raises(ValueError, lambda: torch.softmax(c.d(c.X, "dp", "mp"), -1))


@case
def layer_norm_batch_and_seq_sharded(c):
    c.same(F.layer_norm(c.d(c.B3, "dp", "mp", "None"), (12,)), F.layer_norm(c.B3, (12,)))


@case
def layer_norm_with_affine(c):
    w, b = torch.linspace(0.5, 1.5, 12), torch.linspace(-1, 1, 12)
    c.same(F.layer_norm(c.d(c.B3, "dp", "None", "None"), (12,), c.d(w, "None"), c.d(b, "None")),
           F.layer_norm(c.B3, (12,), w, b))


@case
def mse_loss_batch_sharded(c):
    c.same(F.mse_loss(c.d(c.X, "dp", "None"), c.d(c.Y, "dp", "None")), F.mse_loss(c.X, c.Y))


# ---- shape operators -------------------------------------------------------------------------------------------
@case
def transpose_swaps_shardings(c):
    out = c.d(c.X, "dp", "mp").transpose(0, 1)
    c.same(out, c.X.transpose(0, 1))
    assert out.layout.alias_tensor_map == ("mp", "dp")


@case
def permute_three_dims(c):
    c.same(c.d(c.B3, "dp", "None", "mp").permute(2, 0, 1), c.B3.permute(2, 0, 1))


@case
def t_method(c):
    c.same(c.d(c.X, "dp", "mp").t(), c.X.t())


@case
def reshape_merges_unsharded_dims(c):
    c.same(c.d(c.B3, "dp", "None", "None").reshape(4, 96), c.B3.reshape(4, 96))


@case
def view_splits_unsharded_dim(c):
    c.same(c.d(c.X, "dp", "None").view(8, 3, 4), c.X.view(8, 3, 4))


@case
def view_keeps_leading_sharded_dim(c):
    c.same(c.d(c.B3, "dp", "None", "None").view(4, 2, 4, 12), c.B3.view(4, 2, 4, 12))


@case
def unsqueeze_then_squeeze(c):
    c.same(c.d(c.X, "dp", "mp").unsqueeze(1).squeeze(1), c.X)


@case
def squeeze_all_size_one_dims(c):
    x = c.X.reshape(8, 1, 12, 1)
    c.same(c.d(x, "dp", "None", "mp", "None").squeeze(), x.squeeze())


@case
def squeeze_negative_dim(c):
    x = c.X.reshape(8, 12, 1)
    c.same(c.d(x, "dp", "mp", "None").squeeze(-1), x.squeeze(-1))


@case
def squeeze_dim_that_is_not_one_is_identity(c):
    c.same(c.d(c.X, "dp", "mp").squeeze(0), c.X.squeeze(0))


@case
def expand_new_size(c):
    x = c.X[:, :1].contiguous()
    c.same(c.d(x, "dp", "None").expand(8, 5), x.expand(8, 5))


@case
def expand_with_minus_one(c):
    x = c.X[:, :1].contiguous()
    c.same(c.d(x, "dp", "None").expand(-1, 7), x.expand(-1, 7))


@case
def expand_adds_leading_dim(c):
    c.same(c.d(c.X, "dp", "None").expand(3, 8, 12), c.X.expand(3, 8, 12))


@case
def expand_as(c):
    x = c.X[:, :1].contiguous()
    c.same(c.d(x, "dp", "None").expand_as(c.d(c.Y, "dp", "None")), x.expand_as(c.Y))


@case
def cat_along_unsharded_dim(c):
    c.same(torch.cat([c.d(c.X, "dp", "None"), c.d(c.Y, "dp", "None")], 1), torch.cat([c.X, c.Y], 1))


@case
def stack_new_leading_dim(c):
    c.same(torch.stack([c.d(c.X, "dp", "None"), c.d(c.Y, "dp", "None")], 0), torch.stack([c.X, c.Y], 0))


@case
def chunk_along_unsharded_dim(c):
    c.same(c.d(c.X, "dp", "None").chunk(3, 1)[1], c.X.chunk(3, 1)[1])


@case
def split_sizes_along_unsharded_dim(c):
    got = c.d(c.X, "dp", "None").split([5, 7], 1)
    ref = c.X.split([5, 7], 1)
    for g, r in zip(got, ref):
        c.same(g, r)


@case
def split_int_along_unsharded_dim(c):
    got = torch.split(c.d(c.X, "dp", "None"), 4, 1)
    ref = torch.split(c.X, 4, 1)
    assert len(got) == len(ref)
    for g, r in zip(got, ref):
        c.same(g, r)


@case
def split_along_sharded_dim_raises(c):
    _raises(Exception, lambda: c.d(c.X, "dp", "mp").split(3, 1))


@case
def unbind_unsharded_dim(c):
    got = c.d(c.B3, "None", "dp", "mp").unbind(0)
    ref = c.B3.unbind(0)
    assert len(got) == len(ref)
    for g, r in zip(got, ref):
        c.same(g, r)


@case
def unbind_sharded_dim_raises(c):
    _raises(Exception, lambda: c.d(c.B3, "dp", "None", "None").unbind(0))


@case
def slice_unsharded_dim(c):
    c.same(c.d(c.X, "dp", "None")[:, 2:7], c.X[:, 2:7])


@case
def repeat_interleave_int(c):
    c.same(c.d(c.X, "dp", "None").repeat_interleave(2, dim=1), c.X.repeat_interleave(2, dim=1))


@case
def repeat_interleave_on_batch_sharded_other_dim(c):
    c.same(c.d(c.B3, "dp", "None", "None").repeat_interleave(3, dim=2), c.B3.repeat_interleave(3, dim=2))


@case
def pad_last_dim(c):
    c.same(F.pad(c.d(c.X, "dp", "None"), (1, 2)), F.pad(c.X, (1, 2)))


@case
def pad_with_value(c):
    c.same(F.pad(c.d(c.X, "dp", "None"), (0, 3), value=-2.0), F.pad(c.X, (0, 3), value=-2.0))


@case
def pad_sharded_dim_raises(c):
    _raises(Exception, lambda: F.pad(c.d(c.X, "dp", "mp"), (1, 1)))


# ---- index / gather / scatter / sort ------------------------------------------------------------------------------
@case
def embedding_hidden_sharded_table(c):
    c.same(F.embedding(c.d(c.IDX, "dp", "None"), c.d(c.EMB, "None", "mp")), F.embedding(c.IDX, c.EMB))


@case
def index_select_unsharded_dim(c):
    idx = torch.tensor([0, 3, 5])
    c.same(c.d(c.X, "dp", "None").index_select(1, idx), c.X.index_select(1, idx))


@case
def gather_unsharded_dim(c):
    idx = torch.randint(0, 12, (8, 4), generator=torch.Generator().manual_seed(2))
    c.same(torch.gather(c.d(c.X, "dp", "None"), 1, c.d(idx, "dp", "None")), torch.gather(c.X, 1, idx))


@case
def scatter_unsharded_dim(c):
    idx = torch.stack([torch.randperm(12, generator=torch.Generator().manual_seed(i))[:4] for i in range(8)])
    src = torch.full((8, 4), 9.0)
    c.same(c.d(c.X, "dp", "None").scatter(1, c.d(idx, "dp", "None"), c.d(src, "dp", "None")),
           c.X.scatter(1, idx, src))


@case
def scatter_add_unsharded_dim(c):
    idx = torch.randint(0, 12, (8, 6), generator=torch.Generator().manual_seed(4))
    src = torch.ones(8, 6)
    c.same(c.d(c.X, "dp", "None").scatter_add(1, c.d(idx, "dp", "None"), c.d(src, "dp", "None")),
           c.X.scatter_add(1, idx, src))


@case
def topk_values_and_indices(c):
    got, ref = c.d(c.X, "dp", "None").topk(3, -1), c.X.topk(3, -1)
    c.same(got.values, ref.values)
    c.same(got.indices, ref.indices)


@case
def topk_sharded_dim_raises(c):
    _raises(Exception, lambda: c.d(c.X, "dp", "mp").topk(3, -1))


@case
def sort_ascending(c):
    got, ref = c.d(c.X, "dp", "None").sort(-1), c.X.sort(-1)
    c.same(got.values, ref.values)
    c.same(got.indices, ref.indices)


@case
def sort_descending(c):
    c.same(c.d(c.X, "dp", "None").sort(-1, descending=True).values, c.X.sort(-1, descending=True).values)


@case
def argsort_unsharded_dim(c):
    c.same(c.d(c.X, "dp", "None").argsort(-1), c.X.argsort(-1))


@case
def cumsum_unsharded_dim(c):
    c.same(c.d(c.X, "dp", "None").cumsum(1), c.X.cumsum(1))


@case
def cumsum_batch_sharded_three_dims(c):
    c.same(c.d(c.B3, "dp", "None", "None").cumsum(2), c.B3.cumsum(2))


@case
def cumsum_sharded_dim_raises(c):
    _raises(Exception, lambda: c.d(c.X, "dp", "mp").cumsum(1))


@case
def isin_replicated_test_elements(c):
    el = torch.tensor([0, 3, 7, 15])
    c.same(torch.isin(c.d(c.IDX, "dp", "None"), el), torch.isin(c.IDX, el))


@case
def isin_invert(c):
    el = torch.tensor([1, 2])
    idx = c.IDX[:, :4].contiguous()
    c.same(torch.isin(c.d(idx, "dp", "mp"), el, invert=True), torch.isin(idx, el, invert=True))


@case
def one_hot_batch_sharded(c):
    c.same(F.one_hot(c.d(c.IDX, "dp", "None"), 16), F.one_hot(c.IDX, 16))


# ---- creation from a DTensor -----------------------------------------------------------------------------------------
@case
def new_ones_zeros_full_follow_replicated_layout(c):
    x = c.d(c.X, "dp", "mp")
    for made, ref in ((x.new_ones((4, 6)), torch.ones(4, 6)), (x.new_zeros((4, 6)), torch.zeros(4, 6)),
                      (x.new_full((2, 3), 7.0), torch.full((2, 3), 7.0))):
        c.same(made, ref)


@case
def zeros_like_and_ones_like_keep_layout(c):
    x = c.d(c.X, "dp", "mp")
    z, o = torch.zeros_like(x), torch.ones_like(x)
    assert z.layout.alias_tensor_map == x.layout.alias_tensor_map
    c.same(z, torch.zeros_like(c.X))
    c.same(o, torch.ones_like(c.X))


# ---- random -------------------------------------------------------------------------------------------------------------
@case
def multinomial_rows_are_valid_samples(c):
    p = torch.softmax(c.X, -1)
    s = torch.multinomial(c.d(p, "dp", "None"), 3)
    out = c.full(s)
    assert out.shape == (8, 3) and int(out.min()) >= 0 and int(out.max()) < 12
    for row in out.tolist():
        assert len(set(row)) == 3                       # without replacement


@case
def multinomial_sharded_probability_dim_raises(c):
    p = torch.softmax(c.X, -1)
    _raises(Exception, lambda: torch.multinomial(c.d(p, "dp", "mp"), 2))


@case
def masked_scatter_same_layout(c):
    mask = c.X > 0
    src = torch.arange(96.0).view(8, 12)
    got = c.d(c.X, "None", "None").masked_scatter(c.d(mask, "None", "None"), c.d(src, "None", "None"))
    c.same(got, c.X.masked_scatter(mask, src))


# ---- attention --------------------------------------------------------------------------------------------------------------
@case
def sdpa_batch_and_heads_sharded(c):
    s = ("dp", "mp", "None", "None")
    c.same(F.scaled_dot_product_attention(c.d(c.Q, *s), c.d(c.K, *s), c.d(c.V, *s), is_causal=True),
           F.scaled_dot_product_attention(c.Q, c.K, c.V, is_causal=True))


@case
def sdpa_query_sequence_sharded_causal(c):
    kv = ("dp", "None", "None", "None")
    c.same(F.scaled_dot_product_attention(c.d(c.Q, "dp", "None", "mp", "None"), c.d(c.K, *kv), c.d(c.V, *kv),
                                          is_causal=True),
           F.scaled_dot_product_attention(c.Q, c.K, c.V, is_causal=True))


@case
def sdpa_query_sequence_sharded_full(c):
    kv = ("dp", "None", "None", "None")
    c.same(F.scaled_dot_product_attention(c.d(c.Q, "dp", "None", "mp", "None"), c.d(c.K, *kv), c.d(c.V, *kv)),
           F.scaled_dot_product_attention(c.Q, c.K, c.V))


@case
def sdpa_with_scale(c):
    s = ("dp", "mp", "None", "None")
    c.same(F.scaled_dot_product_attention(c.d(c.Q, *s), c.d(c.K, *s), c.d(c.V, *s), scale=0.3),
           F.scaled_dot_product_attention(c.Q, c.K, c.V, scale=0.3))


@case
def sdpa_with_additive_mask(c):
    mask = torch.randn(8, 8, generator=torch.Generator().manual_seed(3))
    s = ("dp", "mp", "None", "None")
    c.same(F.scaled_dot_product_attention(c.d(c.Q, *s), c.d(c.K, *s), c.d(c.V, *s), attn_mask=mask),
           F.scaled_dot_product_attention(c.Q, c.K, c.V, attn_mask=mask))


@case
def sdpa_query_sequence_sharded_with_explicit_mask(c):
    """A full (S x S) mask with the query sequence sharded: every rank uses the rows of its own queries;
    a mask distributed like the queries is taken as it is."""
    mask = torch.ones(8, 8, dtype=torch.bool).tril()
    q = ("dp", "None", "mp", "None")
    kv = ("dp", "None", "None", "None")
    ref = F.scaled_dot_product_attention(c.Q, c.K, c.V, attn_mask=mask)
    c.same(F.scaled_dot_product_attention(c.d(c.Q, *q), c.d(c.K, *kv), c.d(c.V, *kv), attn_mask=mask), ref)
    add = torch.randn(8, 8, generator=torch.Generator().manual_seed(5))
    ref = F.scaled_dot_product_attention(c.Q, c.K, c.V, attn_mask=add)
    c.same(F.scaled_dot_product_attention(c.d(c.Q, *q), c.d(c.K, *kv), c.d(c.V, *kv),
                                          attn_mask=c.d(add, "mp", "None")), ref)
    _raises(ValueError, lambda: F.scaled_dot_product_attention(
        c.d(c.Q, *q), c.d(c.K, *kv), c.d(c.V, *kv), attn_mask=c.d(add, "None", "mp")))
    _raises(ValueError, lambda: F.scaled_dot_product_attention(
        c.d(c.Q, *kv), c.d(c.K, *kv), c.d(c.V, "dp", "mp", "None", "None")))          # key and value differ


@case
def sdpa_replicated(c):
    c.same(F.scaled_dot_product_attention(c.d(c.Q, *(("None",) * 4)), c.d(c.K, *(("None",) * 4)),
                                          c.d(c.V, *(("None",) * 4)), is_causal=True),
           F.scaled_dot_product_attention(c.Q, c.K, c.V, is_causal=True))


@case
def sdpa_key_sequence_sharded_raises(c):
    kv = ("dp", "None", "mp", "None")
    _raises(NotImplementedError, lambda: F.scaled_dot_product_attention(
        c.d(c.Q, "dp", "None", "None", "None"), c.d(c.K, *kv), c.d(c.V, *kv)))


@case
def sdpa_backward_through_head_sharding(c):
    s = ("dp", "mp", "None", "None")
    qd = c.d(c.Q, *s).requires_grad_()
    out = F.scaled_dot_product_attention(qd, c.d(c.K, *s), c.d(c.V, *s), is_causal=True)
    out.to_local().sum().backward()
    q0 = c.Q.clone().requires_grad_()
    F.scaled_dot_product_attention(q0, c.K, c.V, is_causal=True).sum().backward()
    dp, mp = c.rank // 2, c.rank % 2
    assert torch.allclose(qd.grad, q0.grad.chunk(2, 0)[dp].chunk(2, 1)[mp], atol=1e-5)


# ---- one launch for all cases -----------------------------------------------------------------------------------------------------
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
    out = tmp_path_factory.mktemp("op_cases")
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
    assert not results[name], "\n".join(results[name][:1])
