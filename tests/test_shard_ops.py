"""Distributed-op catalogue: layout inference of the rules, and a 4-rank (gloo) battery in which every
op runs on sharded DTensors and its gathered result must equal the single-device op
(the structure of the reference's tests/torch/shard/ops suites and ut/parallel_ops_infer tests)."""
import pytest
import torch
import torch.nn.functional as F

from dist_utils import run_distributed
from hyper_parallel_b200 import Layout
from hyper_parallel_b200.core.shard import _op_dispatch  # noqa: F401  (loads the YAML registry)
from hyper_parallel_b200.core.shard.ops.parallel_ops import get_distributed_op, registered_ops

L = Layout((2, 4), ("dp", "mp"), list(range(8)))


def infer(name, layouts, extra=()):
    out = get_distributed_op(name).infer_layout(layouts, extra)
    outs = out if isinstance(out, (tuple, list)) else (out,)
    return [(tuple(o.alias_tensor_map), list(o.partial)) for o in outs]


def test_registry_covers_the_catalogue():
    ops = set(registered_ops())
    assert len(ops) >= 200
    for name in ["matmul", "linear", "add", "mul", "sum", "mean", "max", "prod", "all", "softmax", "layer_norm",
                 "rms_norm", "embedding", "reshape", "view", "transpose", "permute", "unsqueeze", "squeeze", "expand",
                 "expand_as", "cat", "split", "index_select", "gather", "scatter", "masked_scatter", "topk", "sort",
                 "cumsum", "unbind", "repeat_interleave", "pad", "isin", "multinomial", "new_ones",
                 "scaled_dot_product_attention", "cross_entropy", "mse_loss"]:
        assert name in ops, name


def test_matmul_and_linear_rules():
    assert infer("matmul", (L("dp", "None"), L("None", "mp"))) == [(("dp", "mp"), [None, None])]
    # contracting dim sharded on mp -> Partial(sum) on mp
    assert infer("matmul", (L("dp", "mp"), L("mp", "None"))) == [(("dp", "None"), [None, "sum"])]
    assert infer("linear", (L("dp", "None"), L("mp", "None"), None)) == [(("dp", "mp"), [None, None])]
    assert infer("linear", (L("dp", "mp"), L("None", "mp"), None)) == [(("dp", "None"), [None, "sum"])]
    with pytest.raises(ValueError):
        infer("matmul", (L("dp", "mp"), L("None", "None")))      # contracting dims disagree


def test_elementwise_broadcast_and_reduce_rules():
    assert infer("add", (L("dp", "None"), L("dp", "None")), ((4, 8), (4, 8))) == [(("dp", "None"), [None, None])]
    assert infer("add", (L("dp", "None"), L("None",)), ((4, 8), (8,))) == [(("dp", "None"), [None, None])]
    assert infer("sum", (L("dp", "mp"),), (1,)) == [(("dp",), [None, "sum"])]
    assert infer("mean", (L("dp", "mp"),), ((0, 1),)) == [((), ["avg", "avg"])]
    assert infer("mse_loss", (L("dp", "None"), L("dp", "None"))) == [((), ["avg", None])]


def test_axis_ops_reject_a_sharded_operating_dim():
    assert infer("softmax", (L("dp", "None"),), (-1,)) == [(("dp", "None"), [None, None])]
    for name, extra in [("softmax", (-1,)), ("cumsum", (1,)), ("topk", (2, -1))]:
        with pytest.raises(ValueError):
            infer(name, (L("dp", "mp"),), extra)
    with pytest.raises(ValueError):
        infer("rms_norm", (L("dp", "None", "mp"),), ((8,),))
    assert infer("layer_norm", (L("dp", "None", "None"),), ((8,),)) == [(("dp", "None", "None"), [None, None])]
    vals, idx = infer("topk", (L("dp", "None"),), (2, -1))
    assert vals == idx == (("dp", "None"), [None, None])


def test_shape_ops_rules():
    assert infer("transpose", (L("dp", "mp"),), (0, 1)) == [(("mp", "dp"), [None, None])]
    assert infer("permute", (L("dp", "None", "mp"),), ((2, 0, 1),)) == [(("mp", "dp", "None"), [None, None])]
    assert infer("unsqueeze", (L("dp", "mp"),), (1,)) == [(("dp", "None", "mp"), [None, None])]
    assert infer("embedding", (L("dp", "None"), L("None", "mp"))) == [(("dp", "None", "mp"), [None, None])]
    assert infer("scaled_dot_product_attention", (L("dp", "mp", "None", "None"),) * 3) == \
        [(("dp", "mp", "None", "None"), [None, None])]


# --------------------------------------------------------------------- battery --
def _battery_worker(rank, world):
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200 import distribute_tensor
    lay = Layout((2, 2), ("dp", "mp"), list(range(4)))
    g = torch.Generator().manual_seed(11)
    X = torch.randn(8, 12, generator=g)
    Y = torch.randn(8, 12, generator=g)
    W = torch.randn(16, 12, generator=g)
    W2 = torch.randn(12, 6, generator=g)
    B3 = torch.randn(4, 8, 12, generator=g)
    IDX = torch.randint(0, 16, (8, 5), generator=g)
    EMB = torch.randn(16, 12, generator=g)

    def d(t, *spec):
        return distribute_tensor(t.clone(), lay(*spec))

    def full(o):
        if isinstance(o, hp.DTensor):
            if o.layout.is_partial():
                o = o.reduce_partial()
            return o.full_tensor()
        return o

    cases = {
        "matmul_col": (lambda: torch.matmul(d(X, "dp", "None"), d(W2, "None", "mp")), lambda: X @ W2),
        "matmul_row_partial": (lambda: torch.matmul(d(X, "dp", "mp"), d(W2, "mp", "None")), lambda: X @ W2),
        "linear_col": (lambda: F.linear(d(X, "dp", "None"), d(W, "mp", "None")), lambda: F.linear(X, W)),
        "linear_row_partial": (lambda: F.linear(d(X, "dp", "mp"), d(W, "None", "mp")), lambda: F.linear(X, W)),
        "add": (lambda: d(X, "dp", "mp") + d(Y, "dp", "mp"), lambda: X + Y),
        "mul_broadcast_row": (lambda: d(X, "dp", "None") * d(Y[0], "None"), lambda: X * Y[0]),
        "scalar_ops": (lambda: (d(X, "dp", "mp") * 2.0 - 1.0) / 3.0, lambda: (X * 2.0 - 1.0) / 3.0),
        "unary": (lambda: torch.tanh(F.gelu(d(X, "dp", "mp"))).abs().sqrt(), lambda: torch.tanh(F.gelu(X)).abs().sqrt()),
        "where": (lambda: torch.where(d(X, "dp", "mp") > 0, d(X, "dp", "mp"), d(Y, "dp", "mp")),
                  lambda: torch.where(X > 0, X, Y)),
        "masked_fill": (lambda: d(X, "dp", "mp").masked_fill(d(Y, "dp", "mp") > 0, -1.0), lambda: X.masked_fill(Y > 0, -1.0)),
        "sum_sharded_dim": (lambda: d(X, "dp", "mp").sum(1), lambda: X.sum(1)),
        "mean_all": (lambda: d(X, "dp", "mp").mean(), lambda: X.mean()),
        "max_sharded_dim": (lambda: d(X, "dp", "mp").amax(1), lambda: X.amax(1)),
        "softmax": (lambda: torch.softmax(d(X, "dp", "None"), -1), lambda: torch.softmax(X, -1)),
        "log_softmax": (lambda: F.log_softmax(d(X, "dp", "None"), -1), lambda: F.log_softmax(X, -1)),
        "layer_norm": (lambda: F.layer_norm(d(B3, "dp", "mp", "None"), (12,)), lambda: F.layer_norm(B3, (12,))),
        "transpose": (lambda: d(X, "dp", "mp").transpose(0, 1), lambda: X.transpose(0, 1)),
        "permute": (lambda: d(B3, "dp", "None", "mp").permute(2, 0, 1), lambda: B3.permute(2, 0, 1)),
        "reshape_merge_unsharded": (lambda: d(B3, "dp", "None", "None").reshape(4, 96), lambda: B3.reshape(4, 96)),
        "view_split_dim": (lambda: d(X, "dp", "None").view(8, 3, 4), lambda: X.view(8, 3, 4)),
        "unsqueeze_squeeze": (lambda: d(X, "dp", "mp").unsqueeze(1).squeeze(1), lambda: X),
        "expand": (lambda: d(X[:, :1].contiguous(), "dp", "None").expand(8, 5), lambda: X[:, :1].expand(8, 5)),
        "cat_unsharded_dim": (lambda: torch.cat([d(X, "dp", "None"), d(Y, "dp", "None")], 1), lambda: torch.cat([X, Y], 1)),
        "chunk": (lambda: d(X, "dp", "None").chunk(3, 1)[1], lambda: X.chunk(3, 1)[1]),
        "slice": (lambda: d(X, "dp", "None")[:, 2:7], lambda: X[:, 2:7]),
        "topk_values": (lambda: d(X, "dp", "None").topk(3, -1).values, lambda: X.topk(3, -1).values),
        "sort_values": (lambda: d(X, "dp", "None").sort(-1).values, lambda: X.sort(-1).values),
        "cumsum": (lambda: d(X, "dp", "None").cumsum(1), lambda: X.cumsum(1)),
        "embedding": (lambda: F.embedding(d(IDX, "dp", "None"), d(EMB, "None", "mp")), lambda: F.embedding(IDX, EMB)),
        "index_select": (lambda: d(X, "dp", "None").index_select(1, torch.tensor([0, 3, 5])),
                         lambda: X.index_select(1, torch.tensor([0, 3, 5]))),
        "repeat_interleave": (lambda: d(X, "dp", "None").repeat_interleave(2, dim=1), lambda: X.repeat_interleave(2, dim=1)),
        "pad": (lambda: F.pad(d(X, "dp", "None"), (1, 2)), lambda: F.pad(X, (1, 2))),
        "mse_loss": (lambda: F.mse_loss(d(X, "dp", "None"), d(Y, "dp", "None")), lambda: F.mse_loss(X, Y)),
    }
    Q = torch.randn(2, 4, 8, 6, generator=g)
    K = torch.randn(2, 4, 8, 6, generator=g)
    V = torch.randn(2, 4, 8, 6, generator=g)
    cases["sdpa_dp_heads"] = (
        lambda: F.scaled_dot_product_attention(d(Q, "dp", "mp", "None", "None"), d(K, "dp", "mp", "None", "None"),
                                               d(V, "dp", "mp", "None", "None"), is_causal=True),
        lambda: F.scaled_dot_product_attention(Q, K, V, is_causal=True))
    cases["sdpa_q_seq_sharded_causal"] = (
        lambda: F.scaled_dot_product_attention(d(Q, "dp", "None", "mp", "None"), d(K, "dp", "None", "None", "None"),
                                               d(V, "dp", "None", "None", "None"), is_causal=True),
        lambda: F.scaled_dot_product_attention(Q, K, V, is_causal=True))
    failures = []
    for name, (dist_fn, ref_fn) in cases.items():
        try:
            got, ref = full(dist_fn()), ref_fn()
            if got.shape != ref.shape or not torch.allclose(got.float(), ref.float(), atol=1e-5, rtol=1e-5):
                failures.append(f"{name}: mismatch")
        except Exception as e:  # noqa: BLE001
            failures.append(f"{name}: {type(e).__name__}: {str(e)[:120]}")
    assert not failures, "\n".join(failures)
    # error paths: an op on a sharded operating dim and an unknown op raise
    with pytest.raises(ValueError):
        torch.softmax(d(X, "dp", "mp"), -1)
    with pytest.raises(NotImplementedError):
        F.scaled_dot_product_attention(d(Q, "dp", "None", "None", "None"), d(K, "dp", "None", "mp", "None"),
                                       d(V, "dp", "None", "mp", "None"))


def test_distributed_ops_match_single_device_on_four_ranks():
    run_distributed(_battery_worker, 4)


def _hook_worker(rank, world):
    import hyper_parallel_b200 as hp
    from torch import nn
    lay = hp.Layout((2,), ("dp",))
    lin = nn.Linear(4, 4, bias=False)
    lin.weight = nn.Parameter(hp.distribute_tensor(lin.weight.detach(), lay("None", "None")))
    seen = []
    lin.register_full_backward_pre_hook(lambda m, go: seen.append("pre"))
    lin.register_full_backward_hook(lambda m, gi, go: seen.append(("post", tuple(go[0].shape))))
    x = hp.DTensor.from_local(torch.randn(3, 4, requires_grad=True), lay("dp", "None"))
    y = lin(x)
    assert isinstance(y, hp.DTensor)
    y.to_local().sum().backward()
    assert seen == ["pre", ("post", (3, 4))], seen
    assert x.to_local().grad is not None and lin.weight.to_local().grad is not None


def test_module_full_backward_hooks_work_with_dtensor_arguments():
    run_distributed(_hook_worker, 2)
