"""custom_shard, parallelize_value_and_grad, custom distributed-op registration through the
environment, DeviceMesh.from_group / flatten, and tied parameters across pipeline stages."""
import os

import pytest
import torch
import torch.nn.functional as F
from torch import nn

from dist_utils import run_distributed

HERE = os.path.dirname(os.path.abspath(__file__))


def _custom_shard_worker(rank, world):
    import hyper_parallel_b200 as hp
    lay = hp.Layout((2, 2), ("dp", "mp"))
    g = torch.Generator().manual_seed(2)
    X = torch.randn(8, 6, generator=g)
    x = hp.distribute_tensor(X.clone(), lay("dp", "mp"))

    def local_fn(t, k):                      # runs on the local shard
        assert not isinstance(t, hp.DTensor) and t.shape == (4, 6)
        return t * k, int(t.shape[0])

    fn = hp.custom_shard(local_fn, lay.mesh, out_placements=(lay("dp", "None"), None),
                         in_placements=(lay("dp", "None"), None))
    y, n = fn(x, 3.0)                        # x is redistributed from ("dp","mp") to ("dp","None")
    assert isinstance(y, hp.DTensor) and n == 4
    assert torch.allclose(y.full_tensor(), X * 3.0)
    # parallelize_value_and_grad: a loss replicated on every rank is seeded with 1 / repeat_num
    W = torch.randn(6, 6, generator=g)
    w = hp.distribute_tensor(W.clone(), lay("None", "None"))
    w.requires_grad_(True)
    xr = hp.distribute_tensor(X.clone(), lay("None", "None"))

    def loss_fn():
        return (torch.matmul(xr, w) ** 2).mean()

    loss, grads = hp.parallelize_value_and_grad(loss_fn, [w])()
    Wr = W.clone().requires_grad_(True)
    ((X @ Wr) ** 2).mean().backward()
    total = grads[0].clone()
    torch.distributed.all_reduce(total)      # what a data-parallel reduction would produce
    assert torch.allclose(total, Wr.grad, atol=1e-5)


def test_custom_shard_and_value_and_grad():
    run_distributed(_custom_shard_worker, 4)


def _custom_op_worker(rank, world):
    os.environ["HYPER_PARALLEL_OPS_YAML_DIR"] = os.path.join(HERE, "custom_ops")
    os.environ["HYPER_PARALLEL_OPS_PYTHON_PATH"] = os.path.join(HERE, "custom_ops")
    import importlib
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200.core.shard import _op_dispatch
    importlib.reload(_op_dispatch)           # picks the environment up, as a fresh process would
    from hyper_parallel_b200.core.shard.ops.parallel_ops import get_distributed_op
    rule = get_distributed_op("stack_rows")
    assert rule is not None and type(rule).__name__ == "StackDistributedOp"
    lay = hp.Layout((2,), ("dp",))
    out = rule.infer_layout((lay("dp", "None"), lay("dp", "None")), ())
    assert tuple(out.alias_tensor_map) == ("None", "dp", "None")
    # the built-in catalogue is still there
    assert get_distributed_op("matmul") is not None

    # rules written for the reference's "Reshape" and "Slice" calling conventions run unchanged:
    # [shape, global shape] -> (layout, local shape); [begin, end, global shape] -> (layout, begin, end)
    def fold_rows(x, shape):
        return x.reshape(shape)

    def window(x, begin, end):
        return x[tuple(slice(b, e) for b, e in zip(begin, end))]

    full = torch.arange(4 * 6 * 2.0).reshape(4, 6, 2)
    d = hp.distribute_tensor(full, lay("dp", "None", "None"))
    disp = _op_dispatch._OP_DISPATCHER
    for _ in range(2):                                       # the second call comes from the plan cache
        y = disp.dispatch(fold_rows, (d, (4, 12)), {})
        assert isinstance(y, hp.DTensor) and tuple(y.shape) == (4, 12) and y.to_local().shape == (2, 12)
        assert torch.equal(y.full_tensor(), full.reshape(4, 12))
        z = disp.dispatch(window, (d, (0, 1, 0), (4, 5, 1)), {})
        assert tuple(z.shape) == (4, 4, 1) and z.to_local().shape == (2, 4, 1)
        assert torch.equal(z.full_tensor(), full[:, 1:5, :1])
    with pytest.raises(ValueError):
        disp.dispatch(window, (d, (1, 0, 0), (4, 6, 2)), {})      # a sharded dim cut short
    with pytest.raises(TypeError):
        disp.dispatch(fold_rows, (d,), {"shape": (4, 12)})        # the form is positional
    # entries that name a stock rule by the reference's file / class names resolve to this package's rules
    assert type(get_distributed_op("my_topk")).__name__ == "TopKDistributedOp"
    assert type(get_distributed_op("my_split_view")).__name__ == "SplitDistributedOp"
    # the package's own reshape / slice keep serving every spelling of those ops
    assert tuple(d.view(4, 12).shape) == (4, 12) and tuple(d.flatten(1).to_local().shape) == (2, 12)
    assert tuple(d[:, 2:4].shape) == (4, 2, 2) and tuple(d.narrow(1, 0, 3).to_local().shape) == (2, 3, 2)


def test_custom_distributed_op_registration_through_the_environment():
    run_distributed(_custom_op_worker, 2)


def _mesh_worker(rank, world):
    import torch.distributed as dist
    import hyper_parallel_b200 as hp
    mesh = hp.init_device_mesh("cpu", (2, 2), mesh_dim_names=("dp", "tp"))
    flat = mesh.flatten("all")
    assert flat.size() == 4 and flat.ndim == 1 and flat.get_local_rank() == rank
    assert mesh.flatten("all") is flat                                   # cached on the root
    t = torch.ones(1) * rank
    dist.all_reduce(t, group=flat.get_group())
    assert t.item() == 6
    sub = mesh["tp"]
    assert sub.size() == 2 and set(sub.rank_list) == {rank - rank % 2, rank - rank % 2 + 1}
    dm = hp.DeviceMesh.from_group(sub.get_group(), "cpu", mesh_dim_names=("tp",))
    assert dm.size() == 2 and dm.get_local_rank() == rank % 2
    t = torch.ones(1)
    dist.all_reduce(t, group=dm.get_group())
    assert t.item() == 2
    assert isinstance(mesh.to_hash(), int) and tuple(mesh.get_coordinate()) == (rank // 2, rank % 2)


def test_device_mesh_flatten_from_group_submesh():
    run_distributed(_mesh_worker, 4)


class _First(nn.Module):
    def __init__(self, emb):
        super().__init__()
        self.emb = emb
        self.lin = nn.Linear(8, 8)

    def forward(self, tok):
        return torch.tanh(self.lin(F.embedding(tok, self.emb)))


class _Last(nn.Module):
    def __init__(self, emb):
        super().__init__()
        self.emb = emb                       # tied: output projection uses the embedding matrix

    def forward(self, h):
        return (h @ self.emb.t()).pow(2).mean() / 2


def _tied_worker(rank, world):
    from hyper_parallel_b200 import PipelineStage, SharedParameterInfo
    from hyper_parallel_b200.core.pipeline_parallel import Schedule1F1B
    torch.manual_seed(3)
    emb_ref = nn.Parameter(torch.randn(12, 8))
    first_ref = _First(emb_ref)
    last_ref = _Last(emb_ref)
    tok = torch.randint(0, 12, (4, 5), generator=torch.Generator().manual_seed(4))
    for tm in tok.chunk(2):
        last_ref(first_ref(tm)).backward()
    # two stages, each with its own copy of the embedding; stage 1's copy starts different and is
    # overwritten by the broadcast from stage 0; gradients are summed after the schedule
    torch.manual_seed(3)
    emb0 = nn.Parameter(torch.randn(12, 8))
    first = _First(emb0)
    if rank == 0:
        mod, emb = first, emb0
    else:
        emb = nn.Parameter(torch.zeros(12, 8))
        mod = _Last(emb)
    stage = PipelineStage(mod, rank, 2, device="cpu", shared_parameters=[SharedParameterInfo(emb, [0, 1])])
    sched = Schedule1F1B(stage, 2)
    sched.run(tok) if rank == 0 else sched.run()
    assert torch.allclose(emb.detach(), emb_ref.detach())               # broadcast at init
    assert torch.allclose(emb.grad, emb_ref.grad, atol=1e-6)            # all-reduced after the schedule


def test_pipeline_tied_parameters_are_broadcast_and_their_grads_summed():
    run_distributed(_tied_worker, 2)


def test_reference_compat_runner_rewrites_and_runs_a_reference_style_test(tmp_path):
    """A test file in the style of the reference's torch tests (NPU devices, HCCL, ``init_dist`` from a
    helper module) runs against this package on two CPU ranks; a failing function is reported."""
    from hyper_parallel_b200.utils import reference_compat as rc
    root = tmp_path / "checkout"
    (root / "tests" / "torch" / "demo").mkdir(parents=True)
    (root / "tests" / "torch" / "demo" / "demo_case.py").write_text(
        "import torch\n"
        "import torch_npu\n"
        "import torch.distributed as dist\n"
        "from hyper_parallel import DTensor, init_device_mesh\n"
        "from hyper_parallel.core.placement_types import Shard, Replicate\n"
        "from tests.torch.utils import init_dist\n\n\n"
        "def test_shard_round_trip():\n"
        "    init_dist()\n"
        "    mesh = init_device_mesh(device_type=\"npu\", mesh_shape=(2,), mesh_dim_names=(\"dp\",))\n"
        "    x = DTensor.from_local(torch.ones(2, 4).npu() * dist.get_rank(), mesh, (Shard(0),))\n"
        "    full = x.redistribute(mesh, (Replicate(),)).to_local()\n"
        "    assert full.shape == (4, 4) and full[2:].eq(1).all() and dist.get_backend() == \"hccl\"\n\n\n"
        "def test_that_fails():\n"
        "    init_dist()\n"
        "    assert False, 'as intended'\n")
    text = rc.rewrite((root / "tests/torch/demo/demo_case.py").read_text())
    assert "hyper_parallel_b200.core.placement_types" in text and "torch_npu" not in text
    assert '"cpu"' in text and ".cpu()" in text and '"gloo"' in text and "npu" not in text
    assert rc.rewrite("import hyper_parallel_b200") == "import hyper_parallel_b200"          # already migrated text is kept
    fa = rc.rewrite("import torch_npu\nout = torch_npu.npu_fusion_attention(q, k, v, 8)\n")
    assert "from hyper_parallel_b200.ops import flash_attention_score as _hpb_fa" in fa
    assert "_hpb_fa.npu_fusion_attention(q, k, v, 8)" in fa and "torch_npu" not in fa
    assert rc.list_test_functions(str(root / "tests/torch/demo/demo_case.py")) == ["test_shard_round_trip", "test_that_fails"]
    out = tmp_path / "gen"
    path = rc.prepare(str(root), "tests/torch/demo/demo_case.py", str(out))
    ok, tb = rc.run_function(str(out), path, "test_shard_round_trip", 2, timeout=120.0)
    assert ok and tb is None
    ok, tb = rc.run_function(str(out), path, "test_that_fails", 2, timeout=120.0)
    assert not ok and "as intended" in tb


def test_platform_facade_offers_the_reference_method_names():
    """Code written against ``get_platform()`` of the reference finds the same helpers here."""
    import hyper_parallel_b200.platform.torch.fully_shard.utils  # noqa: F401  (binds ``platform.torch``: must not
    from hyper_parallel_b200.platform import get_platform        # hide the torch module from the facade)
    p = get_platform()
    assert p.ones((2,)).tolist() == [1.0, 1.0] and p.full((1,), 3.0).item() == 3.0 and p.empty((2, 3)).shape == (2, 3)
    assert p.tensor_type_cast(torch.ones(2), "float16").dtype == torch.float16
    assert p.cast_fp_tensor(torch.bfloat16, torch.ones(2)).dtype == torch.bfloat16
    assert p.cast_fp_tensor(torch.bfloat16, torch.ones(2, dtype=torch.int32)).dtype == torch.int32
    assert p.chunk(torch.arange(8), 0, 4, 1).tolist() == [2, 3]
    assert p.tensor_to_numpy(torch.arange(3)).tolist() == [0, 1, 2]
    assert p.apply_to_tensors(lambda t: t + 1, {"a": [torch.zeros(1), 3]}) == {"a": [torch.ones(1), 3]}
    m = torch.nn.Sequential(torch.nn.Linear(2, 2))
    found = p.search_parameter_by_name(m, "0.weight")
    assert found[0] is m[0] and found[1] == "weight" and p.search_parameter_by_name(m, "0.nope") is None
    new = torch.nn.Parameter(torch.zeros(2, 2))
    assert p.update_parameter_by_name(m, found, new) and m[0].weight is new
    assert dict(p.parameters_dict(m)).keys() == {"0.weight", "0.bias"} and len(list(p.get_cells_and_names(m))) == 2
    assert p.get_param_type_size(new) == 4 and tuple(p.get_param_local_shape(new)) == (2, 2)
    assert p.device_type() == "cuda" and p.get_device_handle() is torch.cuda
    assert p.checkpoint is torch.utils.checkpoint.checkpoint
    state = p.get_rng_state()
    p.manual_seed(3)
    p.set_rng_state(state)
    assert torch.equal(p.get_rng_state(), state)
    mb = p.micro_batch(2)
    assert mb is not None
    p.wait_grad_handle()                                     # nothing in flight: returns
    with pytest.raises(ValueError):
        p.tensor_type_cast(torch.ones(1), "not_a_dtype")


def test_value_and_grad_with_weights_and_sensitivities():
    """The reference's arguments: ``(fn, weights, sens)``; several outputs with and without ``sens``."""
    from hyper_parallel_b200 import parallelize_value_and_grad
    w = torch.nn.Parameter(torch.tensor([1.0, 2.0]))
    x = torch.tensor([3.0, 4.0])

    def two(x):
        return (w * x).sum(), (w * w * x).sum()
    (o1, o2), g = parallelize_value_and_grad(two, [w])(x)
    assert (o1.item(), o2.item()) == (11.0, 19.0) and g[0].tolist() == [3.0, 4.0]      # the first output only
    _, g = parallelize_value_and_grad(two, w, sens=[1.0, 0.5])(x)
    assert g[0].tolist() == [6.0, 12.0]
    with pytest.raises(ValueError):
        parallelize_value_and_grad(two, [w], sens=[1.0])(x)
    out, none = parallelize_value_and_grad(lambda x: (w * x).sum())(x)                  # no weights: into .grad
    assert none is None and w.grad.tolist() == [3.0, 4.0]


def _readme_worker(rank, world):
    """The tensor-parallel example of the reference's README, line for line (torch meta device in place of
    MindSpore's ``no_init_parameters``): dict plan for ``shard``, ``hsdp`` on top, ``model = init_parameters(model)``,
    ``DTensor.from_local(local, layout)``."""
    from hyper_parallel_b200 import DTensor, Layout, hsdp, init_parameters, shard
    layout = Layout((2, 2), ("dp", "mp"))
    x_layout, w_layout, out_layout = layout("dp", "mp"), layout("mp", "None"), layout()

    class SimpleModel(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.weight = torch.nn.Parameter(torch.ones(8, 4))

        def reset_parameters(self):
            torch.nn.init.ones_(self.weight)

        def forward(self, x):
            return torch.sum(torch.matmul(x, self.weight))

    with torch.device("meta"):
        model = SimpleModel()
    plan = {"forward": {"input": (x_layout,), "output": (out_layout,)}, "parameter": {"weight": w_layout}}
    model = shard(model, plan)
    model = hsdp(model, shard_size=2, threshold=0)
    model = init_parameters(model)
    assert model is not None
    out = model(DTensor.from_local(torch.ones(4, 4), x_layout))
    assert isinstance(out, DTensor) and not out.layout.is_partial()
    assert out.to_local().item() == 256.0                      # 8 x 8 ones times 8 x 4 ones, summed


def test_reference_readme_tensor_parallel_example():
    run_distributed(_readme_worker, 4)
