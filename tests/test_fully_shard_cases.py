"""``fully_shard`` cases, one pytest id per case, all in ONE launch of 8 gloo ranks: the wrapping forms
(one layer, nested, a model with buffers, a mesh made with ``from_group``, no mesh), and precision
against a single-process run (full shard over 8, fp16 compute parameters, host-offloaded shards,
4 x 2 replicate x shard, gradient accumulation with and without synchronisation, ignored parameters,
a column placement).  Case list after the reference's ``tests/torch/fully_shard/_test_fully_shard.py:32-160``
and ``tests/torch/fully_shard/_test_fully_shard_precision.py:36-190``."""
import json
import os
import traceback

import pytest
import torch
from torch import nn

from dist_utils import run_distributed

WORLD = 8
CASES = {}


def case(fn):
    CASES[fn.__name__] = fn
    return fn


def _mesh(shape, names):
    import hyper_parallel_b200 as hp
    return hp.init_device_mesh("cpu", shape, mesh_dim_names=names)


class Dense(nn.Module):
    def __init__(self, hin, hout, bias=False):
        super().__init__()
        self.fc = nn.Linear(hin, hout, bias=bias)

    def forward(self, x):
        return torch.relu(self.fc(x))


class Stack(nn.Module):
    def __init__(self, hidden, layers):
        super().__init__()
        self.layers = nn.ModuleList(Dense(hidden, hidden) for _ in range(layers))
        self.head = nn.Linear(hidden, 8)

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return self.head(x)


class WithBuffers(nn.Module):
    def __init__(self, hidden):
        super().__init__()
        self.fc = nn.Linear(hidden, hidden)
        self.bn = nn.BatchNorm1d(hidden)
        self.out = nn.Linear(hidden, hidden)

    def forward(self, x):
        return self.out(self.bn(self.fc(x)))


class MatSum(nn.Module):
    """sum(x @ w): the reference's precision model (tests/torch/common_net.py, ``SimpleModel``)."""

    def __init__(self):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(8, 8))

    def forward(self, x):
        return torch.sum(torch.matmul(x, self.weight))


def _train(build, wrap, steps=2, batch=4, hidden=32, seed=5):
    """Train ``build()`` wrapped by ``wrap`` on this rank's rows and, unwrapped, on all rows in one
    process; the mean losses and the gathered parameters after ``steps`` SGD steps must agree."""
    import torch.distributed as dist
    from hyper_parallel_b200 import SkipDTensorDispatch
    from hyper_parallel_b200.core.fully_shard import StateDictOptions, get_model_state_dict
    world, rank = dist.get_world_size(), dist.get_rank()
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(world * batch, hidden, generator=g)
    torch.manual_seed(seed)
    ref = build()
    torch.manual_seed(seed)
    net = wrap(build())
    ropt = torch.optim.SGD(ref.parameters(), lr=0.05)
    opt = torch.optim.SGD(net.parameters(), lr=0.05)
    for _ in range(steps):
        rloss = ref(x).pow(2).mean()
        ropt.zero_grad()
        rloss.backward()
        ropt.step()
        loss = net(x.chunk(world)[rank]).float().pow(2).mean()
        with SkipDTensorDispatch():
            opt.zero_grad()
        loss.backward()
        with SkipDTensorDispatch():
            opt.step()
        l = loss.detach().clone()
        dist.all_reduce(l)
        assert abs(l.item() / world - rloss.item()) < 1e-4 * max(1.0, abs(rloss.item())), (l.item() / world, rloss.item())
    full = get_model_state_dict(net, options=StateDictOptions(full_state_dict=True))
    for k, v in ref.state_dict().items():
        if v.dtype.is_floating_point:
            assert torch.allclose(full[k].float(), v, atol=1e-4), k
    return net


def _local(g):
    """``.grad`` of a sharded parameter is a DTensor laid out like the parameter; of an ignored
    (plain) parameter a plain tensor."""
    return g.to_local() if hasattr(g, "to_local") else g


def _fp32_policy():
    from hyper_parallel_b200.core.fully_shard import MixedPrecisionPolicy
    return MixedPrecisionPolicy(param_dtype=torch.float32, reduce_dtype=torch.float32, output_dtype=torch.float32,
                                cast_forward_inputs=True)


@case
def one_layer_without_bias(rank):
    from hyper_parallel_b200 import DTensor
    from hyper_parallel_b200.core.fully_shard import fully_shard
    mesh = _mesh((8,), ("dp",))
    net = _train(lambda: Dense(32, 64), lambda m: fully_shard(m, mesh=mesh, reshard_after_forward=True,
                                                              mp_policy=_fp32_policy()))
    assert isinstance(net.fc.weight, DTensor) and net.fc.weight.to_local().shape == (8, 32)


@case
def nested_layers_then_root(rank):
    from hyper_parallel_b200.core.fully_shard import fully_shard
    mesh = _mesh((8,), ("dp",))

    def wrap(m):
        for l in m.layers:
            fully_shard(l, mesh=mesh, reshard_after_forward=True, mp_policy=_fp32_policy())
        return fully_shard(m, mesh=mesh, reshard_after_forward=True, mp_policy=_fp32_policy())
    net = _train(lambda: Stack(32, 2), wrap)
    # the root manages what the layers did not take
    assert [len(s.params) for s in (net.layers[0]._fsdp_state, net.layers[1]._fsdp_state, net._fsdp_state)] == [1, 1, 2]


@case
def model_with_buffers(rank):
    from hyper_parallel_b200 import DTensor
    from hyper_parallel_b200.core.fully_shard import fully_shard
    mesh = _mesh((8,), ("dp",))
    torch.manual_seed(1)
    net = fully_shard(WithBuffers(32), mesh=mesh, mp_policy=_fp32_policy())
    assert isinstance(net.bn.weight, DTensor)
    assert not isinstance(net.bn.running_mean, DTensor) and net.bn.running_mean.shape == (32,)
    before = net.bn.running_mean.clone()
    net(torch.rand(4, 32)).sum().backward()
    assert not torch.equal(before, net.bn.running_mean) and int(net.bn.num_batches_tracked) == 1
    assert net.fc.weight.grad is not None and _local(net.fc.weight.grad).shape == (4, 32)


@case
def mesh_made_from_a_group(rank):
    from hyper_parallel_b200 import DeviceMesh
    from hyper_parallel_b200.core.fully_shard import fully_shard
    group = _mesh((8,), ("dp",)).get_group()
    mesh = DeviceMesh.from_group(group, device_type="cpu", mesh_dim_names=["shard"])
    _train(lambda: Dense(32, 64), lambda m: fully_shard(m, mesh=mesh, mp_policy=_fp32_policy()))


@case
def no_mesh_means_all_ranks(rank):
    from hyper_parallel_b200.core.fully_shard import fully_shard
    net = _train(lambda: Dense(32, 64), lambda m: fully_shard(m, mesh=None, mp_policy=_fp32_policy()))
    assert net.fc.weight.to_local().shape == (8, 32) and net.fc.weight.device_mesh.mesh_shape == (8,)


def _matsum_reference(accumulate):
    torch.manual_seed(0)
    x = torch.rand(8, 8)
    ref = MatSum()
    opt = torch.optim.SGD(ref.parameters(), lr=0.01)
    for _ in range(2):
        for _ in range(4):
            loss = ref(x)
            loss.backward()
            grad = ref.weight.grad.clone()
            if not accumulate:
                opt.step()
                opt.zero_grad()
        if accumulate:
            opt.step()
            opt.zero_grad()
    return x, loss.detach(), grad


def _matsum_fully_shard(mesh, accumulate=False, sync_last_only=False, tol=1e-3, **kw):
    """The reference's precision recipe: every rank feeds the same 8 x 8 input, gradients are
    summed over the ranks, the backward seed is 1 / ranks; two epochs of four steps."""
    import torch.distributed as dist
    from hyper_parallel_b200 import DTensor, SkipDTensorDispatch
    from hyper_parallel_b200.core.fully_shard import fully_shard
    rank = dist.get_rank()
    x, rloss, rgrad = _matsum_reference(accumulate)
    net = fully_shard(MatSum(), mesh=mesh, reshard_after_forward=True, **kw)
    net.set_reduce_op_type("sum")
    opt = torch.optim.SGD(net.parameters(), lr=0.01)
    seed = torch.tensor(1.0 / len(list(mesh.rank_list)))
    grad = None
    with SkipDTensorDispatch():
        for _ in range(2):
            for i in range(4):
                if sync_last_only:
                    net.set_requires_gradient_sync(i == 3)
                loss = net(x)
                loss.backward(seed.to(loss.dtype))
                if net.weight.grad is not None:
                    assert isinstance(net.weight.grad, DTensor), type(net.weight.grad)
                    grad = net.weight.grad.to_local().clone()
                if not accumulate:
                    opt.step()
                    opt.zero_grad()
            if accumulate:
                opt.step()
                opt.zero_grad()
    assert torch.allclose(loss.detach().float(), rloss, rtol=tol, atol=tol), (loss, rloss)
    n = mesh.mesh_shape[-1]
    rows = 8 // n
    lo = rank % n * rows
    assert grad.shape == (rows, 8) and torch.allclose(grad.float(), rgrad[lo:lo + rows], rtol=tol, atol=tol)
    return net


@case
def precision_full_shard_over_8(rank):
    _matsum_fully_shard(_mesh((8,), ("dp",)))


@case
def precision_fp16_compute_parameters(rank):
    from hyper_parallel_b200.core.fully_shard import MixedPrecisionPolicy
    net = _matsum_fully_shard(_mesh((8,), ("dp",)), tol=2e-2,
                              mp_policy=MixedPrecisionPolicy(param_dtype=torch.float16, reduce_dtype=torch.float32,
                                                             output_dtype=torch.float32, cast_forward_inputs=True))
    assert net.weight.to_local().dtype == torch.float32             # the shard stays in full precision
    net.unshard()
    assert net.weight.dtype == torch.float16
    net.reshard()


@case
def precision_host_offloaded_shards(rank):
    from hyper_parallel_b200.core.fully_shard import CPUOffloadPolicy
    net = _matsum_fully_shard(_mesh((8,), ("dp",)), offload_policy=CPUOffloadPolicy(pin_memory=False))
    assert net.weight.to_local().device.type == "cpu"


@case
def precision_replicate_4_x_shard_2(rank):
    _matsum_fully_shard(_mesh((4, 2), ("dp", "op")))


@case
def precision_accumulated_gradients(rank):
    _matsum_fully_shard(_mesh((8,), ("dp",)), accumulate=True)


@case
def precision_accumulation_with_one_synchronisation(rank):
    _matsum_fully_shard(_mesh((4, 2), ("dp", "op")), accumulate=True, sync_last_only=True)


@case
def ignored_parameters_stay_plain(rank):
    from hyper_parallel_b200 import DTensor
    from hyper_parallel_b200.core.fully_shard import fully_shard
    torch.manual_seed(2)
    net = Stack(16, 1)
    fully_shard(net, mesh=_mesh((8,), ("dp",)), ignored_params=[net.head.weight, net.head.bias])
    assert not isinstance(net.head.weight, DTensor) and net.head.weight.shape == (8, 16)
    assert isinstance(net.layers[0].fc.weight, DTensor)
    net(torch.rand(2, 16)).sum().backward()
    assert net.head.weight.grad is not None and net.head.weight.grad.shape == (8, 16)   # local, not reduced


@case
def column_placement_function(rank):
    from hyper_parallel_b200 import Shard
    from hyper_parallel_b200.core.fully_shard import fully_shard
    mesh = _mesh((8,), ("dp",))
    net = _train(lambda: Dense(32, 64), lambda m: fully_shard(m, mesh=mesh, shard_placement_fn=lambda p: Shard(1)))
    assert net.fc.weight.to_local().shape == (64, 4)


def _worker(rank, world, out_dir):
    results = {}
    for name, fn in CASES.items():
        try:
            fn(rank)
            results[name] = ""
        except Exception:  # noqa: BLE001  (recorded per case, reported by the parametrised test)
            results[name] = traceback.format_exc()
    with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
        json.dump(results, f)


@pytest.fixture(scope="module")
def results(tmp_path_factory):
    out = tmp_path_factory.mktemp("fully_shard_cases")
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
