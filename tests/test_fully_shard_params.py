"""fully_shard: parameter state machine, gradient reduction modes and state-dict forms.

Follows the cases of the reference's ``tests/torch/fully_shard/_test_hsdp_param.py`` (1-D and 2-D
meshes, sharded/unsharded transitions, custom shard placement, mixed precision, reduce-scatter and
all-reduce of gradients, accumulation) and ``_test_state_dict.py`` (sharded / full / host-offloaded /
frozen-ignoring state dicts; loading DTensors, local shards, global tensors and a single-device
checkpoint; round trips on 2 and 4 ranks), on gloo ranks."""
import pytest
import torch
from torch import nn

from dist_utils import run_distributed


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(8, 16)
        self.l2 = nn.Linear(16, 8, bias=False)
        self.register_buffer("scale", torch.full((1,), 2.0))

    def forward(self, x):
        return self.l2(torch.relu(self.l1(x))) * self.scale


def _fresh(seed=5):
    torch.manual_seed(seed)
    return Net()


def _param_worker(rank, world, case):
    import torch.distributed as dist
    from hyper_parallel_b200 import init_device_mesh
    from hyper_parallel_b200.core.dtensor import DTensor
    from hyper_parallel_b200.core.fully_shard import MixedPrecisionPolicy, fully_shard
    from hyper_parallel_b200.core.placement_types import Shard

    ref = _fresh()
    net = _fresh()
    if case == "mesh2d":
        mesh = init_device_mesh("cpu", (2, world // 2), mesh_dim_names=("rep", "shard"))
        n = world // 2
    else:
        mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("fsdp",))
        n = world
    kwargs = {}
    if case == "placement":
        kwargs["shard_placement_fn"] = lambda p: Shard(1) if p.dim() == 2 else Shard(0)
    if case == "mp":
        kwargs["mp_policy"] = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32)
    fully_shard(net, mesh=mesh, **kwargs)
    fp = net.l1.weight._fsdp_param

    # sharded state: DTensor parameters holding 1/n of the rows (or columns with the custom placement)
    assert isinstance(net.l1.weight, DTensor) and fp.is_sharded
    dim = 1 if case == "placement" else 0
    want = list(ref.l1.weight.shape)
    want[dim] //= n
    assert list(net.l1.weight.to_local().shape) == want
    sr = fp.mesh_info.shard_rank
    assert torch.equal(net.l1.weight.to_local(), ref.l1.weight.detach().chunk(n, dim=dim)[sr])

    # unshard -> plain tensors of the global shape; twice is a no-op; reshard drops the gathered copy
    for _ in range(2):
        net.unshard()
    assert not fp.is_sharded and not isinstance(net.l1.weight, DTensor)
    from hyper_parallel_b200.core.fully_shard.hsdp_utils import ShardedState
    assert fp.sharded_state is ShardedState.UNSHARDED
    assert tuple(net.l1.weight.shape) == tuple(ref.l1.weight.shape)
    if case == "mp":
        assert net.l1.weight.dtype == torch.bfloat16 and fp.sharded_local.dtype == torch.float32
        assert torch.allclose(net.l1.weight.float(), ref.l1.weight, atol=1e-2)
    else:
        assert torch.equal(net.l1.weight, ref.l1.weight)
    net.reshard()
    net.reshard()
    assert fp.is_sharded and fp.unsharded_param.numel() == 0 and isinstance(net.l1.weight, DTensor)
    assert fp.sharded_state is ShardedState.SHARDED

    # asynchronous unshard (the prefetch path): the handle's wait completes the transition
    h = net.unshard(async_op=True)
    assert h is not None
    h.wait()
    assert not fp.is_sharded
    net.reshard()

    # one backward: reduce-scatter over the shard axis (+ all-reduce over the replica axis on 2-D)
    g = torch.Generator().manual_seed(17)
    x = torch.randn(world * 2, 8, generator=g)
    ref(x).sum().backward()
    xs = x.chunk(world)[rank]
    net.set_reduce_op_type("sum")
    net(xs).float().sum().backward()
    tol = 5e-2 if case == "mp" else 1e-5
    got = net.l1.weight.grad
    assert isinstance(got, DTensor) and tuple(got.placements) == tuple(net.l1.weight.placements)
    got = got.to_local()                                  # the gradient is a DTensor laid out like the parameter
    assert got is not None and tuple(got.shape) == tuple(want)
    assert torch.allclose(got.float(), ref.l1.weight.grad.chunk(n, dim=dim)[sr], atol=tol, rtol=tol)
    # the buffer is untouched and not sharded
    assert not isinstance(net.scale, DTensor) and float(net.scale) == 2.0
    dist.barrier()


@pytest.mark.parametrize("case", ["mesh1d", "mesh2d", "placement", "mp"])
def test_param_state_machine_and_grad_reduction(case):
    run_distributed(_param_worker, 4, case)


def _accum_worker(rank, world):
    from hyper_parallel_b200 import init_device_mesh
    from hyper_parallel_b200.core.fully_shard import fully_shard

    ref = _fresh()
    net = _fresh()
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("rep", "shard"))
    fully_shard(net, mesh=mesh)
    net.set_reduce_op_type("sum")
    g = torch.Generator().manual_seed(23)
    xa, xb = torch.randn(world * 2, 8, generator=g), torch.randn(world * 2, 8, generator=g)
    ref(xa).sum().backward()
    ref(xb).sum().backward()
    fp = net.l1.weight._fsdp_param
    sr = fp.mesh_info.shard_rank

    # micro-batch 1 without synchronisation: the full-size gradient stays on the gathered parameter
    net.set_requires_gradient_sync(False)
    net(xa.chunk(world)[rank]).sum().backward()
    assert fp.sharded_local.grad is None
    # micro-batch 2 with synchronisation: both micro-batches are reduced together
    net.set_requires_gradient_sync(True)
    net(xb.chunk(world)[rank]).sum().backward()
    want = ref.l1.weight.grad.chunk(2, dim=0)[sr]
    assert torch.allclose(net.l1.weight.grad.to_local(), want, atol=1e-5)

    # without the replica all-reduce each replica keeps the sum over its own shard group
    net.zero_grads()
    assert net.l1.weight.grad is None
    net.set_requires_all_reduce(False)
    net(xa.chunk(world)[rank]).sum().backward()
    part = net.l1.weight.grad.to_local().clone()
    import torch.distributed as dist
    dist.all_reduce(part, group=fp.mesh_info.replicate_group)
    ref.zero_grad()
    ref(xa).sum().backward()
    assert torch.allclose(part, ref.l1.weight.grad.chunk(2, dim=0)[sr], atol=1e-5)


def test_grad_accumulation_and_replica_all_reduce_switch():
    run_distributed(_accum_worker, 4)


def _state_dict_worker(rank, world):
    import torch.distributed as dist
    from hyper_parallel_b200.core.dtensor import DTensor
    from hyper_parallel_b200.core.fully_shard import StateDictOptions, fully_shard, get_model_state_dict

    ref = _fresh()
    ref_sd = {k: v.detach().clone() for k, v in ref.state_dict().items()}
    net = _fresh(seed=99)                      # different weights: everything below must come from loads
    fully_shard(net.l1)
    fully_shard(net)
    x = torch.randn(4, 8, generator=torch.Generator().manual_seed(1))
    want = ref(x)

    def check(tag):
        with torch.no_grad():
            got = net(x)
        assert torch.allclose(got, want, atol=1e-5), tag
        assert all(isinstance(p, DTensor) for p in net.parameters()), tag

    # (a) a single-device checkpoint: plain tensors of the global shape
    res = net.load_state_dict(ref_sd)
    assert not res.missing_keys and not res.unexpected_keys
    check("global tensors")

    # (b) sharded state dict: DTensors aliasing the shards; loading them back into a fresh model
    sd = get_model_state_dict(net)
    assert set(sd) == set(ref_sd)
    assert isinstance(sd["l1.weight"], DTensor) and sd["l1.weight"].to_local().shape == (16 // world, 8)
    assert not isinstance(sd["scale"], DTensor)
    other = _fresh(seed=3)
    fully_shard(other.l1)
    fully_shard(other)
    other.load_state_dict(sd)
    with torch.no_grad():
        assert torch.allclose(other(x), want, atol=1e-5)

    # (c) local shards as plain tensors
    shards = {k: (v.to_local().clone() if isinstance(v, DTensor) else v.clone()) for k, v in sd.items()}
    net.load_state_dict({k: torch.zeros_like(v) for k, v in ref_sd.items()})
    assert float(sd["l1.weight"].to_local().abs().sum()) == 0.0      # the sharded state dict aliases the shards
    net.load_state_dict(shards)
    check("local shards")

    # (d) host-offloaded sharded state dict
    cpu_sd = get_model_state_dict(net, options=StateDictOptions(cpu_offload=True))
    assert all(v.device.type == "cpu" for v in cpu_sd.values())
    assert isinstance(cpu_sd["l2.weight"], DTensor)

    # (e) full tensors on every rank; with the host copy only on rank 0
    full = get_model_state_dict(net, options=StateDictOptions(full_state_dict=True))
    for k, v in ref_sd.items():
        assert not isinstance(full[k], DTensor) and torch.allclose(full[k], v), k
    full_cpu = get_model_state_dict(net, options=StateDictOptions(full_state_dict=True, cpu_offload=True))
    if rank == 0:
        assert set(full_cpu) == set(ref_sd) and torch.allclose(full_cpu["l1.bias"], ref_sd["l1.bias"])
    else:
        assert full_cpu == {}

    # (f) frozen parameters are left out on request; torch's own options class is accepted
    net.l1.bias.requires_grad_(False)
    from torch.distributed.checkpoint.state_dict import StateDictOptions as TorchOptions
    trainable = get_model_state_dict(net, options=TorchOptions(ignore_frozen_params=True))
    assert "l1.bias" not in trainable and "l1.weight" in trainable and "scale" in trainable
    with pytest.raises(ValueError):
        get_model_state_dict(net, options=StateDictOptions(broadcast_from_rank0=True))

    # (g) strictness
    with pytest.raises(RuntimeError):
        net.load_state_dict({"l1.weight": ref_sd["l1.weight"]})
    res = net.load_state_dict({"l1.weight": ref_sd["l1.weight"], "extra": torch.zeros(1)}, strict=False)
    assert "l2.weight" in res.missing_keys and res.unexpected_keys == ["extra"]
    with pytest.raises(RuntimeError):
        net.load_state_dict({**ref_sd, "l1.weight": torch.zeros(3, 3)})
    dist.barrier()


@pytest.mark.parametrize("world", [2, 4])
def test_state_dict_forms_and_round_trips(world):
    run_distributed(_state_dict_worker, world)
