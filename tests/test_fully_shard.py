"""fully_shard: precision vs a single-process run (FSDP on 4 ranks, HSDP 2x2, mixed precision),
module methods, state-dict round trips."""
import copy

import pytest
import torch
from torch import nn

from dist_utils import run_distributed


class Net(nn.Module):
    def __init__(self):
        super().__init__()
        self.l1 = nn.Linear(16, 32)
        self.l2 = nn.Linear(32, 16)
        self.l3 = nn.Linear(16, 8, bias=False)

    def forward(self, x):
        return self.l3(torch.relu(self.l2(torch.relu(self.l1(x)))))


def _data(world):
    g = torch.Generator().manual_seed(3)
    return torch.randn(world * 4, 16, generator=g), torch.randn(world * 4, 8, generator=g)


def _reference(world, steps=3):
    torch.manual_seed(11)
    net = Net()
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    x, y = _data(world)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = (net(x) - y).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, {k: v.detach().clone() for k, v in net.state_dict().items()}


def _worker(rank, world, mode):
    import torch.distributed as dist
    from hyper_parallel_b200 import SkipDTensorDispatch, init_device_mesh
    from hyper_parallel_b200.core.fully_shard import (MixedPrecisionPolicy, StateDictOptions, fully_shard,
                                                      get_model_state_dict)
    ref_losses, ref_sd = _reference(world)
    torch.manual_seed(11)
    net = Net()
    mesh = init_device_mesh("cpu", (2, 2), mesh_dim_names=("rep", "shard")) if mode == "hsdp" else None
    mp = MixedPrecisionPolicy(param_dtype=torch.bfloat16, reduce_dtype=torch.float32) if mode == "mp" \
        else MixedPrecisionPolicy()
    for layer in (net.l1, net.l2):
        fully_shard(layer, mesh=mesh, mp_policy=mp)
    fully_shard(net, mesh=mesh, mp_policy=mp)
    net.l1.set_modules_to_forward_prefetch([net.l2])
    net.l2.set_modules_to_backward_prefetch([net.l1])
    n_shard = 2 if mode == "hsdp" else world
    assert net.l1.weight.to_local().shape == (32 // n_shard, 16)
    opt = torch.optim.SGD(net.parameters(), lr=0.1)
    x, y = _data(world)
    xs, ys = x.chunk(world)[rank], y.chunk(world)[rank]
    losses = []
    for _ in range(3):
        with SkipDTensorDispatch():
            opt.zero_grad()
        loss = (net(xs).float() - ys).pow(2).mean()
        loss.backward()
        with SkipDTensorDispatch():
            opt.step()
        l = loss.detach().clone()
        dist.all_reduce(l)
        losses.append(l.item() / world)
    tol = 5e-2 if mode == "mp" else 1e-5
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < tol * max(1.0, abs(b)), (mode, losses, ref_losses)
    full = get_model_state_dict(net, options=StateDictOptions(full_state_dict=True))
    for k, v in ref_sd.items():
        assert torch.allclose(full[k].float(), v, atol=tol), (mode, k)
    sharded = get_model_state_dict(net)
    assert hasattr(sharded["l1.weight"], "to_local")
    if mode == "fsdp":
        # state-dict round trip through global-shape tensors, and unshard()/reshard()
        net.load_state_dict({k: torch.zeros_like(v) for k, v in ref_sd.items()})
        assert float(net.l1.weight.to_local().abs().sum()) == 0.0
        net.load_state_dict(ref_sd)
        h = net.l1.unshard(async_op=True)
        h.wait()
        assert net.l1.weight.shape == (32, 16) and torch.allclose(net.l1.weight, ref_sd["l1.weight"])
        net.l1.reshard()
        assert net.l1.weight.to_local().shape == (32 // world, 16)
        with pytest.raises(ValueError):
            net.set_reduce_op_type("max")
        with pytest.raises(NotImplementedError):
            fully_shard(nn.Linear(16, 6))      # 6 rows over 4 ranks: uneven


@pytest.mark.parametrize("mode", ["fsdp", "hsdp", "mp"])
def test_fully_shard_matches_single_process(mode):
    run_distributed(_worker, 4, mode)
