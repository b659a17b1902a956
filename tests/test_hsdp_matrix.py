"""HSDP matrix on 4 gloo ranks against a single-process SGD run (the reference's
tests/torch/hsdp/hsdp.py cases): pure DP, levels 1-3, fully / partially sharded, with and without
gradient accumulation, synchronous / asynchronous hooks, bucket fusion, prefetch."""
import pytest
import torch
import torch.nn.functional as F
from torch import nn

from dist_utils import run_distributed

HID, LAYERS, BATCH, STEPS, LR = 32, 3, 16, 3, 0.05


def _net():
    torch.manual_seed(5)
    return nn.Sequential(*[nn.Sequential(nn.Linear(HID, HID), nn.Tanh()) for _ in range(LAYERS)])


def _data():
    g = torch.Generator().manual_seed(1)
    return torch.randn(STEPS, BATCH, HID, generator=g), torch.randn(STEPS, BATCH, HID, generator=g)


def _reference(acc):
    net = _net()
    xs, ys = _data()
    opt = torch.optim.SGD(net.parameters(), lr=LR)
    losses = []
    for s in range(STEPS):
        opt.zero_grad()
        tot = 0.0
        for xm, ym in zip(xs[s].chunk(acc), ys[s].chunk(acc)):
            loss = F.mse_loss(net(xm), ym) / acc
            loss.backward()
            tot += loss.item()
        opt.step()
        losses.append(tot)
    return losses, [p.detach().clone() for p in net.parameters()]


def _worker(rank, world, level, shard_size, acc, mode):
    import torch.distributed as dist
    import hyper_parallel_b200 as hp
    ref_losses, ref_params = _reference(acc)
    net = _net()
    # gradients are summed over the ranks (as in the reference); grad_scale turns the sum into the mean
    kw = dict(shard_size=shard_size, threshold=0, optimizer_level=level, enable_grad_accumulation=acc > 1,
              grad_scale=1.0 / world,
              comm_async=mode in ("async", "fusion_async"), comm_fusion=mode in ("fusion", "fusion_async"))
    if mode == "per_layer_prefetch":
        for layer in net:
            hp.hsdp(layer, **kw)
        hp.hsdp(net, **kw)
        for i, layer in enumerate(net):
            if i + 1 < LAYERS:
                layer.set_forward_prefetch_cells([net[i + 1]])
            if i > 0:
                layer.set_backward_prefetch_cells([net[i - 1]])
    else:
        hp.hsdp(net, **kw)
    xs, ys = _data()
    opt = torch.optim.SGD(net.parameters(), lr=LR)
    losses = []
    for s in range(STEPS):
        net.zero_grads()
        x, y = xs[s].chunk(world)[rank], ys[s].chunk(world)[rank]
        tot = torch.zeros(())
        chunks = list(zip(x.chunk(acc), y.chunk(acc)))
        for i, (xm, ym) in enumerate(chunks):
            net.set_requires_grad_sync(i == len(chunks) - 1)
            # every rank holds 1/world of the batch: the global mean is the mean of the rank means
            loss = F.mse_loss(net(xm), ym) / acc
            loss.backward()
            tot += loss.detach()
        hp.hsdp_sync_stream()
        opt.step()
        dist.all_reduce(tot)
        losses.append((tot / world).item())
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-5, (level, shard_size, acc, mode, losses, ref_losses)
    # parameters: gather the shards over the shard group and compare
    for p, ref in zip(net.parameters(), ref_params):
        hpar = getattr(p, "_hsdp_param", None)
        local = p.detach().contiguous()
        if hpar is not None and hpar.shard_size > 1:
            grp = hpar.sharded_group_info.group
            parts = [torch.empty_like(local) for _ in range(hpar.shard_size)]
            dist.all_gather(parts, local, group=grp)
            local = torch.cat(parts, 0)
        assert local.shape == ref.shape and torch.allclose(local, ref, atol=1e-5), (level, shard_size, acc, mode)


CASES = [("level1", 1, 1, "sync"),                       # pure data parallel
         ("level1", 4, 1, "sync"), ("level2", 4, 1, "sync"), ("level3", 4, 1, "sync"),      # fully sharded
         ("level1", 2, 1, "sync"), ("level2", 2, 1, "sync"), ("level3", 2, 1, "sync"),      # shard 2 x replicate 2
         ("level1", 4, 2, "sync"), ("level2", 2, 2, "sync"), ("level3", 4, 2, "sync"),      # gradient accumulation
         ("level2", 4, 1, "async"), ("level3", 2, 1, "async"),
         ("level2", 4, 1, "fusion"), ("level3", 2, 2, "fusion_async"),
         ("level3", 4, 1, "per_layer_prefetch")]


@pytest.mark.parametrize("level,shard_size,acc,mode", CASES)
def test_hsdp_matches_single_process(level, shard_size, acc, mode):
    run_distributed(_worker, 4, level, shard_size, acc, mode)


class _Branchy(nn.Module):
    """A module one of whose parameters gets no gradient (its branch is not on the loss path)."""

    def __init__(self):
        super().__init__()
        torch.manual_seed(7)
        self.used = nn.Linear(HID, HID)
        self.unused = nn.Linear(HID, HID)

    def forward(self, x):
        return torch.tanh(self.used(x))


def _unused_worker(rank, world, level):
    import torch.distributed as dist
    import hyper_parallel_b200 as hp
    ref = _Branchy()
    net = _Branchy()
    hp.hsdp(net, shard_size=world, threshold=0, optimizer_level=level, grad_scale=1.0 / world, comm_fusion=True,
            bucket_size=-1)
    xs, ys = _data()
    opt = torch.optim.SGD(net.parameters(), lr=LR)
    ropt = torch.optim.SGD(ref.parameters(), lr=LR)
    for s in range(STEPS):
        ropt.zero_grad()
        F.mse_loss(ref(xs[s]), ys[s]).backward()
        ropt.step()
        net.zero_grads()
        x, y = xs[s].chunk(world)[rank], ys[s].chunk(world)[rank]
        F.mse_loss(net(x), y).backward()
        hp.hsdp_sync_stream()
        opt.step()
    # the bucket was reduced although `unused` never fired its hook: `used` trained like the reference
    # and nothing stale was left behind for the next step
    state = net.hsdp_scheduler.hsdp_state
    assert all(not b.ready for b in state.grad_buffers)
    w = net.used.weight.detach()
    full = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(full, w.contiguous())
    got = torch.cat(full, 0) if w.shape != ref.used.weight.shape else w
    assert torch.allclose(got, ref.used.weight.detach(), atol=1e-5), (got - ref.used.weight).abs().max()
    assert torch.allclose(net.unused.weight.detach().new_tensor(0.0), torch.tensor(0.0))


@pytest.mark.parametrize("level", ["level1", "level2", "level3"])
def test_bucket_with_a_parameter_that_gets_no_gradient(level):
    run_distributed(_unused_worker, 2, level)


def _acc_visible_worker(rank, world, level, shard_size):
    """Between micro-steps ``param.grad`` shows the running accumulator; the synchronising micro-step
    replaces it by the reduced gradient; the forward in between never lets autograd add into it."""
    import hyper_parallel_b200 as hp
    torch.manual_seed(3)
    net = nn.Linear(8, 8, bias=False)
    ref = nn.Linear(8, 8, bias=False)
    ref.load_state_dict(net.state_dict())
    hp.hsdp(net, shard_size=shard_size, threshold=0, optimizer_level=level, enable_grad_accumulation=True)
    g = torch.Generator().manual_seed(9)
    xs = [torch.randn(4, 8, generator=g) for _ in range(3)]
    rows = 8 // shard_size
    lo = (rank % shard_size) * rows
    total = torch.zeros(8, 8)
    for i, x in enumerate(xs):
        net.set_requires_grad_sync(i == 2)
        net(x).sum().backward()
        ref.zero_grad()
        ref(x).sum().backward()
        total += ref.weight.grad
        got = net.weight.grad
        assert got is not None, (level, i)
        if i < 2:                                   # unreduced, accumulated so far (this rank's rows)
            want = total[lo:lo + rows] if got.shape[0] == rows else total
            if level == "level1" or shard_size == 1:
                assert torch.allclose(got, want, atol=1e-5), (level, i)
        else:                                       # every rank fed the same data: the sum is world x
            assert torch.allclose(got, world * total[lo:lo + rows], atol=1e-4), (level, i)
    net.zero_grads()
    assert net.weight.grad is None


@pytest.mark.parametrize("level,shard_size", [("level1", 2), ("level2", 2), ("level3", 2), ("level1", 1)])
def test_accumulator_is_visible_between_micro_steps(level, shard_size):
    run_distributed(_acc_visible_worker, 2, level, shard_size)
