"""Activation checkpoint / swap: identical losses and gradients with and without it (CPU)."""
import copy

import pytest
import torch
from torch import nn

from hyper_parallel_b200.core.activation_checkpoint import (AsyncSaveOnCpu, CheckpointPolicy, SwapManager,
                                                            SwapState, SwapTensor, checkpoint,
                                                            checkpoint_wrapper, swap_wrapper)


class Block(nn.Module):
    def __init__(self, d=32):
        super().__init__()
        self.a, self.b = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)

    def forward(self, x):
        return x + self.b(torch.nn.functional.gelu(self.a(x)))


def _run(model, x, steps=3):
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    losses = []
    for _ in range(steps):
        opt.zero_grad()
        loss = model(x).pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, [p.detach().clone() for p in model.parameters()]


def _models(wrap):
    torch.manual_seed(0)
    base = nn.Sequential(*[Block() for _ in range(4)])
    other = copy.deepcopy(base)
    wrapped = nn.Sequential(*[wrap(b) for b in other])
    return base, wrapped


def _same(a, b):
    la, pa = a
    lb, pb = b
    assert all(abs(x - y) < 1e-6 for x, y in zip(la, lb)), (la, lb)
    assert all(torch.allclose(x, y, atol=1e-6) for x, y in zip(pa, pb))


def test_full_recompute_matches():
    x = torch.randn(8, 32)
    base, wrapped = _models(lambda b: checkpoint_wrapper(b))
    _same(_run(base, x), _run(wrapped, x))
    assert set(wrapped.state_dict()) == set(base.state_dict())       # wrapper prefix is stripped


def test_selective_policy_save_matmul_swap_gelu():
    calls = {"mm": 0}

    def policy(op, *args, **kwargs):
        name = str(op)
        if "addmm" in name or "mm" in name:
            calls["mm"] += 1
            return CheckpointPolicy.MUST_SAVE
        if "gelu" in name:
            return CheckpointPolicy.MUST_SWAP
        return CheckpointPolicy.PREFER_RECOMPUTE
    x = torch.randn(8, 32)
    base, wrapped = _models(lambda b: checkpoint_wrapper(b, policy_fn=policy))
    _same(_run(base, x), _run(wrapped, x))
    assert calls["mm"] > 0


def test_swap_inputs_and_functional_checkpoint():
    torch.manual_seed(1)
    blk = Block()
    x = torch.randn(4, 32, requires_grad=True)
    y1 = blk(x).sum()
    (g1,) = torch.autograd.grad(y1, x)
    y2 = checkpoint(blk, x, swap_inputs=True).sum()
    (g2,) = torch.autograd.grad(y2, x)
    assert torch.allclose(g1, g2, atol=1e-6) and abs(y1.item() - y2.item()) < 1e-6


def test_swap_wrapper_and_manager_prefetch_chain():
    SwapManager().reset()
    x = torch.randn(8, 32)
    base, wrapped = _models(lambda b: swap_wrapper(b, policy_fn=lambda t: t.numel() >= 64))
    mgr = SwapManager()
    for a, b in zip(wrapped[:-1], wrapped[1:]):
        mgr.set_forward_prefetch_layer(a, b)
    _same(_run(base, x), _run(wrapped, x))
    assert set(wrapped.state_dict()) == set(base.state_dict())


def test_swap_tensor_state_machine():
    t = torch.arange(2048.0)
    st = SwapTensor(t)
    assert st.state == SwapState.DEVICE
    st.launch_offload()
    assert st.state == SwapState.D2H
    st.wait_offload()
    assert st.state == SwapState.HOST
    st.launch_load()
    assert st.state == SwapState.H2D
    assert torch.equal(st.wait_load(), t) and st.state == SwapState.DEVICE
    with AsyncSaveOnCpu(min_numel=1):
        a = torch.randn(64, 64, requires_grad=True)
        b = (a * a).sum()
    b.backward()
    assert torch.allclose(a.grad, 2 * a)


def test_swap_policy_may_answer_with_the_enum_or_a_bool():
    """A ``policy_fn`` written for the reference answers ``ActivationPolicy.SAVE`` / ``SWAP``; a plain
    bool keeps working.  Import paths of the reference's torch backend resolve too."""
    from hyper_parallel_b200.platform.torch.activation_checkpoint import ActivationPolicy, swap_wrapper
    from hyper_parallel_b200.platform.torch.fully_shard.utils import CPUOffloadPolicy, MixedPrecisionPolicy, OffloadPolicy
    from hyper_parallel_b200.platform.platform import get_torch_platform
    from hyper_parallel_b200.core.activation_checkpoint.activation_swap import _wants_swap
    assert _wants_swap(ActivationPolicy.SWAP) and not _wants_swap(ActivationPolicy.SAVE)
    assert _wants_swap(True) and not _wants_swap(False)
    assert issubclass(CPUOffloadPolicy, OffloadPolicy) and MixedPrecisionPolicy().cast_forward_inputs
    assert get_torch_platform().get_world_size() == 1
    seen = []

    def policy(t):
        seen.append(tuple(t.shape))
        return ActivationPolicy.SAVE                      # nothing is swapped, so CPU tensors are fine

    net = swap_wrapper(torch.nn.Sequential(torch.nn.Linear(64, 64), torch.nn.GELU(), torch.nn.Linear(64, 64)), policy)
    x = torch.randn(32, 64, requires_grad=True)
    net(x).sum().backward()
    assert seen and x.grad is not None


def test_swap_manager_manual_interface_by_group_name():
    """Collect tensors under a name, offload / reload the group by hand; on CPU the copies are no-ops but
    the state machine and the method names are those of the reference's manager."""
    from hyper_parallel_b200.core.activation_checkpoint import Storage, SwapManager, SwapTensor
    mgr = SwapManager()
    mgr.reset()
    a, b = torch.randn(64, 64), torch.randn(32)
    sa, sb = SwapTensor(a), SwapTensor(b)
    mgr.add_storage("layer0", Storage(sa))
    mgr.add_storage("layer0", sb)
    mgr.set_current_group_name("layer0")
    assert mgr.get_current_group_name() == "layer0"
    mgr.launch_offload("layer0")
    mgr.wait_offload("layer0")
    mgr.launch_load("layer0")
    mgr.wait_load("layer0")
    assert torch.equal(sa.get_val(), a) and torch.equal(sb.get(), b)
    sa.async_offload()
    sa.wait_offload()
    sa.async_load()
    assert torch.equal(sa.wait_load(), a)
    with pytest.raises(RuntimeError):
        mgr.launch_offload("no such group")
    mgr.reset()
    assert mgr.get_current_group_name() == ""


def test_checkpoint_wrapper_with_a_checkpoint_function_of_the_callers():
    import torch.utils.checkpoint as tuc
    calls = []

    def my_ckpt(fn, *args, use_reentrant=False, **kw):
        calls.append(use_reentrant)
        return tuc.checkpoint(fn, *args, use_reentrant=use_reentrant, **kw)

    torch.manual_seed(0)
    block = nn.Sequential(nn.Linear(8, 8), nn.GELU(), nn.Linear(8, 8))
    ref = copy.deepcopy(block)
    wrapped = checkpoint_wrapper(block, checkpoint_fn=my_ckpt, use_reentrant=False)
    x = torch.randn(4, 8, requires_grad=True)
    xr = x.detach().clone().requires_grad_(True)
    wrapped(x).sum().backward()
    ref(xr).sum().backward()
    assert calls == [False] and torch.allclose(x.grad, xr.grad)
    assert set(wrapped.state_dict()) == set(ref.state_dict())          # keys keep the inner names
