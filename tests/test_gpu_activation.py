"""Activation checkpoint / swap on the GPU: identical losses over three steps and the peak-memory
ordering the reference's ``tests/torch/activation_checkpoint/test_ac.py`` and ``test_act_swap.py``
assert on a 16-layer, 2048-wide stack: nothing saved elsewhere > selective save > full recompute,
and nothing > swap with a size policy > swap of everything."""
import copy

import pytest
import torch
from torch import nn

from hyper_parallel_b200.core.activation_checkpoint import (CheckpointPolicy, SwapManager, checkpoint_wrapper,
                                                            swap_wrapper)

pytestmark = pytest.mark.gpu

D, LAYERS, TOKENS = 2048, 16, 16384


class Block(nn.Module):
    def __init__(self):
        super().__init__()
        self.norm = nn.LayerNorm(D)
        self.up, self.down = nn.Linear(D, 4 * D), nn.Linear(4 * D, D)

    def forward(self, x):
        return x + self.down(torch.nn.functional.gelu(self.up(self.norm(x))))


def _run(model, x):
    opt = torch.optim.SGD(model.parameters(), lr=1e-3)
    torch.cuda.synchronize()
    torch.cuda.empty_cache()
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    losses = []
    for _ in range(3):
        opt.zero_grad(set_to_none=True)
        loss = model(x).float().pow(2).mean()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    torch.cuda.synchronize()
    return losses, torch.cuda.max_memory_allocated() - base


def _save_matmuls(op, *args, **kwargs):
    name = str(op)
    return CheckpointPolicy.MUST_SAVE if ("addmm" in name or "mm" in name) else CheckpointPolicy.PREFER_RECOMPUTE


def test_losses_equal_and_peak_memory_ordering():
    torch.manual_seed(0)
    ref = nn.Sequential(*[Block() for _ in range(LAYERS)]).cuda().bfloat16()
    x = torch.randn(TOKENS, D, device="cuda", dtype=torch.bfloat16)

    def variant(wrap, chain=False):
        m = copy.deepcopy(ref)
        seq = nn.Sequential(*[wrap(b) for b in m])
        if chain:       # offload layer k during layer k+1's forward, reload it during layer k+1's backward
            for a, b in zip(seq[:-1], seq[1:]):
                SwapManager().set_forward_prefetch_layer(a, b)
        return seq

    SwapManager().reset()
    results = {"none": _run(copy.deepcopy(ref), x)}
    results["save"] = _run(variant(lambda b: checkpoint_wrapper(b, policy_fn=_save_matmuls)), x)
    results["recompute"] = _run(variant(lambda b: checkpoint_wrapper(b)), x)
    SwapManager().reset()
    big = TOKENS * 4 * D
    results["swap_policy"] = _run(variant(lambda b: swap_wrapper(b, policy_fn=lambda t: t.numel() >= big),
                                          chain=True), x)
    SwapManager().reset()
    results["swap"] = _run(variant(lambda b: swap_wrapper(b, policy_fn=lambda t: t.numel() >= TOKENS * D),
                                   chain=True), x)
    SwapManager().reset()

    want = results["none"][0]
    for name, (losses, _) in results.items():
        assert all(abs(a - b) <= 1e-5 * max(1.0, abs(b)) for a, b in zip(losses, want)), (name, losses, want)
    peak = {k: v[1] for k, v in results.items()}
    print("peak MiB:", {k: round(v / 2**20) for k, v in peak.items()})
    assert peak["none"] > peak["save"] > peak["recompute"], peak
    assert peak["none"] > peak["swap_policy"] > peak["swap"], peak
