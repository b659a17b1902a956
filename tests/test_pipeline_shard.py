"""Interleaved pipeline (two model chunks per rank) combined with tensor parallelism inside every
stage: 8 gloo ranks = 4 pipeline stages x TP 2, 8 one-layer virtual stages, weights sharded with
``shard_module`` on the stage's own (dp=1, tp=2) sub-mesh, DTensor activations between the stages.
Losses and weight gradients equal the single-process model.  Scenario after the reference's
``tests/torch/pipeline_parallel/pipeline_shard.py:28-106``."""
import pytest
import torch
from torch import nn

from dist_utils import run_distributed

LAYERS, HID, MICRO, BATCH = 8, 16, 4, 8


def _weights():
    g = torch.Generator().manual_seed(5)
    return [torch.randn(HID, HID, generator=g) * 0.3 for _ in range(LAYERS)]


class _Layer(nn.Module):
    def __init__(self, w):
        super().__init__()
        self.weight = nn.Parameter(w.clone())

    def forward(self, x):
        from hyper_parallel_b200 import DTensor
        x = torch.matmul(x, self.weight)
        if isinstance(x, DTensor):
            x = x.reduce_partial()
        return torch.tanh(x)


class _Chunk(nn.Module):
    """One virtual stage: a single layer kept under its global index (as the sharding plan names it)."""

    def __init__(self, index, w, last):
        super().__init__()
        self.mlp_layers = nn.ModuleDict({str(index): _Layer(w)})
        self.last = last

    def forward(self, x):
        for layer in self.mlp_layers.values():
            x = layer(x)
        return x


def _reference(x):
    layers = [_Layer(w) for w in _weights()]
    outs = []
    for xm in x.chunk(MICRO):
        h = xm
        for layer in layers:
            h = layer(h)
        h.backward(torch.ones_like(h))
        outs.append(h.detach())
    return outs, [layer.weight.grad for layer in layers]


def _worker(rank, world):
    from hyper_parallel_b200 import DTensor, Layout, PipelineStage, ShardingPlan, shard_module
    from hyper_parallel_b200.core.pipeline_parallel import ScheduleInterleaved1F1B
    stages, tp = 4, 2
    stage = rank // tp
    lay = Layout((1, tp), ("dp", "tp"), [stage * tp, stage * tp + 1])
    x = torch.linspace(-1.0, 1.0, BATCH * HID).reshape(BATCH, HID)
    ref_out, ref_grads = _reference(x)
    ws = _weights()
    # even layers shard the output dimension (their result stays sharded over tp and travels to the
    # next stage as a sharded DTensor), odd layers the contraction dimension (their product is
    # Partial and gets reduced)
    chunks, pstages = [], []
    for idx in (stage, stage + stages):
        m = _Chunk(idx, ws[idx], idx == LAYERS - 1)
        plan = ShardingPlan(plan={f"mlp_layers.{idx}.weight": ("None", "tp") if idx % 2 == 0 else ("tp", "None")})
        shard_module(m, lay.mesh, plan)
        chunks.append(m)
        pstages.append(PipelineStage(m, idx, LAYERS, device="cpu"))
    sched = ScheduleInterleaved1F1B(pstages, MICRO)
    dx = DTensor.from_local(x.clone(), lay("dp", "None"))
    out = sched.run(dx) if stage == 0 else sched.run()
    if stage == stages - 1:
        for got, want in zip(out, ref_out):
            full = got.full_tensor() if isinstance(got, DTensor) else got
            assert torch.allclose(full, want, atol=1e-5)
    r = rank % tp
    for m, idx in zip(chunks, (stage, stage + stages)):
        g = m.mlp_layers[str(idx)].weight.grad
        g = g.to_local() if isinstance(g, DTensor) else g
        want = ref_grads[idx].chunk(tp, 1)[r] if idx % 2 == 0 else ref_grads[idx].chunk(tp, 0)[r]
        assert torch.allclose(g, want, atol=1e-5), (idx, (g - want).abs().max())


def test_vpp_with_tensor_parallel_stages():
    run_distributed(_worker, 8, timeout=300.0)
