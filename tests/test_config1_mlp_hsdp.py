"""CPU/gloo world_size=2 plumbing test: 2-layer MLP, Layout((2,1),("dp","mp")), w1 column-sharded
and w2 row-sharded on "mp", wrapped in hsdp(shard_size=2, level3); 10 AdamW steps must match a
single-process run to 1e-5 (loss and gathered weights)."""
import torch
import torch.nn.functional as F
from torch import nn

from dist_utils import run_distributed

HID, FFN, BATCH, STEPS, LR = 256, 1024, 8, 10, 1e-3


class MLP(nn.Module):
    def __init__(self, device=None):
        super().__init__()
        self.w1 = nn.Parameter(torch.empty(FFN, HID, device=device))
        self.w2 = nn.Parameter(torch.empty(HID, FFN, device=device))

    def reset_parameters(self):
        nn.init.normal_(self.w1, 0.0, 0.02)
        nn.init.normal_(self.w2, 0.0, 0.02)

    def forward(self, x):
        return F.linear(F.gelu(F.linear(x, self.w1)), self.w2)


def _data():
    g = torch.Generator().manual_seed(0)
    return torch.randn(BATCH, HID, generator=g), torch.randn(BATCH, HID, generator=g)


def _single_process():
    torch.manual_seed(1234)
    m = MLP()
    m.reset_parameters()
    x, y = _data()
    opt = torch.optim.AdamW(m.parameters(), lr=LR)
    losses = []
    for _ in range(STEPS):
        opt.zero_grad()
        loss = F.mse_loss(m(x), y)
        loss.backward()
        opt.step()
        losses.append(loss.item())
    return losses, m.w1.detach().clone(), m.w2.detach().clone()


def _worker(rank, world):
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200 import Layout, DTensor, ShardingPlan, shard_module, hsdp, init_parameters

    ref_losses, ref_w1, ref_w2 = _single_process()
    layout = Layout((2, 1), ("dp", "mp"))
    mesh = layout.mesh
    m = MLP(device="meta")
    shard_module(m, mesh, ShardingPlan(plan={"w1": ("mp", "None"), "w2": ("None", "mp")}))
    hsdp(m, shard_size=2, threshold=0, optimizer_level="level3")
    torch.manual_seed(1234)
    init_parameters(m, device="cpu")
    assert m.w1.to_local().shape == (FFN // 2, HID) and m.w2.to_local().shape == (HID // 2, FFN)

    x, y = _data()
    xs = DTensor.from_local(x.chunk(2)[rank].clone(), layout("dp", "None"))
    ys = DTensor.from_local(y.chunk(2)[rank].clone(), layout("dp", "None"))
    opt = torch.optim.AdamW(m.parameters(), lr=LR)
    losses = []
    for _ in range(STEPS):
        m.zero_grads()
        out = m(xs).reduce_partial()           # row-parallel w2 leaves Partial(sum) on mp
        loss = F.mse_loss(out, ys)             # Partial(avg) over dp
        loss = loss.reduce_partial()           # replicated on both ranks
        loss.backward(torch.tensor(1.0 / loss.layout.repeat_num()))
        hp.hsdp_sync_stream()
        with hp.SkipDTensorDispatch():
            opt.step()
        losses.append(loss.to_local().item())
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-5, (losses, ref_losses)
    # gather the HSDP shards (dim 0 over the dp ranks) and compare with the single-process weights
    import torch.distributed as dist
    for p, ref in ((m.w1, ref_w1), (m.w2, ref_w2)):
        local = p.to_local().detach().contiguous()
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local)
        full = torch.cat(parts, dim=0)
        assert torch.allclose(full, ref, atol=1e-5, rtol=0), (full - ref).abs().max()


def test_config1_mlp_hsdp_level3_matches_single_process():
    run_distributed(_worker, 2)
