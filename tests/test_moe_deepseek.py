"""DeepSeek-V3-style model on CPU: routing invariants, EP=2 (gloo) equals EP=1, redistribute all-to-all."""
import torch

from dist_utils import run_distributed
from hyper_parallel_b200.ops import moe as moe_ops


def test_route_group_limited_topk():
    torch.manual_seed(0)
    T, E, k, G, KG = 64, 32, 4, 4, 2
    logits = torch.randn(T, E)
    bias = torch.randn(E) * 0.1
    idx, w = moe_ops.route_reference(logits, bias, k, G, KG, 2.5)
    assert idx.shape == (T, k) and w.shape == (T, k)
    assert torch.allclose(w.sum(-1), torch.full((T,), 2.5), atol=1e-5)
    groups = idx // (E // G)
    assert all(len(set(r.tolist())) <= KG for r in groups)            # only the kept groups are used
    assert all(len(set(r.tolist())) == k for r in idx)                # distinct experts
    # weights are the un-biased sigmoid scores of the selected experts
    s = torch.sigmoid(logits).gather(1, idx)
    assert torch.allclose(w, s / s.sum(-1, keepdim=True) * 2.5, atol=1e-6)


def _tiny_losses(ep_group, ep_rank, ep_size, tokens):
    from hyper_parallel_b200.models.deepseek_v3 import DeepSeekV3, DeepSeekV3Config
    cfg = DeepSeekV3Config.tiny()
    torch.manual_seed(5)
    full = DeepSeekV3(cfg, None, dtype=torch.float32)
    full.init_weights()
    model = DeepSeekV3(cfg, ep_group, dtype=torch.float32)
    sd = full.state_dict()
    local = model.layers[1].ffn.local_experts
    for k in list(sd):
        if k.endswith("ffn.w_gate_up") or k.endswith("ffn.w_down"):
            if sd[k].dim() == 3 and sd[k].shape[0] != local:
                sd[k] = sd[k][ep_rank * local:(ep_rank + 1) * local].clone()
    model.load_state_dict(sd)
    loss = model(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    return loss.detach(), model


def _ep_worker(rank, world):
    import torch.distributed as dist
    torch.manual_seed(9)
    tokens = torch.randint(0, 512, (2 * world, 17))
    # single-process oracle over the whole batch (EP=1)
    ref_loss, ref = _tiny_losses(None, 0, 1, tokens)
    mine = tokens[rank * 2:(rank + 1) * 2]
    loss, model = _tiny_losses(dist.group.WORLD, rank, world, mine)
    # data parallel over the batch: the mean of the rank losses is the global loss
    tot = loss.clone()
    dist.all_reduce(tot)
    assert abs(tot.item() / world - ref_loss.item()) < 1e-5, (tot.item() / world, ref_loss.item())
    # expert weight gradients: each expert saw all its tokens from both ranks -> grad = world * oracle/ world
    g = model.layers[1].ffn.w_down.grad
    local = g.shape[0]
    ref_g = ref.layers[1].ffn.w_down.grad[rank * local:(rank + 1) * local]
    assert torch.allclose(g / world, ref_g, atol=1e-6), (g / world - ref_g).abs().max()
    # non-expert gradients are data-parallel partial sums
    ga = model.layers[0].attn.wo.grad.clone()
    dist.all_reduce(ga)
    assert torch.allclose(ga / world, ref.layers[0].attn.wo.grad, atol=1e-6)


def test_expert_parallel_matches_single_process():
    run_distributed(_ep_worker, 2)


def _a2a_worker(rank, world):
    from hyper_parallel_b200 import DTensor, Layout
    lay = Layout((world,), ("cp",))
    full = torch.arange(4 * 6 * 2, dtype=torch.float32).reshape(4, 6, 2)
    x = DTensor.from_local(full.chunk(world, dim=0)[rank].clone().requires_grad_(), lay("cp", "None", "None"))
    y = x.redistribute(lay("None", "cp", "None"))                   # S(0) -> S(1): one all-to-all
    assert torch.equal(y.to_local(), full.chunk(world, dim=1)[rank])
    assert torch.equal(y.full_tensor(), full)
    y.to_local().sum().backward()
    assert torch.equal(x.to_local().grad, torch.ones_like(x.to_local()))


def test_redistribute_all_to_all_on_gloo():
    run_distributed(_a2a_worker, 2)
