"""TP=2 (+ sequence parallel) Llama on gloo equals the single-process Llama: loss and gathered grads."""
import torch

from dist_utils import run_distributed


def _reference(cfg, tokens):
    from hyper_parallel_b200.models.llama import Llama
    torch.manual_seed(21)
    m = Llama(cfg, dtype=torch.float32)
    m.init_weights()
    loss = m(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    return loss.detach(), m


def _worker(rank, world):
    import torch.distributed as dist
    from hyper_parallel_b200 import Layout
    from hyper_parallel_b200.models.llama import LlamaConfig
    from hyper_parallel_b200.models.llama_tp import TPLlama, _local
    cfg = LlamaConfig.tiny(vocab_size=256, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                           ffn_size=128)
    torch.manual_seed(3)
    tokens = torch.randint(0, cfg.vocab_size, (2, 9))
    ref_loss, ref = _reference(cfg, tokens)
    layout = Layout((1, world), ("dp", "tp"))
    model = TPLlama(cfg, layout, dtype=torch.float32)
    # load the oracle's weights, sliced the way the TP model shards them
    tp, r, hd = world, rank, cfg.head_dim
    with torch.no_grad():
        _local(model.embed).copy_(ref.embed)
        _local(model.final_norm).copy_(ref.final_norm)
        _local(model.lm_head).copy_(ref.lm_head.chunk(tp, 0)[r])
        for lt, lr in zip(model.layers, ref.layers):
            nq, nk = cfg.num_heads * hd, cfg.num_kv_heads * hd
            q, k, v = lr.wqkv.split([nq, nk, nk], 0)
            _local(lt.wqkv).copy_(torch.cat([q.chunk(tp, 0)[r], k.chunk(tp, 0)[r], v.chunk(tp, 0)[r]], 0))
            _local(lt.wo).copy_(lr.wo.chunk(tp, 1)[r])
            g, u = lr.w_gate_up.chunk(2, 0)
            _local(lt.w_gate_up).copy_(torch.cat([g.chunk(tp, 0)[r], u.chunk(tp, 0)[r]], 0))
            _local(lt.w_down).copy_(lr.w_down.chunk(tp, 1)[r])
            _local(lt.attn_norm).copy_(lr.attn_norm)
            _local(lt.ffn_norm).copy_(lr.ffn_norm)
    loss = model(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    assert abs(loss.item() - ref_loss.item()) < 1e-5, (loss.item(), ref_loss.item())
    l0, r0 = model.layers[0], ref.layers[0]
    assert torch.allclose(_local(l0.wo).grad, r0.wo.grad.chunk(tp, 1)[r], atol=1e-5)
    assert torch.allclose(_local(l0.w_down).grad, r0.w_down.grad.chunk(tp, 1)[r], atol=1e-5)
    g, u = r0.w_gate_up.grad.chunk(2, 0)
    assert torch.allclose(_local(l0.w_gate_up).grad, torch.cat([g.chunk(tp, 0)[r], u.chunk(tp, 0)[r]], 0), atol=1e-5)
    # replicated parameters (norms, embedding) get the full gradient on every rank
    assert torch.allclose(_local(l0.attn_norm).grad, r0.attn_norm.grad, atol=1e-5)
    assert torch.allclose(_local(model.embed).grad, ref.embed.grad, atol=1e-5)
    assert torch.allclose(_local(model.lm_head).grad, ref.lm_head.grad.chunk(tp, 0)[r], atol=1e-5)
    # hsdp on top of TP derives its groups from the mesh axes that do not shard the parameter
    from hyper_parallel_b200 import hsdp
    hsdp(model, shard_size=1, threshold=0)
    hp = model.layers[0].wqkv._hsdp_param
    assert hp.rank_list == [rank] and hp.shard_size == 1
    hp2 = model.embed._hsdp_param
    assert hp2.rank_list == [rank]           # tp replicas are synchronised by the TP region itself


def test_tp2_sequence_parallel_matches_single_process():
    run_distributed(_worker, 2)
