"""The Llama block on the native kernels must agree with its PyTorch formulation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_llama_tiny_gpu_matches_cpu_reference():
    from hyper_parallel_b200.models.llama import Llama, LlamaConfig
    from hyper_parallel_b200.ops import native
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(vocab_size=1024, hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=2,
                           head_dim=128, ffn_size=1024)
    ref = Llama(cfg, dtype=torch.float32)
    ref.init_weights()
    gpu = Llama(cfg, device="cuda", dtype=torch.bfloat16)
    gpu.load_state_dict({k: v.to(torch.bfloat16) for k, v in ref.state_dict().items()})
    # compare against the bf16-rounded weights in fp32 math
    ref.load_state_dict({k: v.float().cpu() for k, v in gpu.state_dict().items()})
    tok = torch.randint(0, cfg.vocab_size, (2, 129))
    loss_ref = ref(tok[:, :-1], tok[:, 1:])
    loss_ref.backward()
    tg = tok.cuda()
    loss = gpu(tg[:, :-1], tg[:, 1:])
    loss.backward()
    native.check_status()
    assert abs(loss.item() - loss_ref.item()) < 2e-2 * abs(loss_ref.item())
    for (n, p), (_, q) in zip(gpu.named_parameters(), ref.named_parameters()):
        err = (p.grad.float().cpu() - q.grad).norm() / (q.grad.norm() + 1e-12)
        assert err < 6e-2, (n, err.item())


def test_smoke_entry():
    import __graft_entry__ as g
    g.smoke()
