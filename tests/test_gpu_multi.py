"""Multi-GPU tests (need >= 2 CUDA devices): the symmetric-memory HSDP path (P2P all-gather,
fused reduce-scatter + AdamW) must train like the torch.distributed path, and a peer wait that
nothing satisfies must time out with a status code instead of hanging."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _need(n):
    if torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")


def _train(rank, world, fused, steps, out):
    import torch.distributed as dist
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200.models.llama import Llama, LlamaConfig
    from hyper_parallel_b200.ops import native
    from hyper_parallel_b200.optim import FusedAdamW
    os.environ["HPB_FUSED_COMM"] = "1" if fused else "0"
    dev = torch.device("cuda", rank)
    cfg = LlamaConfig.tiny(vocab_size=1024, hidden_size=512, num_layers=2, num_heads=4, num_kv_heads=2,
                           head_dim=128, ffn_size=1024)
    model = Llama(cfg, device="meta")
    for layer in model.layers:
        hp.hsdp(layer, shard_size=world, threshold=0, optimizer_level="level3", comm_fusion=True, comm_async=True)
    hp.hsdp(model, shard_size=world, threshold=0, optimizer_level="level3", comm_fusion=True, comm_async=True)
    hp.init_parameters(model, device=dev, seed=0)
    n_symm = sum(len(m.hsdp_scheduler.hsdp_state.symm_buffers) for m in model.modules() if "hsdp_scheduler" in m.__dict__)
    assert (n_symm > 0) == fused
    # two parameter groups (no weight decay and a larger step for the norm weights): they share the flat
    # buffer of their module with the matrices, and both paths must honour the per-group values
    decay = [p for p in model.parameters() if p.dim() > 1]
    no_decay = [p for p in model.parameters() if p.dim() <= 1]
    opt = FusedAdamW([{"params": decay}, {"params": no_decay, "weight_decay": 0.0, "lr": 5e-2}], lr=1e-3,
                     betas=(0.9, 0.95), weight_decay=0.1)
    opt.fuse_into_backward(model)
    g = torch.Generator().manual_seed(100 + rank)
    losses = []
    for _ in range(steps):
        tok = torch.randint(0, cfg.vocab_size, (2, 129), generator=g).to(dev)
        model.zero_grads()
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        hp.hsdp_sync_stream()
        opt.step()
        losses.append(loss.item())
    native.check_status()
    torch.cuda.synchronize()
    # nothing wrote outside the symmetric regions (guard words in front of and behind every buffer)
    for m in model.modules():
        if "hsdp_scheduler" in m.__dict__:
            for buf in m.hsdp_scheduler.hsdp_state.symm_buffers:
                buf.symm.check_canaries()
    # gather the final weights of one parameter for comparison
    w = model.layers[0].wqkv.detach().float().contiguous()
    parts = [torch.empty_like(w) for _ in range(world)]
    dist.all_gather(parts, w)
    nw = model.layers[0].attn_norm.detach().float().contiguous()
    nparts = [torch.empty_like(nw) for _ in range(world)]
    dist.all_gather(nparts, nw)
    if rank == 0:
        torch.save({"losses": losses, "w": torch.cat(parts, 0).cpu(), "norm": torch.cat(nparts, 0).cpu()}, out)


def _worker(rank, world, port, tmp):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from hyper_parallel_b200.core.hsdp.hsdp_scheduler import reset_hsdp_registry
    _train(rank, world, False, 3, os.path.join(tmp, "ref.pt"))
    reset_hsdp_registry()
    _train(rank, world, True, 3, os.path.join(tmp, "fused.pt"))
    reset_hsdp_registry()
    _train(rank, world, True, 3, os.path.join(tmp, "fused2.pt"))      # second identical run: determinism
    reset_hsdp_registry()
    os.environ["HPB_FUSED_AG"] = "1"           # weight gathers inside the consumer GEMMs (and riding ahead)
    try:
        _train(rank, world, True, 3, os.path.join(tmp, "fused_ag.pt"))
    finally:
        os.environ.pop("HPB_FUSED_AG", None)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_symmetric_hsdp_matches_nccl_path(tmp_path, world):
    _need(world)
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    a, b = torch.load(tmp_path / "ref.pt"), torch.load(tmp_path / "fused.pt")
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 2e-2 * abs(x), (a["losses"], b["losses"])
    rel = (a["w"] - b["w"]).norm() / a["w"].norm()
    assert rel < 5e-3, rel.item()
    # the norm weights moved (lr 5e-2) and moved alike: the per-group hyper-parameters reached the fused kernel
    assert (a["norm"] - 1.0).abs().max() > 1e-2
    assert (a["norm"] - b["norm"]).abs().max() < 2e-2, (a["norm"] - b["norm"]).abs().max()
    # the fused path run twice from the same seeds gives the same bits (no race shows up as noise)
    c = torch.load(tmp_path / "fused2.pt")
    assert b["losses"] == c["losses"], ("second run differs", b["losses"], c["losses"])
    assert torch.equal(b["w"], c["w"]), ("second run differs", (b["w"] - c["w"]).abs().max().item())
    # gathering the weights inside the GEMMs moves the same bytes; the input-gradient product then
    # walks its K blocks in arrival order, so the sums agree to rounding, not to the bit
    d = torch.load(tmp_path / "fused_ag.pt")
    for x, y in zip(b["losses"], d["losses"]):
        assert abs(x - y) < 2e-3 * abs(x), ("fused gather vs copy kernel", b["losses"], d["losses"])
    rel_ag = ((b["w"] - d["w"]).norm() / b["w"].norm()).item()
    assert rel_ag < 5e-3, ("fused gather vs copy kernel", rel_ag)


def test_peer_wait_times_out_with_status_not_a_hang():
    """Single GPU: wait on a flag that nothing sets, with a 20 ms limit; the kernel must return and
    record status code 5 (peer flag timeout), and the context must stay usable."""
    from hyper_parallel_b200.ops import native
    from hyper_parallel_b200.parallel.symm import SymmetricMemory
    sm = SymmetricMemory(None, 1024)
    st = native.status_word(sm.device)
    st.zero_()
    sm.world = 2                       # pretend there is a peer whose flag never arrives
    import ctypes
    arr = (ctypes.c_void_p * 2)(sm.pad_ptrs[0], sm.pad_ptrs[0])
    rc = sm.lib.hpb_symm_barrier(arr, 0, 2, 5, 7, 20_000_000, 0, st.data_ptr(), native.stream(sm.device))
    assert rc == 0
    torch.cuda.synchronize()
    code, detail = st.tolist()
    assert code == 5 and (detail >> 8) == 5
    with pytest.raises(RuntimeError, match="peer flag"):
        native.check_status()
    assert torch.ones(4, device="cuda").sum().item() == 4.0      # context still healthy
    sm.world = 1
    sm.close()


def _tp_worker(rank, world, port, tmp):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hyper_parallel_b200.ops import native
    from hyper_parallel_b200.parallel.tp_fused import TPWorkspace
    Ms, K, N = 384, 512, 640
    ws = TPWorkspace(dist.group.WORLD, Ms * K * 2, world * Ms * N * 2)
    ok = True
    for call in range(3):                       # three calls: exercises both buffer parities
        g = torch.Generator(device=dev).manual_seed(50 + call)
        xs = [torch.randn(Ms, K, device=dev, generator=g).to(torch.bfloat16) for _ in range(world)]
        w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
        # all-gather -> GEMM: every rank contributes xs[rank]
        y = ws.ag_gemm(xs[rank], w)
        ref = torch.cat(xs).float() @ w.float().t()
        ok &= ((y.float() - ref).norm() / ref.norm()).item() < 5e-3
        # GEMM -> reduce-scatter: rank r holds a_r; the sum over ranks of a_r @ w^T, my row block
        a_all = [torch.randn(world * Ms, K, device=dev, generator=g).to(torch.bfloat16) for _ in range(world)]
        z = ws.gemm_rs(a_all[rank], w)
        full = sum(a.float() @ w.float().t() for a in a_all)
        refz = full[rank * Ms:(rank + 1) * Ms]
        ok &= ((z.float() - refz).norm() / refz.norm()).item() < 1e-2
    torch.cuda.synchronize()
    native.check_status()
    ws.symm.check_canaries()
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"ok": bool(t.item())}, os.path.join(tmp, "tp.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_ag_gemm_and_gemm_rs_match_reference(tmp_path, world):
    _need(world)
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    mp.spawn(_tp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert torch.load(tmp_path / "tp.pt")["ok"]


def _tp_bwd_worker(rank, world, port, tmp):
    """Column- and row-parallel linears through autograd: all four backward products (fused
    GEMM->reduce-scatter, peer-pull gather + wgrad, fused all-gather->GEMM, wgrad from the staged
    gather) against the single-process formulas."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hyper_parallel_b200.ops import native
    from hyper_parallel_b200.parallel import tensor_parallel as tp
    Ms, K, Ns = 256, 384, 320            # token rows per rank, hidden, output columns per rank
    T = Ms * world
    g = torch.Generator(device=dev).manual_seed(7)          # same seed everywhere: every rank sees all shards

    def rnd(*shape, s=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * s).to(torch.bfloat16)
    xs = [rnd(Ms, K) for _ in range(world)]
    wcs = [rnd(Ns, K, s=0.05) for _ in range(world)]
    gys = [rnd(T, Ns) for _ in range(world)]
    as_ = [rnd(T, K) for _ in range(world)]
    wrs = [rnd(Ns, K, s=0.05) for _ in range(world)]
    gzs = [rnd(Ms, Ns) for _ in range(world)]
    ok = True

    def close(a, b, tol=1e-2):
        return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item() < tol
    for _ in range(2):                                      # twice: both parities of the workspace buffers
        x = xs[rank].clone().requires_grad_()
        wc = wcs[rank].clone().requires_grad_()
        y = tp.column_parallel_linear(x, wc, dist.group.WORLD)
        y.backward(gys[rank])
        X = torch.cat(xs).float()
        dX = sum(gys[r].float() @ wcs[r].float() for r in range(world))
        ok &= close(y, X @ wcs[rank].float().t())
        ok &= close(x.grad, dX[rank * Ms:(rank + 1) * Ms])
        ok &= close(wc.grad, gys[rank].float().t() @ X)
        a = as_[rank].clone().requires_grad_()
        wr = wrs[rank].clone().requires_grad_()
        z = tp.row_parallel_linear(a, wr, dist.group.WORLD)
        z.backward(gzs[rank])
        Z = sum(as_[r].float() @ wrs[r].float().t() for r in range(world))
        dZ = torch.cat(gzs).float()
        ok &= close(z, Z[rank * Ms:(rank + 1) * Ms], 2e-2)
        ok &= close(a.grad, dZ @ wrs[rank].float())
        ok &= close(wr.grad, dZ.t() @ as_[rank].float())
    torch.cuda.synchronize()
    native.check_status()
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"ok": bool(t.item())}, os.path.join(tmp, "tpb.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_backward_products_are_fused_and_correct(tmp_path, world):
    _need(world)
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    mp.spawn(_tp_bwd_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert torch.load(tmp_path / "tpb.pt")["ok"]


def _ep_worker(rank, world, port, tmp):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hyper_parallel_b200.ops import moe, native
    from hyper_parallel_b200.parallel import ep_fused
    T, H, Fh, E, k = 260, 256, 128, 8, 3
    El = E // world
    g = torch.Generator(device=dev).manual_seed(100 + rank)
    x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
    wgu = (torch.randn(El, 2 * Fh, H, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    wd = (torch.randn(El, H, Fh, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, device=dev, generator=g)[:k] for _ in range(T)])
    wts = torch.rand(T, k, device=dev, generator=g)
    ok = True
    for it in range(2):                                   # twice: the workspace is reused
        dy = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        res = []
        for fused in (True, False):
            xa, wa, ga, da = [t.clone().requires_grad_() for t in (x, wts, wgu, wd)]
            f = ep_fused.fused_expert_parallel_ffn if fused else moe.expert_parallel_ffn
            y = f(xa, idx, wa, ga, da, E, dist.group.WORLD)
            y.backward(dy)
            res.append([y] + [t.grad for t in (xa, wa, ga, da)])
        for a, b in zip(*res):
            ok &= ((a.float() - b.float()).norm() / (b.float().norm() + 1e-9)).item() < 2e-2
    torch.cuda.synchronize()
    native.check_status()
    t = torch.tensor([1.0 if ok else 0.0], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    if rank == 0:
        torch.save({"ok": bool(t.item())}, os.path.join(tmp, "ep.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_expert_parallel_dispatch_combine_matches_nccl_path(tmp_path, world):
    _need(world)
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    mp.spawn(_ep_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert torch.load(tmp_path / "ep.pt")["ok"]


def _fsdp_pp_worker(rank, world, port, tmp):
    """fully_shard and a two-stage 1F1B pipeline on NCCL must reproduce a single-GPU run."""
    import torch.distributed as dist
    from torch import nn
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from hyper_parallel_b200 import PipelineStage, SkipDTensorDispatch
    from hyper_parallel_b200.core.fully_shard import fully_shard
    from hyper_parallel_b200.core.pipeline_parallel import Schedule1F1B

    def make():
        torch.manual_seed(21)
        return nn.Sequential(nn.Linear(256, 512), nn.GELU(), nn.Linear(512, 256), nn.Tanh(),
                             nn.Linear(256, 256), nn.GELU(), nn.Linear(256, 64)).to(dev)

    g = torch.Generator().manual_seed(5)
    x = torch.randn(8 * world, 256, generator=g).to(dev)
    y = torch.randn(8 * world, 64, generator=g).to(dev)

    ref = make()
    ref_opt = torch.optim.SGD(ref.parameters(), lr=0.05)
    ref_losses = []
    for _ in range(3):
        ref_opt.zero_grad()
        loss = (ref(x) - y).pow(2).mean()
        loss.backward()
        ref_opt.step()
        ref_losses.append(loss.item())

    # fully_shard: two wrapped halves + the root, forward prefetch, per-rank batch slices
    net = make()
    first, second = nn.Sequential(*list(net)[:4]), nn.Sequential(*list(net)[4:])
    model = nn.Sequential(first, second)
    fully_shard(first)
    fully_shard(second)
    fully_shard(model)
    first.set_modules_to_forward_prefetch([second])
    second.set_modules_to_backward_prefetch([first])
    opt = torch.optim.SGD(model.parameters(), lr=0.05)
    xs, ys = x.chunk(world)[rank], y.chunk(world)[rank]
    for step in range(3):
        with SkipDTensorDispatch():
            opt.zero_grad()
        loss = (model(xs) - ys).pow(2).mean()
        loss.backward()
        with SkipDTensorDispatch():
            opt.step()
        total = loss.detach().clone()
        dist.all_reduce(total)
        assert abs(total.item() / world - ref_losses[step]) < 1e-4 * max(1.0, abs(ref_losses[step])), \
            ("fully_shard", step, total.item() / world, ref_losses[step])
    first.unshard()                                      # acts on this module's own parameter group
    assert torch.allclose(first[0].weight, ref[0].weight, atol=1e-5)
    first.reshard()

    # pipeline: stage r holds half of the layers; 4 micro-batches through 1F1B, one SGD step
    net = make()
    ref2 = make()
    micro = 4
    ref2_losses = []
    for xm, ym in zip(x.chunk(micro), y.chunk(micro)):
        l = (ref2(xm) - ym).pow(2).mean() / micro
        l.backward()
        ref2_losses.append(l.item())

    class Last(nn.Module):
        def __init__(self, body):
            super().__init__()
            self.body, self.targets = body, None

        def forward(self, h):
            t = self.targets.pop(0)
            return (self.body(h) - t).pow(2).mean() / micro

    body = nn.Sequential(*list(net)[:4]) if rank == 0 else Last(nn.Sequential(*list(net)[4:]))
    stage = PipelineStage(body, rank, world, device=dev)
    sched = Schedule1F1B(stage, micro)
    for _ in range(2):                                   # the second run reuses the cached shapes
        for p in body.parameters():
            p.grad = None
        if rank == world - 1:
            body.targets = list(y.chunk(micro))
        out = sched.run(x) if rank == 0 else sched.run()
        if rank == world - 1:
            got = [o.item() for o in out]
            assert all(abs(a - b) < 1e-5 for a, b in zip(got, ref2_losses)), (got, ref2_losses)
        mine = list(ref2)[:4] if rank == 0 else list(ref2)[4:]
        theirs = list(net)[:4] if rank == 0 else list(net)[4:]
        for a, b in zip(mine, theirs):
            for pa, pb in zip(a.parameters(), b.parameters()):
                assert torch.allclose(pa.grad, pb.grad, atol=1e-5)
    dist.barrier()
    dist.destroy_process_group()


def test_fully_shard_and_pipeline_on_nccl(tmp_path):
    _need(2)
    import torch.multiprocessing as mp
    from dist_utils import _free_port
    mp.spawn(_fsdp_pp_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
