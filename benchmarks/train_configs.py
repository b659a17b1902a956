"""Training benchmarks of the hybrid-parallel configurations other than the headline one.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29544 benchmarks/train_configs.py --config {tp_hsdp,moe_ep,pp} [options]

* ``tp_hsdp``  Llama-2-13B, tensor parallel (+ sequence-parallel activations) ``--tp`` wide, HSDP
  (level3, full shard) over the remaining ranks; ``HPB_FUSED_TP=0`` selects NCCL + GEMM instead of
  the fused all-gather->GEMM / GEMM->reduce-scatter kernels.
* ``moe_ep``   DeepSeek-V3 (``--layers``, ``--experts``) with expert parallelism over all ranks.
* ``pp``       Llama-3-8B split into ``--pp`` pipeline stages (x ``--vpp`` chunks per rank), each stage
  ``--tp`` wide tensor parallel,
  schedule ``--schedule {gpipe,1f1b,vpp}``, ``--micro`` micro-batches; ``--balance 1`` lets the
  Fast-Tuner's balancer choose the layers of each virtual stage (the output head of a 128k
  vocabulary costs more than two layers, so the last stage gets fewer).

Timing rules are those of ``bench.py``: warm-up, CUDA events around exactly ``--steps`` steps,
barrier + synchronize on both sides, max over ranks; the step includes the optimizer.  Rank 0
prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def parse(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True, choices=["tp_hsdp", "moe_ep", "pp"])
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1, help="sequences per data-parallel replica (per rank for moe_ep)")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--tp", type=int, default=None)
    ap.add_argument("--pp", type=int, default=None)
    ap.add_argument("--vpp", type=int, default=2)
    ap.add_argument("--micro", type=int, default=8)
    ap.add_argument("--schedule", default="1f1b", choices=["gpipe", "1f1b", "vpp"])
    ap.add_argument("--balance", type=int, default=0,
                    help="pp: 1 = split the layers with the Fast-Tuner's pipeline balancer (fewer layers beside "
                         "the output head) instead of evenly")
    ap.add_argument("--experts", type=int, default=None)
    ap.add_argument("--fp8", type=int, default=1, help="moe_ep: fp8 block-scaled forward GEMMs (1) or bf16 (0)")
    return ap.parse_args(argv)


def timed_steps(step, args, dev, host=None):
    """Device-timed loop over ``step(i)``; with ``host`` (pinned token batches) also the end-to-end loop
    ``step(i, tokens copied from the host in this step)`` + a device->host read of the result.  Returns
    ``(ms per step, last result, clocks, end-to-end ms per step or None)``."""
    import time
    from hyper_parallel_b200.ops import native
    from hyper_parallel_b200.utils.clocks import ClockSampler
    for i in range(args.warmup):
        step(i)
    native.check_status()
    dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(dev.index) as clocks:
        e0.record()
        for i in range(args.steps):
            out = step(args.warmup + i)
        e1.record()
        dist.barrier()
        torch.cuda.synchronize()
    native.check_status()
    e2e = None
    if host is not None:
        dist.barrier()
        torch.cuda.synchronize()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        f0.record()
        for i in range(args.steps):
            tok = host[args.warmup + i].to(dev, non_blocking=True)
            _ = float(step(args.warmup + i, tok).detach())
        f1.record()
        dist.barrier()
        torch.cuda.synchronize()
        e2e = max(f0.elapsed_time(f1), (time.perf_counter() - t0) * 1e3) / args.steps
        native.check_status()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps, e2e or 0.0], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t[0].item(), out, clocks.summary(), (t[1].item() if host is not None else None)


def run_tp_hsdp(args, rank, world, dev):
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200 import Layout
    from hyper_parallel_b200.models.llama import LlamaConfig
    from hyper_parallel_b200.models.llama_tp import TPLlama
    from hyper_parallel_b200.optim import FusedAdamW
    tp = args.tp or min(4, world)
    dp = world // tp
    cfg = LlamaConfig.llama2_13b()
    if args.layers:
        cfg.num_layers = args.layers
    layout = Layout((dp, tp), ("dp", "tp"))
    model = TPLlama(cfg, layout, device=dev)
    model.init_weights()
    kw = dict(shard_size=dp, threshold=0, optimizer_level="level3", comm_fusion=dp > 1, comm_async=dp > 1)
    for layer in model.layers:
        hp.hsdp(layer, **kw)
    hp.hsdp(model, **kw)
    opt = FusedAdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    dp_rank = rank // tp
    g = torch.Generator().manual_seed(dp_rank)
    host = torch.randint(0, cfg.vocab_size, (args.warmup + args.steps, args.batch, args.seq_len + 1),
                         generator=g).pin_memory()
    toks = host.to(dev)

    def step(i, tok=None):
        tok = toks[i] if tok is None else tok
        model.zero_grads()
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        hp.hsdp_sync_stream()
        opt.step()
        return loss

    ms, loss, clocks, e2e = timed_steps(step, args, dev, host)
    tokens = dp * args.batch * args.seq_len
    return {"config": {"model": "llama2_13b", "layers": cfg.num_layers, "parallelism": f"tp{tp}(+sp) x hsdp{dp} level3",
                       "global_batch": dp * args.batch, "seq_len": args.seq_len},
            "arm": {"fused_tp": os.environ.get("HPB_FUSED_TP", "1") != "0"},
            "e2e_ms": e2e, "h2d_bytes": host[0].numel() * host.element_size(),
            "ms_per_step": ms, "value": tokens / (ms / 1e3), "loss": float(loss.detach()), "clocks": clocks,
            "mfu_flops_per_token": cfg.flops_per_token(args.seq_len)}


def run_moe_ep(args, rank, world, dev):
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200.models.deepseek_v3 import DeepSeekV3, DeepSeekV3Config
    from hyper_parallel_b200.optim import FusedAdamW
    cfg = DeepSeekV3Config()
    if args.layers:
        cfg.num_layers = args.layers
    if args.experts:
        cfg.n_routed_experts = args.experts
    cfg.fp8 = bool(args.fp8)
    model = DeepSeekV3(cfg, ep_group=dist.group.WORLD if world > 1 else None, device=dev)
    model.init_weights()
    # the non-expert parameters are data parallel over the expert-parallel ranks: hsdp (level3, full
    # shard) on them; the experts are owned by their rank and left alone (MoE marks them hsdp_ignore)
    if world > 1:
        kw = dict(shard_size=world, threshold=0, optimizer_level="level3", comm_fusion=True, comm_async=True,
                  grad_scale=1.0 / world)
        for layer in model.layers:
            hp.hsdp(layer, **kw)
        hp.hsdp(model, **kw)
    opt = FusedAdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    if world > 1:
        opt.fuse_into_backward(model)
    g = torch.Generator().manual_seed(rank)
    host = torch.randint(0, cfg.vocab_size, (args.warmup + args.steps, args.batch, args.seq_len + 1),
                         generator=g).pin_memory()
    toks = host.to(dev)

    def step(i, tok=None):
        tok = toks[i] if tok is None else tok
        if world > 1:
            model.zero_grads()
        opt.zero_grad(set_to_none=True)
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        if world > 1:
            hp.hsdp_sync_stream()
        opt.step()
        return loss

    ms, loss, clocks, e2e = timed_steps(step, args, dev, host)
    tokens = world * args.batch * args.seq_len
    return {"config": {"model": "deepseek_v3", "layers": cfg.num_layers, "experts": cfg.n_routed_experts,
                       "parallelism": f"ep{world} + hsdp level3 x{world} on the non-expert parameters",
                       "global_batch": world * args.batch, "seq_len": args.seq_len,
                       "precision": "fp8 e4m3 block-scaled forward GEMMs (1x128 / 128x128), bf16 master weights"
                       if cfg.fp8 else "bf16"},
            "e2e_ms": e2e, "h2d_bytes": host[0].numel() * host.element_size(),
            "ms_per_step": ms, "value": tokens / (ms / 1e3), "loss": float(loss.detach()), "clocks": clocks,
            "mfu_flops_per_token": cfg.flops_per_token(args.seq_len)}


def run_pp(args, rank, world, dev):
    from torch import nn
    from hyper_parallel_b200 import PipelineStage
    from hyper_parallel_b200 import ops
    from hyper_parallel_b200.core.pipeline_parallel import Schedule1F1B, ScheduleGPipe, ScheduleInterleaved1F1B
    from hyper_parallel_b200.models.llama import Llama, LlamaBlock, LlamaConfig
    from hyper_parallel_b200.optim import FusedAdamW
    import torch.nn.functional as F
    tp = args.tp or 1
    pp = args.pp or world // tp
    assert pp * tp == world, "pipeline stages x tensor-parallel width must equal the world size"
    cfg = LlamaConfig.llama3_8b()
    if args.layers:
        cfg.num_layers = args.layers
    chunks = args.vpp if args.schedule == "vpp" else 1
    n_virtual = pp * chunks
    per = cfg.num_layers // n_virtual
    ranges = [(i * per, (i + 1) * per) for i in range(n_virtual)]
    if args.balance:
        from hyper_parallel_b200.auto_parallel.fast_tuner.pipeline_balance import (
            balance_pipeline, dense_transformer_profile, layer_ranges)
        prof = dense_transformer_profile(cfg.hidden_size, cfg.ffn_size, cfg.num_heads, cfg.num_kv_heads, cfg.head_dim,
                                         cfg.vocab_size, args.seq_len)
        ranges = layer_ranges(balance_pipeline(cfg.num_layers, cfg.num_layers, pp, chunks, args.micro, prof,
                                               max_offset=3).layers)
    S, B = args.seq_len, args.batch
    stage_rank = rank // tp                      # ranks [s * tp, (s + 1) * tp) form pipeline stage s

    class Chunk(nn.Module):
        """Layers [lo, hi) of the model; the first chunk embeds, the last computes the loss."""

        def __init__(self, lo, hi, first, last):
            super().__init__()
            self.first, self.last = first, last
            self.layers = nn.ModuleList(LlamaBlock(cfg, i, device=dev) for i in range(lo, hi))
            if first:
                self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, device=dev, dtype=torch.bfloat16))
                nn.init.normal_(self.embed, 0.0, 0.02)
            if last:
                self.final_norm = nn.Parameter(torch.ones(cfg.hidden_size, device=dev, dtype=torch.bfloat16))
                self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, device=dev, dtype=torch.bfloat16))
                nn.init.normal_(self.lm_head, 0.0, 0.02)
            for l in self.layers:
                l.reset_parameters()
            self.targets = None

        def forward(self, x):
            mb = x.shape[0]
            if self.first:
                h, resid = F.embedding(x[:, :-1].reshape(-1), self.embed), None
            else:
                h, resid = x.reshape(-1, cfg.hidden_size), None
            for l in self.layers:
                h, resid = l(h, resid, mb, S)
            h = h if resid is None else h + resid
            if not self.last:
                return h.view(mb, S, cfg.hidden_size)
            xn = ops.rmsnorm(h, self.final_norm, cfg.norm_eps)
            logits = ops.linear(xn, self.lm_head)
            tgt = self.targets.pop(0)
            return ops.fused_cross_entropy(logits, tgt.reshape(-1), float(tgt.numel() * args.micro), unit_grad=True)

    class TPChunk(nn.Module):
        """The same slice of the model, tensor parallel (+ sequence-parallel activations) inside the stage."""

        def __init__(self, lo, hi, first, last):
            super().__init__()
            from hyper_parallel_b200 import Layout
            from hyper_parallel_b200.models.llama_tp import TPLlama
            self.first, self.last = first, last
            self.m = TPLlama(cfg, Layout((1, tp), ("dp", "tp"), list(range(stage_rank * tp, stage_rank * tp + tp))), device=dev, first_layer=lo, num_layers=hi - lo,
                             with_embed=first, with_head=last)
            self.m.init_weights()
            self.targets = None

        def forward(self, *x):
            kw = {}
            if self.last:
                tgt = self.targets.pop(0)
                kw = dict(targets=tgt, loss_denominator=float(tgt.numel() * args.micro))
            if self.first:
                return self.m(x[0][:, :-1].contiguous(), **kw)
            return self.m((x[0], x[1]), batch=B, seq_len=S, **kw)

    if tp > 1:
        Chunk = TPChunk  # noqa: F811
        # The fused tensor-parallel kernels rendezvous with their peer inside the kernel while they
        # occupy every SM; a pipeline send that the peer's progress depends on may then not get
        # scheduled.  Inside pipeline stages tensor parallelism therefore uses NCCL + GEMM.
        os.environ["HPB_FUSED_TP"] = "0"
    idx = [stage_rank + c * pp for c in range(chunks)]
    mods = [Chunk(ranges[i][0], ranges[i][1], i == 0, i == n_virtual - 1) for i in idx]
    stages = [PipelineStage(m, i, n_virtual, device=dev) for m, i in zip(mods, idx)]
    if args.schedule == "vpp":
        sched = ScheduleInterleaved1F1B(stages, args.micro)
    else:
        sched = (ScheduleGPipe if args.schedule == "gpipe" else Schedule1F1B)(stages[0], args.micro)
    params = [p for m in mods for p in m.parameters()]
    opt = FusedAdamW(params, lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    g = torch.Generator().manual_seed(0)
    host = torch.randint(0, cfg.vocab_size, (args.warmup + args.steps, B * args.micro, S + 1), generator=g).pin_memory()
    toks = host.to(dev)
    last_mod = mods[-1] if mods[-1].last else None

    def step(i, tok=None):
        tok = toks[i] if tok is None else tok
        opt.zero_grad(set_to_none=True)
        if last_mod is not None:
            last_mod.targets = list(tok[:, 1:].chunk(args.micro))
        out = sched.run(tok) if stage_rank == 0 else sched.run()
        opt.step()
        return torch.stack([o.detach() for o in out]).sum() if out is not None else torch.zeros((), device=dev)

    ms, loss, clocks, e2e = timed_steps(step, args, dev, host)
    trace = sched.trace_report()        # HPB_PP_TRACE=1: mean device time and count per kind of step, per rank
    if trace:
        print(f"[pp trace] rank {rank} stage {stage_rank} {args.schedule}: " +
              "  ".join(f"{k} {v[0]:.2f} ms x{v[1]}" for k, v in sorted(trace.items())), flush=True)
    tl = sched.trace_timeline()         # HPB_PP_TRACE=2: the compute steps of the last step on this rank's stream
    if tl:
        print(f"[pp timeline] rank {rank} {args.schedule}: " +
              " ".join(f"{lab}{m}:{a:.0f}-{b:.0f}" for lab, m, a, b in tl), flush=True)
    lt = loss.clone()
    dist.all_reduce(lt, op=dist.ReduceOp.MAX)
    tokens = B * args.micro * S
    stats = torch.cuda.memory_stats(dev)
    mem = torch.tensor([torch.cuda.max_memory_allocated(dev) / 2**30, torch.cuda.max_memory_reserved(dev) / 2**30,
                        float(stats.get("num_alloc_retries", 0)), float(stats.get("num_device_alloc", 0))],
                       device=dev, dtype=torch.float64)
    dist.all_reduce(mem, op=dist.ReduceOp.MAX)
    return {"config": {"model": "llama3_8b", "layers": cfg.num_layers, "parallelism": f"pp{pp} x tp{tp} {args.schedule}"
                       + (f" x{chunks} chunks" if chunks > 1 else ""), "micro_batches": args.micro,
                       "global_batch": B * args.micro, "seq_len": S,
                       "layers_per_virtual_stage": [hi - lo for lo, hi in ranges]},
            "e2e_ms": e2e, "h2d_bytes": host[0].numel() * host.element_size(),
            "ms_per_step": ms, "value": tokens / (ms / 1e3), "loss": float(lt.detach()), "clocks": clocks,
            "memory_max_over_ranks": {"peak_allocated_gib": round(float(mem[0]), 2),
                                      "peak_reserved_gib": round(float(mem[1]), 2),
                                      "alloc_retries": int(mem[2]), "device_allocs": int(mem[3])},
            "mfu_flops_per_token": cfg.flops_per_token(S)}


def main(argv=None):
    args = parse(argv)
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    res = {"tp_hsdp": run_tp_hsdp, "moe_ep": run_moe_ep, "pp": run_pp}[args.config](args, rank, world, dev)
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("bf16_tflops_sustained", 1400.0)
    except OSError:
        peak = 1400.0
    fpt = res.pop("mfu_flops_per_token")
    res["mfu_of_measured_sustained_bf16"] = fpt * res["value"] / world / (peak * 1e12)
    from hyper_parallel_b200.ops import native
    e2e_ms, h2d = res.pop("e2e_ms", None), res.pop("h2d_bytes", 0)
    tokens_per_step = res["value"] * res["ms_per_step"] / 1e3
    res.update({"metric": "train tokens/sec (device-timed, max over ranks)", "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": args.warmup, "dtype": "bf16", "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "impl": "ours",
                "data": "synthetic (uniform token ids, seed 0; random-init weights)",
                "gpu_launches": native.launch_count})
    if e2e_ms:
        res["e2e"] = {"value": tokens_per_step / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                      "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4}
    from hyper_parallel_b200.utils.logging import MetricsWriter, get_logger
    get_logger("hyper_parallel_b200.bench").info("%s x%d: %.1f ms/step", args.config, world, res["ms_per_step"])
    MetricsWriter(os.environ.get("HPB_METRICS_JSONL")).write(args.steps, config=args.config,
                                                             tokens_per_s=res["value"], ms_per_step=res["ms_per_step"],
                                                             n_gpus=world, loss=res.get("loss", 0.0))
    if rank == 0:
        print(json.dumps(res))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
