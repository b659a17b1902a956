#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B training tokens/s with hsdp full shard (level3) on N B200.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W

Prints ONE JSON line from rank 0.  ``value`` is total tokens/s over all GPUs, timed on the
device with CUDA events (max over ranks) with inputs resident on the device; ``e2e`` is the
same metric through the public API with the per-step host->device copy of the token batch
from pinned memory and a device->host read of the loss inside the timed region.
``--impl reference`` runs the unmodified reference package installed under baseline/_ref.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="llama3_8b", choices=["llama3_8b", "llama2_13b", "tiny"])
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--batch-per-gpu", type=int, default=2)
    ap.add_argument("--layers", type=int, default=None, help="debug only: override the layer count")
    ap.add_argument("--config", default="hsdp", choices=["hsdp", "tp_hsdp", "moe_ep", "pp"],
                    help="hsdp: the headline (Llama-3-8B, hsdp level3); tp_hsdp: Llama-2-13B TP=4 (+SP) x hsdp 2, "
                         "global batch 8; moe_ep: DeepSeek-V3 4 layers, 256 experts, EP over all ranks, fp8; "
                         "pp: Llama-3-8B PP=4 x TP=2, 16 micro-batches")
    ap.add_argument("--schedule", default="1f1b", choices=["gpipe", "1f1b", "vpp"], help="--config pp only")
    ap.add_argument("--check", action="store_true",
                    help="after the timed runs, rebuild the model on the NCCL path (HPB_FUSED_COMM=0) and compare "
                         "the losses of the first two steps with those of the symmetric-memory kernels; the "
                         "result goes into the JSON line (N > 1 only)")
    ap.add_argument("--metrics-jsonl", default=os.environ.get("HPB_METRICS_JSONL"),
                    help="also append the result (and the per-kernel-path switches) as one JSON line to this file")
    return ap.parse_args()


def other_config_argv(args, world):
    """Command line of benchmarks/train_configs.py for the non-headline configurations, as the
    benchmark specification names them (smaller world sizes shrink the parallel degrees, not the model)."""
    base = ["--steps", str(args.steps), "--warmup", str(args.warmup), "--seq-len", str(args.seq_len)]
    if args.layers is not None:
        base += ["--layers", str(args.layers)]
    if args.config == "tp_hsdp":
        tp = min(4, world)
        dp = max(world // tp, 1)
        return ["--config", "tp_hsdp", "--tp", str(tp), "--batch", str(max(8 // dp, 1))] + base
    if args.config == "moe_ep":
        return ["--config", "moe_ep", "--batch", "1", "--fp8", "1"] + (base if args.layers else base + ["--layers", "4"])
    tp = 2 if world >= 4 else 1
    return ["--config", "pp", "--tp", str(tp), "--pp", str(max(world // tp, 1)), "--micro", "16", "--batch", "1",
            "--schedule", args.schedule, "--vpp", "2"] + base


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    return rank, local, world


def model_config(args):
    from hyper_parallel_b200.models.llama import LlamaConfig
    cfg = {"llama3_8b": LlamaConfig.llama3_8b, "llama2_13b": LlamaConfig.llama2_13b,
           "tiny": LlamaConfig.tiny}[args.model]()
    if args.layers is not None:
        cfg.num_layers = args.layers
    return cfg


def make_batches(cfg, args, rank, n):
    g = torch.Generator().manual_seed(0 + rank)
    toks = torch.randint(0, cfg.vocab_size, (n, args.batch_per_gpu, args.seq_len + 1), generator=g,
                         dtype=torch.int64)
    return toks.pin_memory()


def _shared_config(args, layers, hidden, world):
    """One ``config`` dict for both arms (the reference arm's module defines it and imports nothing of
    this package)."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    from reference_arm import bench_config
    return bench_config(args, layers, hidden, world)


def run_ours(args):
    import torch.distributed as dist
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200.models.llama import Llama
    from hyper_parallel_b200.ops import native
    from hyper_parallel_b200.optim import FusedAdamW
    from hyper_parallel_b200.utils.clocks import ClockSampler

    rank, local, world = dist_env()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    cfg = model_config(args)

    def build():
        """Public API: build on meta, shard with hsdp (full shard, level3), deferred init."""
        model = Llama(cfg, device="meta")
        for layer in model.layers:
            hp.hsdp(layer, shard_size=world, threshold=0, optimizer_level="level3", comm_fusion=world > 1,
                    comm_async=world > 1)
        hp.hsdp(model, shard_size=world, threshold=0, optimizer_level="level3", comm_fusion=world > 1,
                comm_async=world > 1)
        for i, layer in enumerate(model.layers):
            if i + 1 < len(model.layers):
                layer.set_forward_prefetch_cells([model.layers[i + 1]])
            if i > 0:
                layer.set_backward_prefetch_cells([model.layers[i - 1]])
        hp.init_parameters(model, device=dev, seed=0)
        opt = FusedAdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
        opt.fuse_into_backward(model)       # optimizer update runs inside backward, per wrapped module
        opt.init_state()
        return model, opt

    model, opt = build()
    n_total = args.warmup + args.steps
    host = make_batches(cfg, args, rank, n_total)
    tokens_per_step = world * args.batch_per_gpu * args.seq_len

    def step(tok_dev):
        inp, tgt = tok_dev[:, :-1], tok_dev[:, 1:]
        model.zero_grads()
        loss = model(inp, tgt)
        loss.backward()
        hp.hsdp_sync_stream()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- device-timed loop (inputs resident) --------------------------------
    dev_batches = host.to(dev)
    first_losses = []
    for i in range(args.warmup):
        loss = step(dev_batches[i])
        if args.check and i < 2:
            first_losses.append(loss.item())
    native.check_status()
    barrier()
    launches0 = native.launch_count
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        ev0.record()
        for i in range(args.steps):
            loss = step(dev_batches[args.warmup + i])
        ev1.record()
        barrier()
    launches = native.launch_count - launches0
    ms = max_over_ranks(ev0.elapsed_time(ev1))
    native.check_status()
    last_loss = loss.item()

    # ---- end-to-end loop: H2D of the batch and D2H of the loss every step ----
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h2d = host[0].numel() * host.element_size()
    t0 = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        tok = host[args.warmup + i].to(dev, non_blocking=True)
        loss = step(tok)
        _ = loss.item()
    e1.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(e0.elapsed_time(e1), wall_ms))

    ms_per_step = ms / args.steps
    value = tokens_per_step / (ms_per_step / 1e3)
    e2e_value = tokens_per_step / (e2e_ms / args.steps / 1e3)
    flops = cfg.flops_per_token(args.seq_len) * tokens_per_step / world
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    peak_tflops = peaks.get("bf16_tflops_sustained", 1400.0)
    mfu = flops / (ms_per_step / 1e3) / (peak_tflops * 1e12)
    check = None
    if args.check and world > 1 and len(first_losses) == 2:
        # the same two steps on NCCL collectives + separate kernels: step 0 checks the gathered weights,
        # step 1 the reduced gradients and the sharded optimizer update
        import gc
        from hyper_parallel_b200.core.hsdp.hsdp_scheduler import teardown_hsdp
        teardown_hsdp(model)
        del model, opt, loss
        gc.collect()
        torch.cuda.empty_cache()
        prev = os.environ.get("HPB_FUSED_COMM")
        os.environ["HPB_FUSED_COMM"] = "0"
        try:
            model, opt = build()
            ref_losses = [step(dev_batches[i]).item() for i in range(2)]
            native.check_status()
            diff = max(abs(a - b) / max(abs(b), 1e-6) for a, b in zip(first_losses, ref_losses))
            check = {"loss_fused": first_losses, "loss_nccl": ref_losses, "max_rel_diff": diff, "ok": diff < 2e-3}
        except Exception as e:  # noqa: BLE001  (the benchmark line must still be printed)
            check = {"error": repr(e)[:200], "ok": False}
        finally:
            if prev is None:
                os.environ.pop("HPB_FUSED_COMM", None)
            else:
                os.environ["HPB_FUSED_COMM"] = prev
        barrier()
    from hyper_parallel_b200.utils.logging import MetricsWriter, get_logger
    log = get_logger("hyper_parallel_b200.bench")
    log.info("llama %s x%d: %.1f ms/step device-timed, %.1f ms/step end to end, mfu %.3f", args.model, world,
             ms_per_step, e2e_ms / args.steps, mfu)
    MetricsWriter(args.metrics_jsonl).write(args.steps, tokens_per_s=value, ms_per_step=ms_per_step,
                                            e2e_ms_per_step=e2e_ms / args.steps, mfu=mfu, loss=last_loss,
                                            n_gpus=world, fused_comm=os.environ.get("HPB_FUSED_COMM", "1"),
                                            fused_ag=os.environ.get("HPB_FUSED_AG", "0"),
                                            ride=os.environ.get("HPB_RIDE", "1"), nvls=os.environ.get("HPB_NVLS", "1"))
    if rank == 0:
        print(json.dumps({
            "metric": "train tokens/sec (device-timed, max over ranks)", "value": value,
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (uniform token ids, seed 0; random-init N(0,0.02) weights)",
            "impl": "ours",
            "config": _shared_config(args, cfg.num_layers, cfg.hidden_size, world),
            "mfu_of_measured_sustained_bf16": mfu, "loss": last_loss,
            "clocks": clocks.summary(),
            "e2e": {"value": e2e_value, "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": launches,
            **({"check": check} if check is not None else {}),
        }))
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        try:
            from reference_arm import run_reference
            from reference_configs import run_reference_config
        except Exception as e:  # noqa: BLE001
            if int(os.environ.get("RANK", "0")) == 0:
                print(json.dumps({"impl": "reference", "unavailable": f"reference harness failed to import: {e}"}))
            return
        if args.config == "hsdp":
            run_reference(args)
        else:
            run_reference_config(args, other_config_argv(args, world))
        return
    if args.config != "hsdp":
        sys.path.insert(0, os.path.join(ROOT, "benchmarks"))
        import train_configs
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29571")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        os.environ.setdefault("LOCAL_RANK", "0")
        train_configs.main(other_config_argv(args, world))
        return
    run_ours(args)


if __name__ == "__main__":
    main()
