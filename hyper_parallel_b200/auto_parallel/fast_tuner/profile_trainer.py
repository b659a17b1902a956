"""The trainer that the strategy search launches to profile a candidate.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \\
        -m hyper_parallel_b200.auto_parallel.fast_tuner.profile_trainer --profile-config profile_000.json

It closes the loop that the reference closes with external trainers (TorchTitan / MindFormers /
MindSpeed launched by hyper_parallel/auto_parallel/fast-tuner/fast_tuner/utils/profiling/
profile_launch.py:35-76 and parsed from vendor kernel traces by profile_parser.py:43-800): here the
framework profiles itself.  The candidate written by ``profiling.write_profile_config`` (already
shrunk to the ranks at hand, pp = 1) is built from this package's own model families -- the dense
Llama decoder, or the DeepSeek-V3 MoE decoder when the model has experts -- with a few layers, sharded
with ``hsdp`` over the data-parallel ranks (experts over the expert-parallel group), and stepped a
few times under ``utils.tracing.LayerTimer``.  Rank 0 writes ``<config>.records.jsonl``: one JSON
line per module kind (``dense`` / ``moe`` / ``head`` / ``embed``) and phase (``fwd`` / ``bwd``) with
the mean device time in milliseconds -- the numbers the pipeline balancer needs -- and
``<config>.memory.json`` with the peak allocated bytes.

Runs on CUDA ranks (NCCL) and, for the tests, on CPU ranks (gloo) with tiny shapes.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Optional

import torch
import torch.distributed as dist
from torch import nn


def _classify(name: str, mod: nn.Module) -> Optional[str]:
    base = [c.__name__ for c in type(mod).__mro__]
    if "LlamaBlock" in base:
        return "dense"
    if "DeepSeekBlock" in base:
        return "moe" if getattr(mod, "is_moe", False) else "dense"
    return None


def build_model(model: dict, ep_group, device, layers_dense: int, layers_moe: int):
    """A short stack of the candidate's layer types with the candidate's widths."""
    import hyper_parallel_b200 as hp  # noqa: F401  (registers the package)
    if model.get("expert_num"):
        from hyper_parallel_b200.models.deepseek_v3 import DeepSeekV3, DeepSeekV3Config
        cfg = DeepSeekV3Config(
            vocab_size=model["vocab_size"], hidden_size=model["hidden_size"], num_layers=layers_dense + layers_moe,
            first_k_dense=layers_dense, num_heads=model["num_attention_heads"],
            q_lora_rank=model.get("q_lora_rank") or max(model["hidden_size"] // 4, 16),
            kv_lora_rank=model.get("kv_lora_rank") or max(model["hidden_size"] // 8, 16),
            qk_nope_head_dim=model.get("qk_nope_head_dim", 128), qk_rope_head_dim=model.get("qk_rope_head_dim", 64),
            v_head_dim=model.get("v_head_dim", 128), dense_ffn_size=model["ffn_hidden_size"],
            moe_ffn_size=model.get("moe_ffn_hidden_size") or model["ffn_hidden_size"],
            n_routed_experts=model["expert_num"], n_shared_experts=model.get("shared_expert_num", 0),
            top_k=model.get("num_experts_per_tok", 1), n_group=1, topk_group=1)
        return DeepSeekV3(cfg, ep_group=ep_group, device=device,
                          dtype=torch.bfloat16 if device.type == "cuda" else torch.float32), cfg
    from hyper_parallel_b200.models.llama import Llama, LlamaConfig
    heads = model["num_attention_heads"]
    cfg = LlamaConfig(vocab_size=model["vocab_size"], hidden_size=model["hidden_size"], num_layers=layers_dense,
                      num_heads=heads, num_kv_heads=model.get("num_kv_heads") or heads,
                      head_dim=model["hidden_size"] // heads, ffn_size=model["ffn_hidden_size"])
    return Llama(cfg, device=device, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32), cfg


def run(config_path: str, steps: int = 3, warmup: int = 1, layers: int = 2) -> str:
    with open(config_path) as f:
        cand = json.load(f)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if cuda:
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        device = torch.device("cuda", local)
    else:
        device = torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        dist.init_process_group("nccl" if cuda else "gloo")
    import hyper_parallel_b200 as hp
    from hyper_parallel_b200.collectives import cc
    from hyper_parallel_b200.utils.tracing import LayerTimer

    model_d = cand["model"]
    ep = max(1, min(int(cand.get("ep", 1)), world))
    ep_group = None
    if model_d.get("expert_num") and ep > 1:
        base = rank // ep * ep
        ep_group = cc.group_for_ranks(tuple(range(base, base + ep)))
    n_moe = layers if model_d.get("expert_num") else 0
    n_dense = 1 if n_moe else layers
    torch.manual_seed(0)
    model, cfg = build_model(model_d, ep_group, device, n_dense, n_moe)
    model.init_weights()
    timer = LayerTimer(model, _classify)
    if world > 1:
        for layer in model.layers:
            hp.hsdp(layer, shard_size=world, threshold=0, optimizer_level="level3")
        hp.hsdp(model, shard_size=world, threshold=0, optimizer_level="level3")
    opt = torch.optim.SGD([p for p in model.parameters() if p.requires_grad], lr=1e-3)
    mbs = int(cand.get("mbs", 1))
    seq = int(model_d.get("seq_length", 128))
    g = torch.Generator().manual_seed(rank)
    if cuda:
        torch.cuda.reset_peak_memory_stats(device)
    for it in range(warmup + steps):
        if it == warmup:
            timer.timer.totals.clear()
            timer.timer.counts.clear()
            timer.timer.pending = []
        tok_step = timer.timer.start("step|all|all")
        tok = torch.randint(0, cfg.vocab_size, (mbs, seq + 1), generator=g).to(device)
        if hasattr(model, "zero_grads"):
            model.zero_grads()
        else:
            opt.zero_grad()
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        if world > 1:
            hp.hsdp_sync_stream()
        opt.step()
        timer.timer.stop(tok_step)
    timer.step = steps
    out = config_path.replace(".json", ".records.jsonl")
    if rank == 0:
        if os.path.exists(out):
            os.remove(out)
        timer.dump(out)
        # the head and the embedding are not modules of the model families: their cost is the part of
        # the step that the decoder layers do not account for, split 2:1 between head and embedding
        # and 1:2 between forward and backward
        with open(out) as f:
            recs = [json.loads(l) for l in f if l.strip()]
        step_ms = sum(r["ms"] for r in recs if r["module"] == "step")
        layer_ms = sum(r["ms"] for r in recs if r["module"] in ("dense", "moe"))     # one record per layer and phase
        rest = max(step_ms - layer_ms, 0.0)
        recs = [r for r in recs if r["module"] != "step"]
        for kind, share in (("head", 2.0 / 3.0), ("embed", 1.0 / 3.0)):
            recs.append({"module": kind, "name": kind, "phase": "fwd", "ms": rest * share / 3.0, "step": steps})
            recs.append({"module": kind, "name": kind, "phase": "bwd", "ms": rest * share * 2.0 / 3.0, "step": steps})
        with open(out, "w") as f:
            for r in recs:
                f.write(json.dumps(r) + "\n")
        with open(config_path.replace(".json", ".memory.json"), "w") as f:
            json.dump({"peak_allocated_bytes": int(torch.cuda.max_memory_allocated(device)) if cuda else 0,
                       "layers_dense": n_dense, "layers_moe": n_moe, "records": len(recs)}, f)
    if world > 1:
        dist.barrier()
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--profile-config", required=True)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--layers", type=int, default=2)
    ns = ap.parse_args(argv)
    run(ns.profile_config, ns.steps, ns.warmup, ns.layers)
    if dist.is_initialized():
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
