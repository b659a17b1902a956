"""Reference arm of bench.py: the UNMODIFIED reference package (installed under baseline/_ref)
driving the same Llama architecture, metric and configuration.

Nothing from hyper_parallel_b200 is imported here: the model is written in stock PyTorch
modules (cuBLAS GEMMs, fused SDPA, ``nn.RMSNorm``), sharded with the reference's own
``hsdp(..., optimizer_level="level3")`` public API and stepped with ``torch.optim.AdamW`` on
fp32 master copies (the reference ships no optimizer).
"""
from __future__ import annotations

import json
import math
import os
import subprocess
import sys
import threading
import time

import torch
import torch.nn.functional as F
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

CONFIGS = {
    "llama3_8b": dict(vocab=128256, hidden=4096, layers=32, heads=32, kv_heads=8, head_dim=128,
                      ffn=14336, theta=500000.0),
    "llama2_13b": dict(vocab=32000, hidden=5120, layers=40, heads=40, kv_heads=40, head_dim=128,
                       ffn=13824, theta=10000.0),
    "tiny": dict(vocab=512, hidden=256, layers=2, heads=4, kv_heads=2, head_dim=64, ffn=512,
                 theta=500000.0),
}


def _rope(x, theta):
    # x: [B, S, H, D], rotate-half convention
    B, S, H, D = x.shape
    half = D // 2
    inv = torch.exp2(-math.log2(theta) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32)) / D)
    ang = torch.arange(S, device=x.device, dtype=torch.float32)[:, None] * inv[None, :]
    cs, sn = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1).to(x.dtype)


class Block(nn.Module):
    def __init__(self, c, dtype):
        super().__init__()
        self.c = c
        h, hd = c["hidden"], c["head_dim"]
        self.attn_norm = nn.RMSNorm(h, eps=1e-5, dtype=dtype)
        self.wqkv = nn.Linear(h, (c["heads"] + 2 * c["kv_heads"]) * hd, bias=False, dtype=dtype)
        self.wo = nn.Linear(c["heads"] * hd, h, bias=False, dtype=dtype)
        self.ffn_norm = nn.RMSNorm(h, eps=1e-5, dtype=dtype)
        self.w_gate_up = nn.Linear(h, 2 * c["ffn"], bias=False, dtype=dtype)
        self.w_down = nn.Linear(c["ffn"], h, bias=False, dtype=dtype)

    def forward(self, x):
        c = self.c
        B, S, _ = x.shape
        nh, nkv, hd = c["heads"], c["kv_heads"], c["head_dim"]
        qkv = self.wqkv(self.attn_norm(x))
        q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
        q = _rope(q.view(B, S, nh, hd), c["theta"]).transpose(1, 2)
        k = _rope(k.view(B, S, nkv, hd), c["theta"]).transpose(1, 2)
        v = v.view(B, S, nkv, hd).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=(nh != nkv))
        x = x + self.wo(a.transpose(1, 2).reshape(B, S, nh * hd))
        g, u = self.w_gate_up(self.ffn_norm(x)).chunk(2, dim=-1)
        return x + self.w_down(F.silu(g) * u)


class RefLlama(nn.Module):
    def __init__(self, c, dtype=torch.bfloat16):
        super().__init__()
        self.c = c
        self.embed = nn.Embedding(c["vocab"], c["hidden"], dtype=dtype)
        self.layers = nn.ModuleList(Block(c, dtype) for _ in range(c["layers"]))
        self.final_norm = nn.RMSNorm(c["hidden"], eps=1e-5, dtype=dtype)
        self.lm_head = nn.Linear(c["hidden"], c["vocab"], bias=False, dtype=dtype)

    def forward(self, anchor, tokens, targets):
        # `anchor` is an unused float tensor: the reference's forward pre-hook sets
        # requires_grad on the first positional input, which integer token ids cannot take
        x = self.embed(tokens)
        for layer in self.layers:
            x = layer(x)
        logits = self.lm_head(self.final_norm(x))
        return F.cross_entropy(logits.view(-1, logits.shape[-1]).float(), targets.reshape(-1))


class _Clocks:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, idx):
        self.idx, self.lines, self.proc = idx, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.idx), "-lms", "200"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: [self.lines.append(l) for l in self.proc.stdout], daemon=True)
            self.t.start()
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        return False

    def summary(self):
        import statistics
        sm, mx, reasons = [], [], set()
        for l in self.lines:
            p = [x.strip() for x in l.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for n, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons)}


def bench_config(args, layers, hidden, world):
    """The ``config`` entry of the JSON line; bench.py builds the same dict for its own arm."""
    return {"model": args.model, "layers": layers, "hidden": hidden,
            "global_batch": world * args.batch_per_gpu, "seq_len": args.seq_len,
            "parallelism": f"hsdp level3 full shard x{world}", "optimizer": "AdamW, fp32 master/m/v",
            "l2": "no flush needed: each step streams >100 GB of weights/activations, far above the 126 MB L2"}


def _unavailable(why):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}))


def run_reference(args):
    if not os.path.isdir(os.path.join(REF_DIR, "hyper_parallel")):
        return _unavailable("baseline/_ref is empty: reference package not installed on this machine")
    os.environ.setdefault("HYPER_PARALLEL_PLATFORM", "torch")
    sys.path.insert(0, REF_DIR)
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    try:
        # the reference defaults to "hccl" unless a default group already exists
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        from hyper_parallel import hsdp, hsdp_sync_stream
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference import/init failed: {type(e).__name__}: {e}")

    c = dict(CONFIGS[args.model])
    if args.layers is not None:
        c["layers"] = args.layers

    def build(comm_async, comm_fusion):
        """Model + optimizer + step function for one communication mode of the reference's hsdp()."""
        torch.manual_seed(0)
        model = RefLlama(c).to(dev)
        for p in model.parameters():
            if p.dim() > 1:
                nn.init.normal_(p, 0.0, 0.02)
        kw = dict(shard_size=world, optimizer_level="level3", comm_async=comm_async, comm_fusion=comm_fusion)
        for layer in model.layers:
            hsdp(layer, **kw)
        hsdp(model, **kw)
        for i, layer in enumerate(model.layers):
            if i + 1 < len(model.layers):
                layer.set_forward_prefetch_cells([model.layers[i + 1]])
            if i > 0:
                layer.set_backward_prefetch_cells([model.layers[i - 1]])
        # One optimizer per wrapped module: the fp32 copies of its gradients exist only while that
        # module is stepped (with one optimizer over everything, 4 bytes per parameter of fp32
        # gradients stay alive on top of master / exp_avg / exp_avg_sq, which does not fit one GPU).
        groups = [[p for p in layer.parameters() if p.requires_grad] for layer in model.layers]
        seen = {id(p) for g in groups for p in g}
        groups.append([p for p in model.parameters() if p.requires_grad and id(p) not in seen])
        units = []
        for params in groups:
            masters = [p.detach().float().clone().requires_grad_() for p in params]
            units.append((params, masters, torch.optim.AdamW(masters, lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                                                             weight_decay=0.1, fused=True)))
        anchor = torch.zeros(1, device=dev)

        def step(tok):
            loss = model(anchor, tok[:, :-1], tok[:, 1:])
            loss.backward(torch.ones_like(loss))
            hsdp_sync_stream()
            for params, masters, opt in units:
                for p, m in zip(params, masters):
                    m.grad = p.grad.float().view_as(m) if p.grad is not None else None
                    p.grad = None
                opt.step()
                opt.zero_grad(set_to_none=True)
                with torch.no_grad():
                    torch._foreach_copy_([p.data for p in params],
                                         [m.data.view_as(p.data) for p, m in zip(params, masters)])
            return loss

        return step

    def probe(mode, tok, steps=2):
        """Seconds per step of one mode over a few steps, or None (and the traceback on rank 0's
        stderr and in the directory that ``HPB_LOG_DIR`` names, default ``bench_logs``) when the
        reference raises in that mode."""
        import gc
        import traceback
        try:
            step = build(*mode)
            step(tok)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                step(tok)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / steps
        except Exception:  # noqa: BLE001
            if rank == 0:
                text = traceback.format_exc()
                sys.stderr.write(f"[reference arm] mode comm_async={mode[0]} comm_fusion={mode[1]} failed:\n{text}")
                try:
                    log_dir = os.path.join(os.path.dirname(HERE), os.environ.get("HPB_LOG_DIR", "bench_logs"))
                    os.makedirs(log_dir, exist_ok=True)
                    with open(os.path.join(log_dir,
                                           f"reference_mode_async{int(mode[0])}_fusion{int(mode[1])}_N{world}.txt"),
                              "w") as f:
                        f.write(text)
                except OSError:
                    pass
            dt = None
        step = None
        gc.collect()
        torch.cuda.empty_cache()
        ok = torch.tensor([0.0 if dt is None else 1.0, dt or 0.0], device=dev, dtype=torch.float64)
        if world > 1:
            lo = ok.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN)
            dist.all_reduce(ok, op=dist.ReduceOp.MAX)
            return None if lo[0].item() == 0.0 else ok[1].item()
        return dt

    try:
        # The reference's fastest WORKING communication mode is the baseline: every combination of
        # its comm_async / comm_fusion switches is tried for a few steps first.
        g0 = torch.Generator().manual_seed(12345 + rank)
        tok0 = torch.randint(0, c["vocab"], (args.batch_per_gpu, args.seq_len + 1), generator=g0).to(dev)
        modes = [(True, True), (False, True), (True, False), (False, False)] if world > 1 else [(False, False)]
        tried = {}
        for mode in modes:
            tried[mode] = probe(mode, tok0)
        working = {m: t for m, t in tried.items() if t is not None}
        if not working:
            raise RuntimeError("no communication mode of the reference's hsdp() ran: "
                               + ", ".join(f"async={m[0]} fusion={m[1]}" for m in tried))
        best = min(working, key=working.get)
        step = build(*best)
        mode_note = {f"async={int(m[0])},fusion={int(m[1])}": (None if t is None else round(t * 1e3, 1))
                     for m, t in tried.items()}

        n_total = args.warmup + args.steps
        g = torch.Generator().manual_seed(0 + rank)
        host = torch.randint(0, c["vocab"], (n_total, args.batch_per_gpu, args.seq_len + 1), generator=g,
                             dtype=torch.int64).pin_memory()
        devb = host.to(dev)

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def mx(ms):
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            if world > 1:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            return t.item()

        for i in range(args.warmup):
            step(devb[i])
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with _Clocks(local) as clocks:
            e0.record()
            for i in range(args.steps):
                loss = step(devb[args.warmup + i])
            e1.record()
            barrier()
        ms = mx(e0.elapsed_time(e1))
        last = loss.item()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        f0.record()
        for i in range(args.steps):
            tok = host[args.warmup + i].to(dev, non_blocking=True)
            _ = step(tok).item()
        f1.record()
        barrier()
        e2e_ms = mx(max(f0.elapsed_time(f1), (time.perf_counter() - t0) * 1e3))
    except Exception as e:  # noqa: BLE001
        import traceback
        traceback.print_exc(file=sys.stderr)
        msg = f"reference run failed at N={world}: {type(e).__name__}: {e}"
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass
        return _unavailable(msg)

    toks = world * args.batch_per_gpu * args.seq_len
    if rank == 0:
        print(json.dumps({
            "metric": "train tokens/sec (device-timed, max over ranks)", "value": toks / (ms / args.steps / 1e3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic (uniform token ids, seed 0; random-init N(0,0.02) weights)",
            "impl": "reference",
            "config": bench_config(args, c["layers"], c["hidden"], world),
            "arm": {"sharding": f"reference hsdp(optimizer_level='level3', shard_size={world}, comm_async={best[0]}, "
                                f"comm_fusion={best[1]})",
                    "optimizer": "torch.optim.AdamW(fused) on fp32 master copies, one optimizer per wrapped module",
                    "modes_tried_ms_per_step": mode_note},
            "loss": last, "clocks": clocks.summary(),
            "e2e": {"value": toks / (e2e_ms / args.steps / 1e3), "unit": "tokens/s",
                    "ms_per_step": e2e_ms / args.steps,
                    "h2d_bytes_per_step": host[0].numel() * host.element_size(), "d2h_bytes_per_step": 4},
            "gpu_launches": 0,
        }))
    dist.destroy_process_group()
