"""Reference arms of ``bench.py --config {tp_hsdp, moe_ep, pp}``: the UNMODIFIED reference package
(installed under baseline/_ref) driving stock-PyTorch models of the same architectures, through the
reference's own public API:

* ``tp_hsdp``  column / row parallel linears sharded with ``shard_module`` + ``ShardingPlan`` on a
  ``(dp, tp)`` mesh (token-sharded activations between the blocks; the reference resolves the partial
  sum of a row-parallel output with an all-reduce followed by a local slice), ``hsdp`` (level3) over
  the data-parallel axis;
* ``moe_ep``   the reference has no expert parallelism: its ``hsdp`` shards the non-expert parameters
  and the harness itself routes tokens with ``all_to_all_single`` and runs the experts with
  ``torch._grouped_mm`` (library kernels), bf16;
* ``pp``       ``PipelineStage`` + ``ScheduleInterleaved1F1B`` (the reference's GPipe raises and its 1F1B
  is the one-chunk case of the interleaved schedule), tensor parallelism inside a stage through
  ``shard_module`` as above.

Nothing from hyper_parallel_b200 is imported.  Every arm prints the same JSON line as the repo's own
arm with ``"impl": "reference"``; an arm that the reference cannot run prints
``{"impl": "reference", "unavailable": ...}`` with the exception text.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import sys
import time
import traceback

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import nn

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")


def _parse(argv):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--tp", type=int, default=None)
    ap.add_argument("--pp", type=int, default=None)
    ap.add_argument("--vpp", type=int, default=2)
    ap.add_argument("--micro", type=int, default=8)
    ap.add_argument("--schedule", default="1f1b")
    ap.add_argument("--experts", type=int, default=None)
    ap.add_argument("--fp8", type=int, default=0)
    # test hooks: small shapes on CPU ranks
    ap.add_argument("--tiny", type=int, default=0)
    return ap.parse_args(argv)


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:400]}))


def _rope(x, theta):
    B, S, H, D = x.shape
    half = D // 2
    inv = torch.exp2(-math.log2(theta) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32)) / D)
    ang = torch.arange(S, device=x.device, dtype=torch.float32)[:, None] * inv[None, :]
    cs, sn = ang.cos()[None, :, None, :], ang.sin()[None, :, None, :]
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1).to(x.dtype)


class _W(nn.Module):
    """A bias-free linear whose weight the reference shards (``F.linear`` with an explicit ``None`` bias:
    the reference's rule for ``linear`` wants three operands)."""

    def __init__(self, n_out, n_in, dtype, device, std=0.02):
        super().__init__()
        self.weight = nn.Parameter(torch.empty(n_out, n_in, dtype=dtype, device=device).normal_(0.0, std))

    def forward(self, x):
        return F.linear(x, self.weight, None)


# ----------------------------------------------------------------------------------- tp_hsdp / pp --
class _TPBlock(nn.Module):
    """Llama block on one tensor-parallel rank: token-sharded residual stream, column-parallel
    qkv / gate+up, row-parallel out / down, all four through the reference's shard_module."""

    def __init__(self, c, mesh, tp, dtype, device, ref):
        super().__init__()
        self.c, self.mesh, self.tp, self.ref = c, mesh, tp, ref
        h, hd = c["hidden"], c["head_dim"]
        self.attn_norm = nn.RMSNorm(h, eps=1e-5, dtype=dtype, device=device)
        self.ffn_norm = nn.RMSNorm(h, eps=1e-5, dtype=dtype, device=device)
        self.wqkv = self._col(_W((c["heads"] + 2 * c["kv_heads"]) * hd, h, dtype, device))
        self.wo = self._row(_W(h, c["heads"] * hd, dtype, device))
        self.w_gate = self._col(_W(c["ffn"], h, dtype, device))
        self.w_up = self._col(_W(c["ffn"], h, dtype, device))
        self.w_down = self._row(_W(h, c["ffn"], dtype, device))

    def _col(self, m):
        if self.tp == 1:
            return m
        R, S = self.ref["Replicate"], self.ref["Shard"]
        plan = self.ref["ShardingPlan"](plan={"weight": (R(), S(0))}, input_plan={"input": (R(), R())},
                                        output_plan={"output": (R(), S(1))}, return_local_tensor=[""])
        return self.ref["shard_module"](m, device_mesh=self.mesh, sharding_plan=plan)

    def _row(self, m):
        if self.tp == 1:
            return m
        R, S = self.ref["Replicate"], self.ref["Shard"]
        plan = self.ref["ShardingPlan"](plan={"weight": (R(), S(1))}, input_plan={"input": (R(), S(1))},
                                        output_plan={"output": (R(), S(0))}, return_local_tensor=[""])
        return self.ref["shard_module"](m, device_mesh=self.mesh, sharding_plan=plan)

    def _in(self, x, placements):
        if self.tp == 1:
            return x
        return self.ref["DTensor"].from_local(x, self.mesh, placements)

    def forward(self, x, batch, seq):
        """x: [T/tp, h] token shard of [batch*seq, h]."""
        c, tp = self.c, self.tp
        R, S = self.ref["Replicate"], self.ref["Shard"]
        nh, nkv, hd = c["heads"] // tp, c["kv_heads"] // tp, c["head_dim"]
        qkv = self.wqkv(self._in(self.attn_norm(x), (R(), S(0))))               # [T, (nh + 2 nkv) hd / tp]
        qkv = qkv.view(batch, seq, c["heads"] // tp + 2 * (c["kv_heads"] // tp), hd)
        q, k, v = qkv.split([nh, nkv, nkv], dim=2)
        q = _rope(q, c["theta"]).transpose(1, 2)
        k = _rope(k, c["theta"]).transpose(1, 2)
        a = F.scaled_dot_product_attention(q, k, v.transpose(1, 2), is_causal=True, enable_gqa=(nh != nkv))
        a = a.transpose(1, 2).reshape(batch * seq, nh * hd)
        x = x + self.wo(self._in(a, (R(), S(1))))
        hn = self._in(self.ffn_norm(x), (R(), S(0)))
        act = F.silu(self.w_gate(hn)) * self.w_up(hn)
        return x + self.w_down(self._in(act, (R(), S(1))))


def _ref_api():
    os.environ.setdefault("HYPER_PARALLEL_PLATFORM", "torch")
    if REF_DIR not in sys.path:
        sys.path.insert(0, REF_DIR)
    import hyper_parallel as hpr
    from hyper_parallel.core.placement_types import Replicate, Shard
    from hyper_parallel.core.shard.api import shard_module
    from hyper_parallel.core.shard.sharding_plan import ShardingPlan
    return {"hp": hpr, "Replicate": Replicate, "Shard": Shard, "shard_module": shard_module,
            "ShardingPlan": ShardingPlan, "DTensor": hpr.DTensor, "init_device_mesh": hpr.init_device_mesh}


LLAMA = {
    "llama2_13b": dict(vocab=32000, hidden=5120, layers=40, heads=40, kv_heads=40, head_dim=128, ffn=13824, theta=10000.0),
    "llama3_8b": dict(vocab=128256, hidden=4096, layers=32, heads=32, kv_heads=8, head_dim=128, ffn=14336, theta=500000.0),
    "tiny": dict(vocab=256, hidden=64, layers=4, heads=4, kv_heads=4, head_dim=16, ffn=128, theta=10000.0),
}


def _local(p):
    return p._local_tensor if hasattr(p, "_local_tensor") else p


class _Units:
    """fp32 master copies + one fused AdamW per wrapped module (the reference ships no optimizer)."""

    def __init__(self, modules, root, fused):
        groups = [[p for p in m.parameters() if p.requires_grad] for m in modules]
        seen = {id(p) for g in groups for p in g}
        groups.append([p for p in root.parameters() if p.requires_grad and id(p) not in seen])
        self.units = []
        for params in groups:
            if not params:
                continue
            masters = [_local(p).detach().float().clone().requires_grad_() for p in params]
            self.units.append((params, masters, torch.optim.AdamW(masters, lr=3e-4, betas=(0.9, 0.95), eps=1e-8,
                                                                  weight_decay=0.1, fused=fused)))

    def step(self):
        for params, masters, opt in self.units:
            for p, m in zip(params, masters):
                g = _local(p).grad if _local(p).grad is not None else p.grad
                g = _local(g) if g is not None else None
                m.grad = g.float().reshape(m.shape) if (g is not None and g.numel() == m.numel()) else None
                _local(p).grad = None
                if p is not _local(p):
                    p.grad = None
            opt.step()
            opt.zero_grad(set_to_none=True)
            with torch.no_grad():
                for p, m in zip(params, masters):
                    if _local(p).data.numel() == m.numel():
                        _local(p).data.copy_(m.data.view_as(_local(p).data))


class _RefTPLlama(nn.Module):
    def __init__(self, c, mesh, tp, dtype, device, ref, first=0, count=None, with_embed=True, with_head=True):
        super().__init__()
        self.c, self.tp = c, tp
        count = c["layers"] if count is None else count
        self.embed = nn.Embedding(c["vocab"], c["hidden"], dtype=dtype, device=device) if with_embed else None
        self.layers = nn.ModuleList(_TPBlock(c, mesh, tp, dtype, device, ref) for _ in range(first, first + count))
        self.final_norm = nn.RMSNorm(c["hidden"], eps=1e-5, dtype=dtype, device=device) if with_head else None
        self.lm_head = nn.Linear(c["hidden"], c["vocab"], bias=False, dtype=dtype, device=device) if with_head else None

    def forward(self, anchor, x, targets, tp_rank, batch, seq):
        """x: token ids [batch, seq] (first stage) or the token-sharded hidden state; targets [batch, seq]."""
        T = batch * seq
        lo, hi = tp_rank * (T // self.tp), (tp_rank + 1) * (T // self.tp)
        if self.embed is not None:
            x = self.embed(x.reshape(-1)[lo:hi])
        for layer in self.layers:
            x = layer(x, batch, seq)
        if self.lm_head is None:
            return x
        logits = self.lm_head(self.final_norm(x))
        return F.cross_entropy(logits.float(), targets.reshape(-1)[lo:hi]) / self.tp


def _timed(step, args, dev, world, host, to_dev):
    def barrier():
        if world > 1:
            dist.barrier()
        if dev.type == "cuda":
            torch.cuda.synchronize()

    def mx(v):
        t = torch.tensor([v], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()
    devb = to_dev(host)
    for i in range(args.warmup):
        step(devb[i])
    barrier()
    cuda = dev.type == "cuda"
    t0 = time.perf_counter()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    for i in range(args.steps):
        loss = step(devb[args.warmup + i])
    if cuda:
        e1.record()
    barrier()
    ms = mx(e0.elapsed_time(e1) if cuda else (time.perf_counter() - t0) * 1e3) / args.steps
    last = float(loss.detach()) if loss is not None else 0.0
    t0 = time.perf_counter()
    for i in range(args.steps):
        tok = to_dev(host[args.warmup + i])
        out = step(tok)
        _ = float(out.detach()) if out is not None else 0.0
    barrier()
    e2e = mx((time.perf_counter() - t0) * 1e3) / args.steps
    return ms, e2e, last


def _emit(args, world, cfg, arm, tokens, ms, e2e, loss, h2d):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({
            "metric": "train tokens/sec (device-timed, max over ranks)", "value": tokens / (ms / 1e3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "impl": "reference",
            "data": "synthetic (uniform token ids, seed 0; random-init weights)", "config": cfg, "arm": arm,
            "loss": loss, "e2e": {"value": tokens / (e2e / 1e3), "unit": "tokens/s", "ms_per_step": e2e,
                                  "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4},
            "gpu_launches": 0}))


def run_tp_hsdp(args, ref, rank, world, dev, dtype):
    tp = args.tp or min(4, world)
    dp = world // tp
    c = dict(LLAMA["tiny" if args.tiny else "llama2_13b"])
    if args.layers:
        c["layers"] = args.layers
    mesh = ref["init_device_mesh"](device_type="npu" if dev.type == "cuda" else "cpu", mesh_shape=(dp, tp),
                                   mesh_dim_names=("dp", "tp"))
    torch.manual_seed(0)
    model = _RefTPLlama(c, mesh, tp, dtype, dev, ref)
    hsdp, sync = ref["hp"].hsdp, ref["hp"].hsdp_sync_stream
    if dp > 1:
        for layer in model.layers:
            hsdp(layer, shard_size=dp, optimizer_level="level3")
        hsdp(model, shard_size=dp, optimizer_level="level3")
    units = _Units(list(model.layers), model, fused=dev.type == "cuda")
    anchor = torch.zeros(1, device=dev)
    tp_rank, dp_rank = rank % tp, rank // tp
    g = torch.Generator().manual_seed(dp_rank)
    host = torch.randint(0, c["vocab"], (args.warmup + args.steps, args.batch, args.seq_len + 1), generator=g)
    if dev.type == "cuda":
        host = host.pin_memory()

    def step(tok):
        loss = model(anchor, tok[:, :-1], tok[:, 1:], tp_rank, args.batch, args.seq_len)
        loss.backward(torch.ones_like(loss))
        sync()
        units.step()
        return loss

    ms, e2e, last = _timed(step, args, dev, world, host, lambda t: t.to(dev, non_blocking=True))
    cfg = {"model": "llama2_13b", "layers": c["layers"], "parallelism": f"tp{tp}(+sp) x hsdp{dp} level3",
           "global_batch": dp * args.batch, "seq_len": args.seq_len}
    arm = {"sharding": "reference shard_module (column / row parallel linears, token-sharded activations; partial "
                       "sums resolved by all-reduce + slice) + hsdp(optimizer_level='level3') over dp",
           "optimizer": "torch.optim.AdamW on fp32 master copies"}
    _emit(args, world, cfg, arm, dp * args.batch * args.seq_len, ms, e2e, last, host[0].numel() * host.element_size())


# ------------------------------------------------------------------------------------------ pp --
def run_pp(args, ref, rank, world, dev, dtype):
    """Llama-3-8B over pp stages x tp ranks with the reference's PipelineStage + ScheduleInterleaved1F1B
    (``--schedule 1f1b``: one chunk per rank; ``vpp``: ``--vpp`` chunks; the reference's GPipe raises)."""
    if args.schedule == "gpipe":
        raise RuntimeError("the reference's ScheduleGPipe raises AttributeError ('stage' is not defined): not runnable")
    tp = args.tp or 1
    pp = args.pp or world // tp
    if tp > 1 and os.environ.get("REF_PP_TP", "0") != "1":
        # Observed on 4 B200 (PP=2 x TP=2): the run never finished its first step and was ended by the
        # command's time limit.  The reference builds the tensor-parallel mesh of a stage with
        # collective new_group calls whose rank lists differ from stage to stage, so the ranks of
        # different stages wait for each other in group creation.  The arm does not run this again.
        raise RuntimeError("PipelineStage with shard_module inside the stages (PP x TP) does not complete on CUDA "
                           "ranks: per-stage tensor-parallel meshes issue unmatched collective new_group calls "
                           "(hang observed at PP=2 x TP=2 on 4 GPUs); pipeline-only runs (tp = 1) work")
    chunks = args.vpp if args.schedule == "vpp" else 1
    c = dict(LLAMA["tiny" if args.tiny else "llama3_8b"])
    if args.layers:
        c["layers"] = args.layers
    n_virtual = pp * chunks
    per = c["layers"] // n_virtual
    stage_rank, tp_rank = rank // tp, rank % tp
    S, B = args.seq_len, args.batch
    mesh = None
    if tp > 1:
        # every rank builds the meshes of ALL stages, in the same order: the reference creates the
        # process groups of a mesh with collective new_group calls, so ranks that built only their own
        # stage's mesh would issue different sequences of them
        for s_ in range(pp):
            try:
                m_ = ref["init_device_mesh"](device_type="npu" if dev.type == "cuda" else "cpu", mesh_shape=(1, tp),
                                             mesh_dim_names=("dp", "tp"), rank_list=list(range(s_ * tp, s_ * tp + tp)))
            except Exception:  # noqa: BLE001  (a mesh this rank is not part of may refuse to build)
                if s_ == stage_rank:
                    raise
                m_ = None
            if s_ == stage_rank:
                mesh = m_
    torch.manual_seed(0)

    class Chunk(nn.Module):
        def __init__(self, v):
            super().__init__()
            self.first, self.last = v == 0, v == n_virtual - 1
            self.m = _RefTPLlama(c, mesh, tp, dtype, dev, ref, first=v * per, count=per, with_embed=self.first,
                                 with_head=self.last)
            self.targets = []

        def forward(self, x):
            if self.first:
                x = x[:, :-1]
            tgt = self.targets.pop(0) if self.last else None
            out = self.m(None, x, tgt, tp_rank, B, S)
            return out / args.micro if self.last else out

    idx = [stage_rank + k * pp for k in range(chunks)]
    mods = [Chunk(v) for v in idx]
    PipelineStage, Sched = ref["hp"].PipelineStage, ref["hp"].ScheduleInterleaved1F1B
    group = None
    stages = [PipelineStage(m, v, n_virtual, dev) for m, v in zip(mods, idx)]
    sched = Sched(stages, args.micro)
    units = _Units(mods, nn.ModuleList(mods), fused=dev.type == "cuda")
    g = torch.Generator().manual_seed(0)
    host = torch.randint(0, c["vocab"], (args.warmup + args.steps, B * args.micro, S + 1), generator=g)
    if dev.type == "cuda":
        host = host.pin_memory()
    last_mod = mods[-1] if mods[-1].last else None

    def step(tok):
        if last_mod is not None:
            last_mod.targets = list(tok[:, 1:].chunk(args.micro))
        # The reference's stage re-uses its receive descriptors of the previous run() through a branch
        # that reads an undefined variable (core/pipeline_parallel/stage.py:284-286), so a second
        # run() on the same objects raises; its own tests call run() once.  The harness empties those
        # two caches between steps (attributes of the stage objects; no reference file is touched).
        for st in stages:
            for name in ("grad_recv_info", "args_recv_info"):
                d = getattr(st, name, None)
                if isinstance(d, dict):
                    d.clear()
        out = sched.run(tok) if stage_rank == 0 else sched.run()
        units.step()
        if last_mod is not None and out:
            return torch.stack([o.detach().float().reshape(()) for o in out]).sum()
        return torch.zeros((), device=dev)

    ms, e2e, last = _timed(step, args, dev, world, host, lambda t: t.to(dev, non_blocking=True))
    cfg = {"model": "llama3_8b", "layers": c["layers"],
           "parallelism": f"pp{pp} x tp{tp} {args.schedule}" + (f" x{chunks} chunks" if chunks > 1 else ""),
           "micro_batches": args.micro, "global_batch": B * args.micro, "seq_len": S}
    arm = {"schedule": "reference PipelineStage + ScheduleInterleaved1F1B", "tp": "reference shard_module" if tp > 1 else "none",
           "optimizer": "torch.optim.AdamW on fp32 master copies"}
    _emit(args, world, cfg, arm, B * args.micro * S, ms, e2e, last, host[0].numel() * host.element_size())


# -------------------------------------------------------------------------------------- moe_ep --
class _RefMLA(nn.Module):
    def __init__(self, c, dtype, dev):
        super().__init__()
        self.c = c
        h, nh = c["hidden"], c["heads"]
        qk = c["nope"] + c["rope"]
        kw = dict(bias=False, dtype=dtype, device=dev)
        self.wq_a, self.q_norm = nn.Linear(h, c["q_lora"], **kw), nn.RMSNorm(c["q_lora"], eps=1e-6, dtype=dtype, device=dev)
        self.wq_b = nn.Linear(c["q_lora"], nh * qk, **kw)
        self.wkv_a = nn.Linear(h, c["kv_lora"] + c["rope"], **kw)
        self.kv_norm = nn.RMSNorm(c["kv_lora"], eps=1e-6, dtype=dtype, device=dev)
        self.wkv_b = nn.Linear(c["kv_lora"], nh * (c["nope"] + c["v"]), **kw)
        self.wo = nn.Linear(nh * c["v"], h, **kw)

    def forward(self, x, B, S):
        c = self.c
        nh, dn, dr, dv = c["heads"], c["nope"], c["rope"], c["v"]
        q = self.wq_b(self.q_norm(self.wq_a(x))).view(B, S, nh, dn + dr)
        q = torch.cat([q[..., :dn], _rope(q[..., dn:], 10000.0)], dim=-1)
        kv_a = self.wkv_a(x)
        k_rope = _rope(kv_a[..., c["kv_lora"]:].view(B, S, 1, dr), 10000.0)
        kv = self.wkv_b(self.kv_norm(kv_a[..., :c["kv_lora"]])).view(B, S, nh, dn + dv)
        k = torch.cat([kv[..., :dn], k_rope.expand(B, S, nh, dr)], dim=-1)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), kv[..., dn:].transpose(1, 2), is_causal=True)
        return self.wo(a.transpose(1, 2).reshape(B * S, nh * dv))


class _RefFFN(nn.Module):
    def __init__(self, h, f, dtype, dev):
        super().__init__()
        self.w_gate_up = nn.Linear(h, 2 * f, bias=False, dtype=dtype, device=dev)
        self.w_down = nn.Linear(f, h, bias=False, dtype=dtype, device=dev)

    def forward(self, x):
        g, u = self.w_gate_up(x).chunk(2, dim=-1)
        return self.w_down(F.silu(g) * u)


class _RefMoE(nn.Module):
    """Sigmoid group-limited top-k routing; tokens to their experts' ranks with all_to_all_single;
    experts with torch._grouped_mm (a python loop when that is unavailable)."""

    def __init__(self, c, world, rank, dtype, dev):
        super().__init__()
        self.c, self.world, self.rank = c, world, rank
        E, h, f = c["experts"], c["hidden"], c["moe_ffn"]
        self.El = E // world
        self.gate = nn.Parameter(torch.empty(E, h, dtype=torch.float32, device=dev).normal_(0.0, 0.006))
        self.w_gate_up = nn.Parameter(torch.empty(self.El, h, 2 * f, dtype=dtype, device=dev).normal_(0.0, 0.006))
        self.w_down = nn.Parameter(torch.empty(self.El, f, h, dtype=dtype, device=dev).normal_(0.0, 0.006))
        self.w_gate_up._ep_owned = True
        self.w_down._ep_owned = True
        self.shared = _RefFFN(h, f, dtype, dev)

    def _experts(self, x, counts):
        """x grouped by local expert (counts[e] rows each)."""
        offs = torch.cumsum(counts, 0).to(torch.int32)
        if hasattr(torch, "_grouped_mm") and x.is_cuda:
            h = torch._grouped_mm(x, self.w_gate_up, offs=offs)
            g, u = h.chunk(2, dim=-1)
            return torch._grouped_mm((F.silu(g) * u).contiguous(), self.w_down, offs=offs)
        out, lo = [], 0
        for e, n in enumerate(counts.tolist()):
            xe = x[lo:lo + n]
            g, u = (xe @ self.w_gate_up[e]).chunk(2, dim=-1)
            out.append((F.silu(g) * u) @ self.w_down[e])
            lo += n
        return torch.cat(out) if out else x.new_zeros(0, x.shape[1])

    def forward(self, x):
        c = self.c
        T, k, E = x.shape[0], c["top_k"], c["experts"]
        s = torch.sigmoid(x.float() @ self.gate.t())
        G = c["n_group"]
        gs = s.view(T, G, E // G).topk(2, dim=-1).values.sum(-1)
        keep = torch.zeros_like(gs).scatter_(1, gs.topk(c["topk_group"], dim=-1).indices, 1.0)
        masked = (s.view(T, G, E // G) * keep[..., None]).view(T, E)
        idx = masked.topk(k, dim=-1).indices
        w = s.gather(1, idx)
        w = (w / w.sum(-1, keepdim=True) * 2.5).to(x.dtype)
        flat = idx.reshape(-1)
        order = torch.argsort(flat, stable=True)
        xs = x[order // k]
        counts = torch.bincount(flat, minlength=E)
        if self.world > 1:
            recv_counts = torch.empty_like(counts)
            dist.all_to_all_single(recv_counts, counts)
            send = counts.view(self.world, self.El).sum(1).tolist()
            recv = recv_counts.view(self.world, self.El).sum(1).tolist()
            xr = torch.empty(sum(recv), x.shape[1], dtype=x.dtype, device=x.device)
            xr = _A2A.apply(xs, send, recv)
            rc = recv_counts.view(self.world, self.El)
            # rows arrive grouped by source then expert: regroup by expert
            src_off = torch.cumsum(torch.tensor([0] + recv[:-1], device=x.device), 0)
            pos = []
            for e in range(self.El):
                for s_ in range(self.world):
                    start = src_off[s_] + rc[s_, :e].sum()
                    pos.append(torch.arange(int(rc[s_, e]), device=x.device) + start)
            perm = torch.cat(pos) if pos else torch.zeros(0, dtype=torch.long, device=x.device)
            ye = self._experts(xr[perm], rc.sum(0))
            back = torch.empty_like(ye)
            back[perm] = ye
            ys = _A2A.apply(back, recv, send)
        else:
            ys = self._experts(xs, counts)
        y = torch.zeros_like(x)
        y.index_add_(0, order // k, ys * w.reshape(-1)[order][:, None])
        return y + self.shared(x)


class _A2A(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, send, recv):
        ctx.send, ctx.recv = send, recv
        out = torch.empty(sum(recv), x.shape[1], dtype=x.dtype, device=x.device)
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=recv, input_split_sizes=send)
        return out

    @staticmethod
    def backward(ctx, g):
        out = torch.empty(sum(ctx.send), g.shape[1], dtype=g.dtype, device=g.device)
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.send, input_split_sizes=ctx.recv)
        return out, None, None


class _RefDSBlock(nn.Module):
    def __init__(self, c, moe, world, rank, dtype, dev):
        super().__init__()
        self.attn_norm = nn.RMSNorm(c["hidden"], eps=1e-6, dtype=dtype, device=dev)
        self.ffn_norm = nn.RMSNorm(c["hidden"], eps=1e-6, dtype=dtype, device=dev)
        self.attn = _RefMLA(c, dtype, dev)
        self.ffn = _RefMoE(c, world, rank, dtype, dev) if moe else _RefFFN(c["hidden"], c["dense_ffn"], dtype, dev)

    def forward(self, x, B, S):
        x = x + self.attn(self.attn_norm(x), B, S)
        return x + self.ffn(self.ffn_norm(x))


class _RefDeepSeek(nn.Module):
    def __init__(self, c, world, rank, dtype, dev):
        super().__init__()
        self.embed = nn.Embedding(c["vocab"], c["hidden"], dtype=dtype, device=dev)
        self.layers = nn.ModuleList(_RefDSBlock(c, i >= c["first_dense"], world, rank, dtype, dev) for i in range(c["layers"]))
        self.final_norm = nn.RMSNorm(c["hidden"], eps=1e-6, dtype=dtype, device=dev)
        self.lm_head = nn.Linear(c["hidden"], c["vocab"], bias=False, dtype=dtype, device=dev)

    def forward(self, anchor, tok, tgt):
        B, S = tok.shape
        x = self.embed(tok.reshape(-1))
        for layer in self.layers:
            x = layer(x, B, S)
        return F.cross_entropy(self.lm_head(self.final_norm(x)).float(), tgt.reshape(-1))


DEEPSEEK = dict(vocab=129280, hidden=7168, layers=4, first_dense=1, heads=128, q_lora=1536, kv_lora=512, nope=128,
                rope=64, v=128, dense_ffn=18432, moe_ffn=2048, experts=256, top_k=8, n_group=8, topk_group=4)
DEEPSEEK_TINY = dict(vocab=256, hidden=64, layers=2, first_dense=1, heads=4, q_lora=32, kv_lora=16, nope=16, rope=8,
                     v=16, dense_ffn=128, moe_ffn=32, experts=8, top_k=2, n_group=2, topk_group=1)


def run_moe_ep(args, ref, rank, world, dev, dtype):
    c = dict(DEEPSEEK_TINY if args.tiny else DEEPSEEK)
    if args.layers:
        c["layers"] = args.layers
    if args.experts:
        c["experts"] = args.experts
    torch.manual_seed(0)
    model = _RefDeepSeek(c, world, rank, dtype, dev)
    hsdp, sync = ref["hp"].hsdp, ref["hp"].hsdp_sync_stream
    if world > 1 and os.environ.get("REF_NO_HSDP", "0") != "1":
        # the expert weights are owned by their rank: kept away from hsdp by wrapping only the other
        # sub-modules (the reference's hsdp takes every parameter of the cell it is given)
        for layer in model.layers:
            hsdp(layer.attn, shard_size=world, optimizer_level="level3", grad_scale=1.0 / world)
            if isinstance(layer.ffn, _RefMoE):
                hsdp(layer.ffn.shared, shard_size=world, optimizer_level="level3", grad_scale=1.0 / world)
            else:
                hsdp(layer.ffn, shard_size=world, optimizer_level="level3", grad_scale=1.0 / world)
        hsdp(model.lm_head, shard_size=world, optimizer_level="level3", grad_scale=1.0 / world)
        # (the embedding stays replicated: the reference's forward hook marks the first positional input
        # as requiring a gradient, which integer token ids cannot; its gradient is all-reduced below)
    units = _Units(list(model.layers), model, fused=dev.type == "cuda")
    small = [p for n, p in model.named_parameters()
             if ("norm" in n or n.endswith("gate") or n.startswith("embed")) and p.requires_grad]
    anchor = torch.zeros(1, device=dev)
    g = torch.Generator().manual_seed(rank)
    host = torch.randint(0, c["vocab"], (args.warmup + args.steps, args.batch, args.seq_len + 1), generator=g)
    if dev.type == "cuda":
        host = host.pin_memory()

    def step(tok):
        loss = model(anchor, tok[:, :-1], tok[:, 1:])
        loss.backward()
        sync()
        if world > 1:               # norm weights and router gates: replicated, plain all-reduce
            for p in small:
                if p.grad is not None:
                    dist.all_reduce(p.grad)
                    p.grad.div_(world)
        units.step()
        return loss

    ms, e2e, last = _timed(step, args, dev, world, host, lambda t: t.to(dev, non_blocking=True))
    cfg = {"model": "deepseek_v3", "layers": c["layers"], "experts": c["experts"],
           "parallelism": f"ep{world} + hsdp level3 x{world} on the non-expert parameters",
           "global_batch": world * args.batch, "seq_len": args.seq_len, "precision": "bf16"}
    arm = {"sharding": "reference hsdp(level3) on the attention / dense / shared-expert / embedding parameters",
           "experts": "all_to_all_single + torch._grouped_mm in the harness (the reference has no expert parallelism, no fp8)",
           "optimizer": "torch.optim.AdamW on fp32 master copies"}
    _emit(args, world, cfg, arm, world * args.batch * args.seq_len, ms, e2e, last,
          host[0].numel() * host.element_size())


def run_reference_config(bench_args, argv):
    """Entry point used by ``bench.py --impl reference --config X``."""
    args = _parse(argv)
    if not os.path.isdir(os.path.join(REF_DIR, "hyper_parallel")):
        return _unavailable("baseline/_ref is empty: reference package not installed on this machine")
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29531")
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    dtype = torch.bfloat16 if cuda else torch.float32
    try:
        if not dist.is_initialized():
            if cuda:
                dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
            else:
                dist.init_process_group("gloo", rank=rank, world_size=world)
        ref = _ref_api()
        {"tp_hsdp": run_tp_hsdp, "moe_ep": run_moe_ep, "pp": run_pp}[args.config](args, ref, rank, world, dev, dtype)
    except Exception as e:  # noqa: BLE001
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"reference run of config {args.config} failed at N={world}: {type(e).__name__}: {e}")
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:  # noqa: BLE001
                pass


if __name__ == "__main__":
    run_reference_config(None, sys.argv[1:])
