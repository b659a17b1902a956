"""Mixture-of-experts building blocks: routing, token permutation, expert-parallel FFN.

``route``                 sigmoid gating with group-limited top-k selection and an aux-free bias
``expert_parallel_ffn``   dispatch (all-to-all) -> grouped SwiGLU expert GEMMs -> combine (all-to-all)

CUDA tensors use the kernels of ``libhpb200.so`` (router top-k kernel, grouped tcgen05 GEMM);
CPU tensors and the gloo test path use the PyTorch formulation below, which is the oracle.
The reference has no MoE / expert-parallel code; its only related primitive is the generic
all-to-all of ``redistribute`` (hyper_parallel/core/tensor_redistribution.py:84-151).
"""
from __future__ import annotations

import ctypes
from typing import List, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..collectives import cc
from . import functional as Fn
from . import native


# ------------------------------------------------------------------ routing --
def route_reference(logits: torch.Tensor, bias: torch.Tensor, top_k: int, n_group: int, topk_group: int,
                    scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``logits[T, E]`` (fp32) -> ``(expert index [T, k] int64, gate weight [T, k] fp32)``."""
    T, E = logits.shape
    scores = torch.sigmoid(logits.float())
    sel = scores + bias.float()[None, :]
    if n_group > 1:
        g = sel.view(T, n_group, E // n_group)
        group_score = g.topk(min(2, E // n_group), dim=-1).values.sum(-1)         # [T, n_group]
        keep = group_score.topk(topk_group, dim=-1).indices
        mask = torch.zeros(T, n_group, dtype=torch.bool, device=logits.device).scatter_(1, keep, True)
        sel = sel.masked_fill(~mask[:, :, None].expand(T, n_group, E // n_group).reshape(T, E), float("-inf"))
    idx = sel.topk(top_k, dim=-1).indices
    w = scores.gather(1, idx)
    w = w / (w.sum(-1, keepdim=True) + 1e-20) * scale
    return idx, w


class _RouteKernel(torch.autograd.Function):
    """Router top-k on the CUDA kernel; the backward (a [T, k]-sized computation) is plain tensor math."""

    @staticmethod
    def forward(ctx, logits, bias, top_k, n_group, topk_group, scale):
        T, E = logits.shape
        logits = logits.contiguous()
        idx = torch.empty((T, top_k), dtype=torch.int64, device=logits.device)
        w = torch.empty((T, top_k), dtype=torch.float32, device=logits.device)
        lib = native.lib()
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.hpb_moe_route.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, cf, vp]
        lib.hpb_moe_route.restype = ci
        rc = lib.hpb_moe_route(logits.data_ptr(), bias.float().contiguous().data_ptr(), idx.data_ptr(),
                               w.data_ptr(), None, T, E, top_k, n_group, topk_group, float(scale),
                               native.stream(logits.device))
        native.check(rc, "hpb_moe_route")
        ctx.save_for_backward(logits, idx)
        ctx.scale = scale
        ctx.mark_non_differentiable(idx)
        return idx, w

    @staticmethod
    def backward(ctx, _gidx, gw):
        logits, idx = ctx.saved_tensors
        sel = torch.sigmoid(logits.gather(1, idx))
        S = sel.sum(-1, keepdim=True) + 1e-20
        gs = ctx.scale * (gw - (gw * sel).sum(-1, keepdim=True) / S) / S
        dl = torch.zeros_like(logits).scatter_(1, idx, gs * sel * (1.0 - sel))
        return dl, None, None, None, None, None


def _kernel_route_ok(E: int, top_k: int, n_group: int) -> bool:
    if E % 32 or E > 512 or top_k > 32 or E % n_group:
        return False
    if n_group > 1:
        vpl, epg = E // 32, E // n_group
        if epg % vpl:
            return False
        lpg = epg // vpl
        if lpg & (lpg - 1) or 32 % lpg:
            return False
    return (E // 32) in (1, 2, 4, 8, 16)


def route(x: torch.Tensor, gate_w: torch.Tensor, bias: torch.Tensor, top_k: int, n_group: int,
          topk_group: int, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Gate GEMM + group-limited top-k.  Gradients flow to ``gate_w`` and ``x`` through the weights."""
    if x.is_cuda and x.dtype == torch.bfloat16:
        logits = Fn.linear(x, gate_w.to(torch.bfloat16)).float()
        if _kernel_route_ok(logits.shape[1], top_k, n_group):
            return _RouteKernel.apply(logits, bias, top_k, n_group, topk_group, scale)
    else:
        logits = F.linear(x.float(), gate_w.float())
    return route_reference(logits, bias, top_k, n_group, topk_group, scale)


# ------------------------------------------------- variable-size all-to-all --
def _all_to_all_v(x: torch.Tensor, in_splits: List[int], out_splits: List[int], group) -> torch.Tensor:
    n = cc.group_size(group)
    out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
    if n == 1:
        out.copy_(x)
        return out
    if dist.get_backend(group) == "gloo":
        ins = [c.contiguous() for c in x.split(in_splits, dim=0)]
        outs = list(out.split(out_splits, dim=0))
        outs = [torch.empty_like(o) for o in outs]
        # gloo has no all_to_all: every rank broadcasts its pieces through all_gather_object-free p2p
        reqs = []
        me = dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group)
        for r in range(n):
            if r == me:
                outs[r].copy_(ins[r])
            else:
                reqs.append(dist.isend(ins[r], dst=ranks[r], group=group))
                reqs.append(dist.irecv(outs[r], src=ranks[r], group=group))
        for q in reqs:
            q.wait()
        return torch.cat(outs, dim=0) if outs else out
    dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
    return out


class _AllToAllV(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        return _all_to_all_v(x, in_splits, out_splits, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all_v(g.contiguous(), ctx.out_splits, ctx.in_splits, ctx.group), None, None, None


def all_to_all_v(x, in_splits, out_splits, group):
    """Differentiable all-to-all with per-rank row counts."""
    return _AllToAllV.apply(x, list(in_splits), list(out_splits), group)


# ------------------------------------------------------------- grouped FFN --
def grouped_swiglu_ffn(x: torch.Tensor, counts: List[int], w_gate_up: torch.Tensor, w_down: torch.Tensor):
    """``x`` rows are grouped by local expert (``counts[e]`` rows each); returns the expert outputs."""
    if x.is_cuda and x.dtype == torch.bfloat16 and native.available():
        from .grouped import grouped_linear
        h = grouped_linear(x, w_gate_up, counts)
        a = Fn.swiglu(h)
        return grouped_linear(a, w_down, counts)
    outs = []
    start = 0
    for e, c in enumerate(counts):
        if c == 0:
            continue
        xe = x[start:start + c]
        gu = F.linear(xe, w_gate_up[e])
        g, u = gu.chunk(2, dim=-1)
        outs.append(F.linear((F.silu(g.float()) * u.float()).to(x.dtype), w_down[e]))
        start += c
    if not outs:
        return x.new_zeros((0, w_down.shape[1]))
    return torch.cat(outs, dim=0)


def expert_parallel_ffn(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor,
                        w_gate_up: torch.Tensor, w_down: torch.Tensor, num_experts: int, ep_group=None):
    """MoE layer body: ``y[t] = sum_k topk_w[t,k] * expert_{topk_idx[t,k]}(x[t])``.

    Experts ``[r * E_local, (r+1) * E_local)`` live on EP rank ``r``.  Steps: sort the (token,
    expert) pairs by expert; exchange per-expert counts; all-to-all the rows to their expert's
    rank; regroup by local expert; grouped SwiGLU FFN; all-to-all back; un-sort; weighted sum.
    """
    T, k = topk_idx.shape
    H = x.shape[-1]
    ep = cc.group_size(ep_group)
    e_local = num_experts // ep
    flat_e = topk_idx.reshape(-1)
    order = torch.argsort(flat_e, stable=True)                 # pair ids sorted by expert
    token_of = order // k
    xs = x.index_select(0, token_of)                           # [T*k, H] rows grouped by expert
    counts = torch.bincount(flat_e, minlength=num_experts)
    if ep > 1:
        send_counts = counts.view(ep, e_local)
        recv_counts = torch.empty_like(send_counts)
        _exchange_counts(recv_counts, send_counts, ep_group)
        in_splits = send_counts.sum(1).tolist()
        out_splits = recv_counts.sum(1).tolist()
        recv = all_to_all_v(xs, in_splits, out_splits, ep_group)           # grouped by (src rank, expert)
        rc = recv_counts.tolist()
        # regroup rows by local expert: order of blocks is (src, e) -> want (e, src)
        blocks = []
        offs = 0
        index = []
        for s in range(ep):
            for e in range(e_local):
                index.append((e, s, offs, rc[s][e]))
                offs += rc[s][e]
        perm = torch.cat([torch.arange(o, o + c, device=x.device) for e, s, o, c in sorted(index) if c > 0]) \
            if offs > 0 else torch.zeros(0, dtype=torch.long, device=x.device)
        grouped = recv.index_select(0, perm)
        local_counts = [sum(rc[s][e] for s in range(ep)) for e in range(e_local)]
        out_grouped = grouped_swiglu_ffn(grouped, local_counts, w_gate_up, w_down)
        inv = torch.empty_like(perm)
        inv[perm] = torch.arange(perm.numel(), device=x.device)
        back = out_grouped.index_select(0, inv)
        ys = all_to_all_v(back, out_splits, in_splits, ep_group)
    else:
        ys = grouped_swiglu_ffn(xs, counts.tolist(), w_gate_up, w_down)
    # un-sort and combine
    w_sorted = topk_w.reshape(-1).index_select(0, order).to(ys.dtype)
    contrib = ys * w_sorted[:, None]
    y = torch.zeros(T, H, dtype=contrib.dtype, device=x.device).index_add_(0, token_of, contrib)
    return y.to(x.dtype)


def _exchange_counts(recv: torch.Tensor, send: torch.Tensor, group) -> None:
    n = cc.group_size(group)
    if dist.get_backend(group) == "gloo":
        gathered = [torch.empty_like(send) for _ in range(n)]
        dist.all_gather(gathered, send.contiguous(), group=group)
        me = dist.get_rank(group)
        for s in range(n):
            recv[s] = gathered[s][me]
        return
    dist.all_to_all_single(recv.view(-1), send.contiguous().view(-1), group=group)
