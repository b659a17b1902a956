"""1-D tensor parallelism with sequence-parallel activations (Megatron-style), as autograd functions.

The reference expresses this declaratively (``shard_module`` + layout rules: a column-sharded
weight gives a sharded output, a row-sharded weight gives ``Partial`` that ``redistribute`` turns
into an all-reduce / reduce-scatter, hyper_parallel/core/shard/ops/parallel_matmul.py:22-79,
hyper_parallel/core/tensor_redistribution.py:233-321); that path exists in this framework too
(``core/shard``).  The functions here are the *performance* path for the model zoo: they hold the
two collective+GEMM pairs of a transformer block as single operations, so that they can be
served either by NCCL + the tcgen05 GEMM (``HPB_FUSED_TP=0``, the measured baseline) or by the
fused kernels that move the activation panels over NVLink peer memory from inside the GEMM.

Activations between blocks are sharded along the token dimension (``[T / tp, H]``):

``column_parallel_linear``  all-gather(x) -> x W_shard^T            (qkv, gate_up, lm_head)
``row_parallel_linear``     a W_shard^T -> reduce-scatter over tokens (wo, down)
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..collectives import cc
from ..ops import functional as Fn


def _fused_enabled() -> bool:
    return os.environ.get("HPB_FUSED_TP", "1") != "0"


def _gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    n = cc.group_size(group)
    if n == 1:
        return x
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    cc.all_gather_into(out, x.contiguous(), group)
    return out


def _scatter_sum_tokens(x: torch.Tensor, group) -> torch.Tensor:
    n = cc.group_size(group)
    if n == 1:
        return x
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    cc.reduce_scatter_into(out, x.contiguous(), group, "sum")
    return out


def _workspace(group, x: torch.Tensor, shard_rows: int, k: int, n_out: int):
    """Symmetric-memory workspace of the fused kernels, or ``None`` when they do not apply.  It is
    sized for the forward product and for the two backward products of the same layer (which gather
    / scatter along the other matrix dimension), so that it never has to grow inside a step."""
    n = cc.group_size(group)
    if n == 1 or n > 8 or not _fused_enabled() or not x.is_cuda or x.dtype != torch.bfloat16:
        return None
    if cc.get_backend(group) != "nccl" or (k % 8) or (n_out % 8) or (shard_rows * k) % 8:
        return None
    from .tp_fused import TPWorkspace
    wide = max(k, n_out)
    return TPWorkspace.get(group, shard_rows * wide * 2, n * shard_rows * wide * 2)


def _mm(a, b, **kw):
    """GEMM on the tcgen05 kernel for bf16 CUDA tensors, PyTorch otherwise (CPU tests)."""
    return Fn.gemm(a, b, **kw)


class _ColumnParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_shard, w, group, symm):
        ctx.group, ctx.symm = group, symm
        ctx.save_for_backward(x_shard, w)
        ws = _workspace(group, x_shard, x_shard.shape[0], x_shard.shape[1], w.shape[0])
        if ws is not None:
            # one kernel: peers' token panels are pulled over NVLink while the first panels multiply
            return ws.ag_gemm(x_shard.contiguous(), w.contiguous())
        x = _gather_tokens(x_shard, group)
        y = torch.empty((x.shape[0], w.shape[0]), dtype=x.dtype, device=x.device)
        if x.is_cuda and x.dtype == torch.bfloat16:
            _mm(x, w, out=y)
        else:
            y = x @ w.t()
        return y

    @staticmethod
    def backward(ctx, dy):
        x_shard, w = ctx.saved_tensors
        group = ctx.group
        dy = dy.contiguous()
        dx = dw = None
        ws = _workspace(group, x_shard, x_shard.shape[0], x_shard.shape[1], w.shape[0])
        if ws is not None and dy.shape[0] == x_shard.shape[0] * ws.n:
            # fused backward: dx = reduce-scatter(dy W) inside the GEMM epilogue (the weight shard is
            # transposed once so that the kernel sees a K-major operand); the token shards are
            # re-gathered by peer pulls for the weight-gradient product
            if ctx.needs_input_grad[0]:
                dx = ws.gemm_rs(dy, w.t().contiguous())
            x = ws.gather(x_shard.contiguous()) if ctx.needs_input_grad[1] else None
        else:
            x = _gather_tokens(x_shard, group)             # re-gather instead of keeping the full activation
            if ctx.needs_input_grad[0]:
                if dy.is_cuda and dy.dtype == torch.bfloat16:
                    dx_full = _mm(dy, w, b_mn=True)
                else:
                    dx_full = dy @ w
                dx = _scatter_sum_tokens(dx_full, group)
        if ctx.needs_input_grad[1]:
            if ctx.symm is not None and dy.is_cuda:
                buf, i = ctx.symm
                view, acc = buf.wgrad_target(i)
                _mm(dy, x, a_mn=True, b_mn=True, out=view, accumulate=acc)
                if buf.mark_ready(i):
                    buf.on_all_ready()
            elif dy.is_cuda and dy.dtype == torch.bfloat16:
                dw = _mm(dy, x, a_mn=True, b_mn=True)
            else:
                dw = dy.t() @ x
        return dx, dw, None, None


class _RowParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, w, group, symm):
        ctx.group, ctx.symm = group, symm
        ctx.save_for_backward(a, w)
        n = cc.group_size(group)
        ws = _workspace(group, a, a.shape[0] // max(n, 1), a.shape[1], w.shape[0]) if a.shape[0] % max(n, 1) == 0 else None
        if ws is not None:
            # one kernel: partial tiles go straight into the owner's receive area, then are summed
            return ws.gemm_rs(a.contiguous(), w.contiguous())
        if a.is_cuda and a.dtype == torch.bfloat16:
            y = _mm(a, w)
        else:
            y = a @ w.t()
        return _scatter_sum_tokens(y, group)

    @staticmethod
    def backward(ctx, dy_shard):
        a, w = ctx.saved_tensors
        da = dw = None
        n = cc.group_size(ctx.group)
        ws = _workspace(ctx.group, a, a.shape[0] // max(n, 1), a.shape[1], w.shape[0]) \
            if a.shape[0] % max(n, 1) == 0 else None
        if ws is not None:
            # fused backward: da = all-gather(dy) W inside one kernel (transposed weight shard as the
            # K-major operand); the gathered dy stays in the workspace's staging matrix and feeds the
            # weight-gradient product directly
            dy_shard = dy_shard.contiguous()
            da = ws.ag_gemm(dy_shard, w.t().contiguous())
            dy = ws.gathered(dy_shard.shape[0] * n, dy_shard.shape[1])
            cuda = True
        else:
            dy = _gather_tokens(dy_shard.contiguous(), ctx.group)
            cuda = dy.is_cuda and dy.dtype == torch.bfloat16
            if ctx.needs_input_grad[0]:
                da = _mm(dy, w, b_mn=True) if cuda else dy @ w
        if ctx.needs_input_grad[1]:
            if ctx.symm is not None and cuda:
                buf, i = ctx.symm
                view, acc = buf.wgrad_target(i)
                _mm(dy, a, a_mn=True, b_mn=True, out=view, accumulate=acc)
                if buf.mark_ready(i):
                    buf.on_all_ready()
            else:
                dw = _mm(dy, a, a_mn=True, b_mn=True) if cuda else dy.t() @ a
        return da, dw, None, None


def _symm_of(w) -> Optional[tuple]:
    return getattr(w, "_hpb_symm", None) if (w.requires_grad and torch.is_grad_enabled()) else None


def column_parallel_linear(x_shard: torch.Tensor, w_shard: torch.Tensor, group) -> torch.Tensor:
    """``[T/tp, K] -> [T, N/tp]``: all-gather the token shards, multiply by this rank's rows of W."""
    return _ColumnParallel.apply(x_shard, w_shard, group, _symm_of(w_shard))


def row_parallel_linear(a: torch.Tensor, w_shard: torch.Tensor, group) -> torch.Tensor:
    """``[T, K/tp] -> [T/tp, N]``: multiply by this rank's columns of W, reduce-scatter over tokens."""
    return _RowParallel.apply(a, w_shard, group, _symm_of(w_shard))


class _CopyToTP(torch.autograd.Function):
    """Identity forward, all-reduce backward (replicated tensor entering a tensor-parallel region)."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        cc.all_reduce_(g, "sum", ctx.group)
        return g, None


def copy_to_tensor_parallel(x, group):
    return _CopyToTP.apply(x, group) if cc.group_size(group) > 1 else x


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, target: torch.Tensor, vocab_start: int, group,
                                 denom: float) -> torch.Tensor:
    """Mean token cross-entropy over a vocabulary sharded across ``group``.

    ``logits_local[T, V/tp]`` holds the columns ``[vocab_start, vocab_start + V/tp)``.
    """
    return _VocabParallelCE.apply(logits_local, target, vocab_start, group, denom)


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target, vocab_start, group, denom):
        lf = logits.float()
        vloc = logits.shape[1]
        mx = lf.max(dim=-1).values
        cc.all_reduce_(mx, "max", group)
        ex = torch.exp(lf - mx[:, None])
        se = ex.sum(-1)
        cc.all_reduce_(se, "sum", group)
        local_t = target - vocab_start
        in_range = (local_t >= 0) & (local_t < vloc)
        safe = local_t.clamp(0, vloc - 1)
        tl = torch.where(in_range, lf.gather(1, safe[:, None])[:, 0], torch.zeros_like(mx))
        cc.all_reduce_(tl, "sum", group)
        loss = (mx + se.log() - tl).sum() / denom
        p = ex / se[:, None]
        p[torch.arange(p.shape[0], device=p.device)[in_range], safe[in_range]] -= 1.0
        ctx.save_for_backward((p / denom).to(logits.dtype))
        return loss

    @staticmethod
    def backward(ctx, g):
        (d,) = ctx.saved_tensors
        return d * g.to(d.dtype), None, None, None, None
