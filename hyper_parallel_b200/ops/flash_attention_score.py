"""``flash_attention_score``: fused attention with the argument surface of ``npu_fusion_attention``.

The reference shards exactly this operator (hyper_parallel/core/shard/ops/
parallel_npu_flash_attention_score.py:50-1105): five tensor layouts, five ``sparse_mode`` values, a
``pre_tockens`` / ``next_tockens`` band and packed variable-length batches.  This module is the
single-device operator those rules wrap on a B200; the distributed rule lives in
``core/shard/ops/parallel_flash_attention_score.py``.

Layouts (``N`` = ``head_num``, ``D`` = head dimension, ``H = N * D``):
``BSH [B,S,H]``, ``SBH [S,B,H]``, ``BNSD [B,N,S,D]``, ``BSND [B,S,N,D]`` and ``TND [T,N,D]`` (packed
sequences; ``actual_seq_qlen`` / ``actual_seq_kvlen`` are the cumulative end offsets of every
sequence).  Key/value may have fewer heads than the query (grouped-query attention).

Which (query ``i``, key ``j``) pairs are kept, with ``d = Skv - Sq``:

====  ===================  =====================================================
mode  name                 kept
====  ===================  =====================================================
0     defaultMask          ``i - j <= pre_tockens`` and ``j - i <= next_tockens``,
                           and ``atten_mask[i, j] == 0`` when a mask is given
1     allMask              ``atten_mask[i, j] == 0``
2     leftUpCausal         ``j <= i``
3     rightDownCausal      ``j <= i + d``
4     band                 ``-pre_tockens <= j - (i + d) <= next_tockens``
====  ===================  =====================================================

(in modes 2-4 ``atten_mask`` is the compressed lower-triangular template of the NPU kernel and
carries no information; it is accepted and ignored).

Result: ``(attention_out, softmax_max, softmax_sum, softmax_out)``.  ``attention_out`` has the
layout of ``query``; ``softmax_max`` / ``softmax_sum`` are fp32 ``[B, N, Sq, 8]`` (``[T, N, 8]`` for
``TND``) with the row statistic repeated 8 times; ``softmax_out`` is an empty placeholder.

bf16 inputs with ``D == 128`` on a GPU, equal query/key lengths, no ``pse`` / mask / dropout and a
causal (modes 2, 3) or full (mode 0 without band) pattern run on this library's tcgen05 kernels;
there the kernels return the log-sum-exp ``L`` only, so the statistics are reported as
``softmax_max = L``, ``softmax_sum = 1`` (the same ``max + log(sum)``).  Everything else is computed
in fp32 with explicit masks.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

SPARSE_DEFAULT_MASK = 0
SPARSE_ALL_MASK = 1
SPARSE_LEFT_UP_CAUSAL = 2
SPARSE_RIGHT_DOWN_CAUSAL = 3
SPARSE_BAND = 4

LAYOUTS = ("BSH", "SBH", "BNSD", "BSND", "TND")
_NO_LIMIT = 2147483647


def keep_mask(sq: int, skv: int, sparse_mode: int, pre_tockens: int, next_tockens: int,
              atten_mask: Optional[torch.Tensor], device) -> Optional[torch.Tensor]:
    """Boolean ``[.., sq, skv]`` tensor of the kept pairs, or ``None`` when every pair is kept."""
    if sparse_mode not in (0, 1, 2, 3, 4):
        raise ValueError(f"sparse_mode must be 0..4, got {sparse_mode}")
    if sparse_mode == SPARSE_ALL_MASK:
        if atten_mask is None:
            raise ValueError("sparse_mode=1 (allMask) requires atten_mask to be provided")
        return ~atten_mask.to(torch.bool)
    i = torch.arange(sq, device=device)[:, None]
    j = torch.arange(skv, device=device)[None, :]
    if sparse_mode == SPARSE_DEFAULT_MASK:
        keep = None
        if pre_tockens < sq or next_tockens < skv:
            keep = ((i - j) <= pre_tockens) & ((j - i) <= next_tockens)
        if atten_mask is not None:
            free = ~atten_mask.to(torch.bool)
            keep = free if keep is None else (keep & free)
        return keep
    d = skv - sq
    if sparse_mode == SPARSE_LEFT_UP_CAUSAL:
        return j <= i
    if sparse_mode == SPARSE_RIGHT_DOWN_CAUSAL:
        return j <= i + d
    rel = j - (i + d)
    return (rel >= -pre_tockens) & (rel <= next_tockens)


def _dense_attention(q, k, v, scale, keep, pse, keep_prob):
    """fp32 attention on ``[B, N, S, D]`` tensors; returns ``(out, row max, row sum)``."""
    n, nkv = q.shape[1], k.shape[1]
    if n % nkv:
        raise ValueError(f"query heads ({n}) must be a multiple of key/value heads ({nkv})")
    qf, kf, vf = q.float(), k.float(), v.float()
    if nkv != n:
        kf = kf.repeat_interleave(n // nkv, dim=1)
        vf = vf.repeat_interleave(n // nkv, dim=1)
    s = qf @ kf.transpose(-1, -2)
    if pse is not None:
        s = s + pse.float()
    s = s * scale
    if keep is not None:
        s = s.masked_fill(~keep, float("-inf"))
    m = s.amax(dim=-1, keepdim=True)
    m = torch.where(torch.isfinite(m), m, torch.zeros_like(m))       # rows with no kept key
    e = torch.exp(s - m)
    l = e.sum(dim=-1, keepdim=True)
    p = e / l.clamp_min(1e-30)
    if keep_prob < 1.0:
        p = torch.nn.functional.dropout(p, 1.0 - keep_prob)
    return (p @ vf).to(q.dtype), m, l


class _KernelAttention(torch.autograd.Function):
    """Forward and backward on the tcgen05 kernels, ``[B, S, N, 128]`` bf16."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal):
        from .attention import flash_attention_forward
        out, lse = flash_attention_forward(q, k, v, causal=causal, scale=scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale, ctx.causal = scale, causal
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        from .attention import flash_attention_backward
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = flash_attention_backward(q, k, v, out, lse, do.contiguous(), causal=ctx.causal,
                                              scale=ctx.scale)[:3]
        return dq, dk, dv, None, None


def _kernel_pattern(sparse_mode, pre_tockens, next_tockens, sq, skv, atten_mask) -> Optional[bool]:
    """``True`` causal / ``False`` full when the pattern is one the kernels implement, else ``None``."""
    if sq != skv:
        return None
    if sparse_mode in (SPARSE_LEFT_UP_CAUSAL, SPARSE_RIGHT_DOWN_CAUSAL):
        return True
    if sparse_mode == SPARSE_BAND and pre_tockens >= sq and next_tockens == 0:
        return True
    if sparse_mode == SPARSE_DEFAULT_MASK and atten_mask is None:
        if pre_tockens >= sq and next_tockens >= skv:
            return False
        if pre_tockens >= sq and next_tockens == 0:
            return True
    return None


def _kernel_usable(q, k, pse, keep_prob) -> bool:
    if not q.is_cuda or q.dtype != torch.bfloat16 or q.shape[-1] != 128 or pse is not None or keep_prob < 1.0:
        return False
    from . import native
    return native.available()


def _to_bsnd(t: torch.Tensor, layout: str, heads: int) -> torch.Tensor:
    if layout == "BSH":
        return t.reshape(t.shape[0], t.shape[1], heads, t.shape[2] // heads)
    if layout == "SBH":
        return t.reshape(t.shape[0], t.shape[1], heads, t.shape[2] // heads).transpose(0, 1)
    if layout == "BNSD":
        return t.transpose(1, 2)
    return t                                                            # BSND


def _from_bsnd(t: torch.Tensor, layout: str) -> torch.Tensor:
    if layout == "BSH":
        return t.reshape(t.shape[0], t.shape[1], -1)
    if layout == "SBH":
        return t.transpose(0, 1).reshape(t.shape[1], t.shape[0], -1)
    if layout == "BNSD":
        return t.transpose(1, 2)
    return t


def _attend(q, k, v, scale, sparse_mode, pre_tockens, next_tockens, atten_mask, pse, keep_prob):
    """``q [B,Sq,N,D]``, ``k/v [B,Skv,Nkv,D]`` -> ``(out [B,Sq,N,D], max [B,N,Sq,1], sum [B,N,Sq,1])``."""
    sq, skv = q.shape[1], k.shape[1]
    pattern = _kernel_pattern(sparse_mode, pre_tockens, next_tockens, sq, skv, atten_mask)
    if pattern is not None and _kernel_usable(q, k, pse, keep_prob):
        out, lse = _KernelAttention.apply(q, k, v, float(scale), bool(pattern))
        return out, lse.unsqueeze(-1), torch.ones_like(lse).unsqueeze(-1)
    keep = keep_mask(sq, skv, sparse_mode, pre_tockens, next_tockens, atten_mask, q.device)
    out, m, l = _dense_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale, keep, pse,
                                 keep_prob)
    return out.transpose(1, 2), m, l


def _ends(lens: Sequence[int], what: str, total: int) -> list:
    ends = [int(x) for x in lens]
    if any(b < a for a, b in zip([0] + ends[:-1], ends)) or (ends and ends[-1] > total):
        raise ValueError(f"{what} must be non-decreasing cumulative offsets within {total}, got {ends}")
    return ends


def flash_attention_score(query, key, value, head_num, input_layout, pse=None, padding_mask=None,
                          atten_mask=None, scale=1.0, keep_prob=1.0, pre_tockens=_NO_LIMIT,
                          next_tockens=_NO_LIMIT, inner_precise=0, prefix=None, actual_seq_qlen=None,
                          actual_seq_kvlen=None, sparse_mode=0, gen_mask_parallel=True, sync=False
                          ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """See the module docstring.  ``padding_mask``, ``inner_precise``, ``prefix``,
    ``gen_mask_parallel`` and ``sync`` are accepted for signature compatibility and unused."""
    if torch.overrides.has_torch_function((query, key, value)):
        return torch.overrides.handle_torch_function(
            flash_attention_score, (query, key, value), query, key, value, head_num, input_layout, pse,
            padding_mask, atten_mask, scale, keep_prob, pre_tockens, next_tockens, inner_precise, prefix,
            actual_seq_qlen, actual_seq_kvlen, sparse_mode, gen_mask_parallel, sync)
    if input_layout not in LAYOUTS:
        raise ValueError(f"Unsupported input_layout: '{input_layout}'. Supported layouts: {list(LAYOUTS)}")
    if prefix is not None:
        raise NotImplementedError("prefix (sparse modes 5 and 6) is not supported")
    head_num = int(head_num)
    empty = query.new_empty(0)

    if input_layout == "TND":
        if actual_seq_qlen is None or actual_seq_kvlen is None:
            raise ValueError("input_layout='TND' requires actual_seq_qlen and actual_seq_kvlen")
        q_ends = _ends(actual_seq_qlen, "actual_seq_qlen", query.shape[0])
        k_ends = _ends(actual_seq_kvlen, "actual_seq_kvlen", key.shape[0])
        if len(q_ends) != len(k_ends):
            raise ValueError("actual_seq_qlen and actual_seq_kvlen must list the same number of sequences")
        t, n = query.shape[0], query.shape[1]
        out = torch.zeros_like(query)
        smax = torch.zeros(t, n, 1, dtype=torch.float32, device=query.device)
        ssum = torch.zeros(t, n, 1, dtype=torch.float32, device=query.device)
        outs, q0, k0 = [], 0, 0
        for q1, k1 in zip(q_ends, k_ends):
            if q1 > q0:
                if k1 > k0:
                    o, m, l = _attend(query[None, q0:q1], key[None, k0:k1], value[None, k0:k1], scale, sparse_mode,
                                      pre_tockens, next_tockens, atten_mask, pse, keep_prob)
                    outs.append((q0, q1, o[0], m[0].transpose(0, 1).detach(), l[0].transpose(0, 1).detach()))
            q0, k0 = q1, k1
        if outs:
            # one concatenation keeps the graph simple: rows no sequence covers stay zero
            pieces, cursor = [], 0
            for a, b, o, m, l in outs:
                if a > cursor:
                    pieces.append(out[cursor:a])
                pieces.append(o)
                smax[a:b], ssum[a:b] = m, l
                cursor = b
            if cursor < t:
                pieces.append(out[cursor:])
            out = torch.cat(pieces, dim=0)
        return out, smax.expand(t, n, 8).contiguous(), ssum.expand(t, n, 8).contiguous(), empty

    d = query.shape[-1] if input_layout in ("BNSD", "BSND") else query.shape[-1] // head_num
    if input_layout in ("BSH", "SBH"):
        if query.shape[-1] % head_num or key.shape[-1] % d:
            raise ValueError(f"hidden sizes {query.shape[-1]} / {key.shape[-1]} do not divide into heads of "
                             f"{d} (head_num={head_num})")
        kv_heads = key.shape[-1] // d
    else:
        kv_heads = key.shape[1] if input_layout == "BNSD" else key.shape[2]
    q = _to_bsnd(query, input_layout, head_num)
    k = _to_bsnd(key, input_layout, kv_heads)
    v = _to_bsnd(value, input_layout, kv_heads)
    if q.shape[2] != head_num:
        raise ValueError(f"head_num={head_num} does not match the query's {q.shape[2]} heads")
    out, m, l = _attend(q, k, v, scale, sparse_mode, pre_tockens, next_tockens, atten_mask, pse, keep_prob)
    b, sq = q.shape[0], q.shape[1]
    return (_from_bsnd(out, input_layout), m.expand(b, head_num, sq, 8).contiguous(),
            l.expand(b, head_num, sq, 8).contiguous(), empty)


#: the name user code written against the NPU operator calls
npu_fusion_attention = flash_attention_score
