"""``scaled_dot_product_attention(q, k, v)`` on ``[B, H, S, D]`` tensors.

Same parallel modes as hyper_parallel/core/shard/ops/parallel_scaled_dot_product_attention.py:32-376
of the reference: DP (batch sharded), MP (heads sharded), and SP = **query sequence sharded with
K/V replicated along that axis**.  For causal SP each rank attends to keys ``[0, (i+1)*S_local)``
where ``i`` is its position on the sequence axis: K/V are narrowed to that window and, for
``i > 0``, an explicit lower-right-aligned mask replaces ``is_causal``.  Sharding the K/V
sequence would need ring attention and raises ``NotImplementedError``.
"""
from __future__ import annotations

import torch

from ._common import make
from .parallel_ops import DistributedOp


class ScaledDotProductAttentionDistributedOp(DistributedOp):
    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        q, k, v = layouts[0], layouts[1], layouts[2]
        if q is None or k is None or v is None:
            raise ValueError("For scaled_dot_product_attention, q/k/v must be distributed tensors")
        nd = len(q.dim_axes)
        if q.dim_axes[-1] or k.dim_axes[-1] or v.dim_axes[-1]:
            raise ValueError("For scaled_dot_product_attention, the head dim must not be sharded")
        if k.dim_axes[-2] or v.dim_axes[-2]:
            raise NotImplementedError(
                "scaled_dot_product_attention: KV sequence sharding requires Ring Attention; replicate "
                "K/V along the sequence axis (gather them) first")
        if k.dim_axes != v.dim_axes:
            raise ValueError("For scaled_dot_product_attention, Key and Value must have identical sharding "
                             f"(key {k.alias_tensor_map}, value {v.alias_tensor_map})")
        for d in range(nd - 2):
            if not (q.dim_axes[d] == k.dim_axes[d] == v.dim_axes[d]):
                raise ValueError("For scaled_dot_product_attention, batch/head dims of q, k, v must be "
                                 "sharded identically")
        for m in layouts[3:]:
            if m is None:
                continue
            # a distributed mask: its query-row dim is sharded like q's (rows already local) or not at all
            # (the rows of this rank's queries are cut out below); the other dims follow q from the right
            md = len(m.dim_axes)
            if md < 2 or m.dim_axes[-1]:
                raise ValueError("For scaled_dot_product_attention, the key dim of attn_mask must not be sharded")
            if m.dim_axes[-2] and m.dim_axes[-2] != q.dim_axes[-2]:
                raise ValueError("For scaled_dot_product_attention, the query dim of attn_mask must be sharded "
                                 "like the query sequence, or not at all")
            for j in range(3, md + 1):
                if m.dim_axes[-j] and (j > nd or m.dim_axes[-j] != q.dim_axes[-j]):
                    raise ValueError("For scaled_dot_product_attention, batch/head dims of attn_mask must be "
                                     "sharded like the query's, or not at all")
        return make(q, q.dim_axes)

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        q = layouts[0]
        seq_axes = q.dim_axes[-2]
        if not seq_axes:
            return None
        mesh = q.mesh
        n, idx = 1, 0
        for a in seq_axes:
            idx = idx * mesh.mesh_shape[a] + mesh.get_local_rank(a)
            n *= mesh.mesh_shape[a]

        def impl(query, key, value, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, **kw):
            sq = query.shape[-2]
            if not is_causal:
                if attn_mask is not None and attn_mask.dim() >= 2 and attn_mask.shape[-2] == n * sq and n > 1:
                    attn_mask = attn_mask.narrow(-2, idx * sq, sq)      # the rows of this rank's queries
                return func(query, key, value, attn_mask=attn_mask, dropout_p=dropout_p,
                            is_causal=False, scale=scale, **kw)
            kv_len = (idx + 1) * sq
            key = key.narrow(-2, 0, kv_len)
            value = value.narrow(-2, 0, kv_len)
            if idx == 0:
                return func(query, key, value, dropout_p=dropout_p, is_causal=True, scale=scale, **kw)
            # query row r is global position idx*sq + r: it sees keys [0, idx*sq + r]
            rows = torch.arange(sq, device=query.device)[:, None] + idx * sq
            cols = torch.arange(kv_len, device=query.device)[None, :]
            mask = cols <= rows
            return func(query, key, value, attn_mask=mask, dropout_p=dropout_p, is_causal=False,
                        scale=scale, **kw)
        return impl
