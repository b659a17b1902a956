"""Ulysses-style context parallelism: switch activations between sequence-sharded and head-sharded.

In the reference this is only *expressible* as a ``redistribute`` (S(seq) <-> S(head), one
all-to-all, hyper_parallel/core/redistribute_infer.py:368-405) and is listed as future work
(README.en.md:67).  These helpers package it: before attention ``seq_to_head`` gives every rank
all positions of ``H / n`` heads, after attention ``head_to_seq`` goes back.  Both are differentiable.
"""
from __future__ import annotations

import torch

from ..collectives import cc


def seq_to_head(x: torch.Tensor, group, seq_dim: int = 1, head_dim: int = 2) -> torch.Tensor:
    """``[B, S/n, H, D] -> [B, S, H/n, D]`` (one all-to-all over ``group``)."""
    return cc.all_to_all(x, head_dim, seq_dim, group)


def head_to_seq(x: torch.Tensor, group, seq_dim: int = 1, head_dim: int = 2) -> torch.Tensor:
    """``[B, S, H/n, D] -> [B, S/n, H, D]``."""
    return cc.all_to_all(x, seq_dim, head_dim, group)


def ulysses_attention(q, k, v, group, attn_fn):
    """Run ``attn_fn(q, k, v)`` (full-sequence attention on a subset of heads) on sequence-sharded inputs."""
    if cc.group_size(group) == 1:
        return attn_fn(q, k, v)
    q, k, v = (seq_to_head(t, group) for t in (q, k, v))
    return head_to_seq(attn_fn(q, k, v), group)
