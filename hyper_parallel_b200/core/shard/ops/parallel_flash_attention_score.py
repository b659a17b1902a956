"""Layout rule of ``flash_attention_score`` / ``npu_fusion_attention``.

Parallel modes, as in hyper_parallel/core/shard/ops/parallel_npu_flash_attention_score.py:50-1105 of
the reference:

* **DP**: the batch dimension of q/k/v sharded identically;
* **MP**: the head dimension (the hidden dimension of ``BSH`` / ``SBH``) sharded identically --
  ``head_num`` becomes the local head count;
* **SP**: the *query* sequence sharded while key/value hold the full sequence on every rank of that
  axis.  A shard holding query rows ``[r*L, (r+1)*L)`` of ``Sq = n*L`` must apply the global mask to
  its rows, so the mask parameters are rewritten (below);
* ``TND`` (packed sequences): sharding the token dimension of q and k/v alike splits the batch of
  sequences (DP); sharding q's token dimension finer than k/v's splits sequences across ranks
  (context parallel), which needs ``sparse_mode=3`` and re-based cumulative lengths;
* sharding the key/value sequence of the other layouts would need ring attention and raises
  ``NotImplementedError``.

Mask rewrite for SP.  A pair (global query row ``i``, key ``j``) is kept iff
``lo <= j - i - ref <= hi`` with ``(lo, hi, ref)`` = ``(-pre, next, 0)`` for mode 0,
``(-Skv, 0, 0)`` for mode 2, ``(-Skv, 0, Skv - Sq)`` for mode 3 and ``(-pre, next, Skv - Sq)`` for
mode 4.  With ``i = i_local + r*L`` the same set in local coordinates is a band around the local
reference diagonal ``ref_local``: ``lo + s <= j - i_local - ref_local <= hi + s`` where
``s = r*L + ref - ref_local``.  Mode 0 stays mode 0 (``ref_local = 0``); modes 2-4 become a mode-4
band (``ref_local = Skv - L``).  Mode 1 (explicit mask only) is passed through; an explicit mask
whose row count is the global ``Sq`` is narrowed to the shard's rows.

Outputs: ``attention_out`` as ``query``; ``softmax_max`` / ``softmax_sum`` ``[B, N, Sq, 8]``
sharded like (batch, heads, query sequence, -) -- ``[T, N, 8]`` like (tokens, heads, -) for ``TND``;
``softmax_out`` (an empty placeholder) replicated.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from ._common import make
from .parallel_ops import DistributedOp

_DIMS = {
    "BSH": {"batch": 0, "seq": 1, "head": 2},
    "SBH": {"seq": 0, "batch": 1, "head": 2},
    "BNSD": {"batch": 0, "head": 1, "seq": 2, "dim": 3},
    "BSND": {"batch": 0, "seq": 1, "head": 2, "dim": 3},
    "TND": {"seq": 0, "head": 1, "dim": 2},
}


def _input_layout_of(extra_args) -> str:
    for a in extra_args:
        if isinstance(a, str):
            if a not in _DIMS:
                raise ValueError(f"Unsupported input_layout: '{a}'. Supported layouts: {list(_DIMS)}")
            return a
    raise ValueError("Missing required parameter 'input_layout'")


def _split(layout, dim: int) -> Tuple[int, int]:
    """(number of shards, index of this rank's shard) of tensor dimension ``dim``."""
    n, idx = 1, 0
    mesh = layout.mesh
    for a in layout.dim_axes[dim]:
        idx = idx * mesh.mesh_shape[a] + mesh.get_local_rank(a)
        n *= mesh.mesh_shape[a]
    return n, idx


def shard_mask_params(sparse_mode: int, pre_tockens: int, next_tockens: int, shard: int, n_shards: int,
                      local_q: int, kv_len: int) -> Tuple[int, int, int]:
    """Mask parameters for query shard ``shard`` of ``n_shards`` (module docstring)."""
    if sparse_mode == 1 or sparse_mode not in (0, 2, 3, 4):
        return sparse_mode, pre_tockens, next_tockens
    q_len = local_q * n_shards
    if sparse_mode == 0:
        s = shard * local_q
        return 0, pre_tockens - s, next_tockens + s
    lo, hi = (-kv_len, 0) if sparse_mode in (2, 3) else (-pre_tockens, next_tockens)
    ref = 0 if sparse_mode == 2 else kv_len - q_len
    s = shard * local_q + ref - (kv_len - local_q)
    return 4, -(lo + s), hi + s


def shard_packed_lengths(q_ends: Sequence[int], kv_ends: Sequence[int], shard: int, local_tq: int,
                         local_tk: int, kv_sharded: bool) -> Tuple[List[int], List[int]]:
    """Cumulative sequence ends seen by the rank that holds packed query rows
    ``[shard*local_tq, (shard+1)*local_tq)``.

    With k/v sharded the same way (whole sequences per rank) both lists are re-based and clamped.
    With k/v complete on every rank (context parallel, right-down causal) a sequence whose last
    ``c`` query rows live on later ranks keeps all its keys but the last ``c``: the local rows are
    then again the trailing rows of the (shortened) key range."""
    off = shard * local_tq
    new_q = [min(max(e - off, 0), local_tq) for e in q_ends]
    if kv_sharded:
        koff = shard * local_tk
        return new_q, [min(max(e - koff, 0), local_tk) for e in kv_ends]
    cut = [max(e - off, 0) - nq for e, nq in zip(q_ends, new_q)]
    return new_q, [k - c for k, c in zip(kv_ends, cut)]


class FlashAttentionScoreDistributedOp(DistributedOp):
    def _check(self, layouts, fmt: str):
        q, k, v = layouts[0], layouts[1], layouts[2]
        if q is None or k is None or v is None:
            raise ValueError(f"For {self.op_name}, query/key/value must be distributed tensors")
        if k.dim_axes != v.dim_axes:
            raise ValueError("Key and Value must have identical sharding strategies.\n"
                             f"Key: {k.dim_axes}\nValue: {v.dim_axes}")
        dims = _DIMS[fmt]
        for what in ("batch", "head", "dim"):
            if what in dims and q.dim_axes[dims[what]] != k.dim_axes[dims[what]]:
                label = "hidden" if (what == "head" and fmt in ("BSH", "SBH")) else what
                raise ValueError(f"Query and Key/Value must have identical {label} sharding strategy.\n"
                                 f"Input layout: {fmt}\nQuery: {q.dim_axes}\nKey/Value: {k.dim_axes}")
        if "dim" in dims and q.dim_axes[dims["dim"]]:
            raise ValueError(f"For {self.op_name}, the head dimension D must not be sharded")
        sd = dims["seq"]
        if fmt != "TND" and k.dim_axes[sd]:
            raise NotImplementedError(
                f"KV sequence sharding is not supported for layout '{fmt}' without Ring Attention; "
                "replicate key/value along the sequence axis (gather them) first")
        return q, k, dims

    def infer_layout(self, layouts, extra_args):
        self._check_partial_inputs(layouts)
        fmt = _input_layout_of(extra_args)
        q, _, dims = self._check(layouts, fmt)
        if fmt == "TND":
            stats = make(q, [q.dim_axes[0], q.dim_axes[1], ()])
        else:
            stats = make(q, [q.dim_axes[dims["batch"]], q.dim_axes[dims["head"]], q.dim_axes[dims["seq"]], ()])
        return (make(q, q.dim_axes), stats, make(q, stats.dim_axes), make(q, [()]))

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        fmt = _input_layout_of(extra_args)
        q_layout, k_layout, dims = self._check(layouts, fmt)
        head_split, _ = _split(q_layout, dims["head"])
        seq_split, seq_idx = _split(q_layout, dims["seq"])
        kv_split, _ = _split(k_layout, dims["seq"])
        if head_split == 1 and seq_split == 1:
            return None
        sd = dims["seq"]
        name = self.op_name

        def impl(query, key, value, head_num, input_layout, pse=None, padding_mask=None, atten_mask=None,
                 scale=1.0, keep_prob=1.0, pre_tockens=2147483647, next_tockens=2147483647, inner_precise=0,
                 prefix=None, actual_seq_qlen=None, actual_seq_kvlen=None, sparse_mode=0,
                 gen_mask_parallel=True, sync=False):
            if head_num % head_split:
                raise ValueError(f"head_num({head_num}) not divisible by head_split_num({head_split})")
            head_num = head_num // head_split
            if seq_split > 1 and fmt == "TND":
                if actual_seq_qlen is None or actual_seq_kvlen is None:
                    raise ValueError("When using TND layout with sequence parallelism, actual_seq_qlen and "
                                     "actual_seq_kvlen must be provided.")
                if seq_split % kv_split:
                    raise ValueError("TND layout requires Query split number to be an integer multiple of Key "
                                     f"split number, got {seq_split} and {kv_split}")
                cp = seq_split // kv_split
                if cp > 1:
                    if kv_split > 1:
                        raise NotImplementedError(
                            f"For {name}, TND context parallelism combined with a sharded key/value token "
                            "dimension is not supported; keep key/value complete on the context-parallel axis")
                    if sparse_mode != 3:
                        raise ValueError(f"TND layout with context parallelism (s1_split_num={cp} > 1) requires "
                                         f"sparse_mode=3 (rightDownCausal), but got sparse_mode={sparse_mode}.")
                    if query.shape[0] * seq_split != key.shape[0] * kv_split:
                        raise ValueError("TND layout with context parallelism requires Query and Key to have the "
                                         "same global T-dimension")
                elif query.shape[0] != key.shape[0]:
                    raise ValueError("TND layout with DP-only (s1_split_num=1) requires Query and Key to have "
                                     "the same local T-dimension")
                actual_seq_qlen, actual_seq_kvlen = shard_packed_lengths(
                    actual_seq_qlen, actual_seq_kvlen, seq_idx, query.shape[0], key.shape[0], kv_split > 1)
            elif seq_split > 1:
                local_q, kv_len = query.shape[sd], key.shape[sd]
                if atten_mask is not None and sparse_mode in (0, 1) and atten_mask.shape[-2] == local_q * seq_split:
                    atten_mask = atten_mask.narrow(-2, seq_idx * local_q, local_q)
                sparse_mode, pre_tockens, next_tockens = shard_mask_params(
                    sparse_mode, pre_tockens, next_tockens, seq_idx, seq_split, local_q, kv_len)
            result = func(query, key, value, head_num, input_layout, pse, padding_mask, atten_mask, scale, keep_prob,
                          pre_tockens, next_tockens, inner_precise, prefix, actual_seq_qlen, actual_seq_kvlen,
                          sparse_mode, gen_mask_parallel, sync)
            return tuple(result[:4]) if isinstance(result, (tuple, list)) else result
        return impl
