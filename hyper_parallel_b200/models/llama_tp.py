"""Tensor-parallel (+ sequence-parallel) Llama built from ``parallel.tensor_parallel``.

Weights are sharded over the ``tp`` axis of a ``(dp, tp)`` mesh and are exposed as DTensor
parameters, so that ``hsdp()`` on top of it derives the data-parallel group from the mesh axes
that do not shard the parameter (hyper_parallel/core/hsdp/hsdp_param.py:69-124 of the reference)
and distributed checkpoints know the global layout.  Heads are split across ranks: each rank
holds ``[q_local | k_local | v_local]`` rows of the fused QKV weight and ``[gate_local | up_local]``
rows of the fused MLP weight.  Activations between blocks are sharded over tokens
(``[T / tp, H]``); the embedding is replicated and each rank embeds its own token slice; the
output head is vocabulary-parallel with a vocabulary-parallel cross-entropy.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..core.dtensor import DTensor
from ..core.layout import Layout
from ..ops import attention as attn_ops
from ..parallel import tensor_parallel as tp_ops
from .llama import LlamaConfig, _RopeQK


def _local(p):
    return p.to_local() if isinstance(p, DTensor) else p


def _tp_param(shape, layout: Optional[Layout], spec, device, dtype) -> nn.Parameter:
    """Parameter holding this rank's shard of a tensor of global ``shape`` laid out as ``spec``."""
    if layout is None:
        return nn.Parameter(torch.empty(shape, device=device, dtype=dtype))
    lay = layout(*spec)
    local = torch.empty(lay.get_local_shape(shape), device=device, dtype=dtype)
    p = nn.Parameter(DTensor._wrap(local, lay))
    if not lay.sharded_axes:
        # replicated over tp: its gradient is all-reduced inside the TP region (copy_to_tensor_parallel),
        # so data-parallel sharding / reduction must only span the remaining axes
        p.hsdp_exclude_axes = tuple(a for a in layout.alias_name if a != "dp")
    return p


class TPLlamaBlock(nn.Module):
    def __init__(self, cfg: LlamaConfig, layer_idx: int, layout: Optional[Layout], tp_axis: str = "tp",
                 device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        mesh = layout.mesh if layout is not None else None
        self.group = mesh.get_group(tp_axis) if mesh is not None else None
        self.tp = mesh.size(tp_axis) if mesh is not None else 1
        self.tp_rank = mesh.get_local_rank(tp_axis) if mesh is not None else 0
        h, hd = cfg.hidden_size, cfg.head_dim
        if cfg.num_heads % self.tp or cfg.num_kv_heads % self.tp or cfg.ffn_size % self.tp:
            raise ValueError("heads, kv heads and ffn size must be divisible by the tensor-parallel size")
        rep = ("None",)
        self.attn_norm = _tp_param((h,), layout, rep, device, dtype)
        self.ffn_norm = _tp_param((h,), layout, rep, device, dtype)
        self.wqkv = _tp_param(((cfg.num_heads + 2 * cfg.num_kv_heads) * hd, h), layout, (tp_axis, "None"), device, dtype)
        self.wo = _tp_param((h, cfg.num_heads * hd), layout, ("None", tp_axis), device, dtype)
        self.w_gate_up = _tp_param((2 * cfg.ffn_size, h), layout, (tp_axis, "None"), device, dtype)
        self.w_down = _tp_param((h, cfg.ffn_size), layout, ("None", tp_axis), device, dtype)

    # -- initialisation: every rank draws the full tensors (same seed) and keeps its slice -----
    def reset_parameters(self):
        cfg, tp, r = self.cfg, self.tp, self.tp_rank
        std, hd = cfg.init_std, cfg.head_dim
        full = lambda p: p.layout.get_global_shape(_local(p).shape) if isinstance(p, DTensor) else p.shape  # noqa: E731

        def draw(p):
            t = torch.empty(tuple(full(p)), dtype=torch.float32, device=_local(p).device)
            return t.normal_(0.0, std)
        with torch.no_grad():
            wqkv = draw(self.wqkv)
            nq, nk = cfg.num_heads * hd, cfg.num_kv_heads * hd
            q, k, v = wqkv.split([nq, nk, nk], dim=0)
            _local(self.wqkv).copy_(torch.cat([q.chunk(tp, 0)[r], k.chunk(tp, 0)[r], v.chunk(tp, 0)[r]], 0))
            _local(self.wo).copy_(draw(self.wo).chunk(tp, 1)[r])
            gu = draw(self.w_gate_up)
            g, u = gu.chunk(2, dim=0)
            _local(self.w_gate_up).copy_(torch.cat([g.chunk(tp, 0)[r], u.chunk(tp, 0)[r]], 0))
            _local(self.w_down).copy_(draw(self.w_down).chunk(tp, 1)[r])
            _local(self.attn_norm).fill_(1.0)
            _local(self.ffn_norm).fill_(1.0)

    def forward(self, h, resid, batch: int, seq_len: int):
        """``h`` / ``resid``: token-sharded ``[T / tp, H]`` (tokens of the whole local batch, split over tp)."""
        cfg = self.cfg
        nh, nkv, hd = cfg.num_heads // self.tp, cfg.num_kv_heads // self.tp, cfg.head_dim
        attn_norm = tp_ops.copy_to_tensor_parallel(_local(self.attn_norm), self.group)
        ffn_norm = tp_ops.copy_to_tensor_parallel(_local(self.ffn_norm), self.group)
        if resid is None:
            resid = h
            x = ops.rmsnorm(h, attn_norm, cfg.norm_eps)
        else:
            x, resid = ops.add_rmsnorm(h, resid, attn_norm, cfg.norm_eps)
        qkv = tp_ops.column_parallel_linear(x, _local(self.wqkv), self.group)        # [T, (nh + 2 nkv) hd]
        if qkv.is_cuda:
            qkv = _RopeQK.apply(qkv, nh, nkv, hd, seq_len, cfg.rope_theta)
            a = attn_ops.causal_attention_packed(qkv.view(batch, seq_len, -1), nh, nkv)
            q = None
        else:
            q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
            q = ops.apply_rope(q.reshape(-1, nh, hd), seq_len, cfg.rope_theta).reshape(-1, nh * hd)
            k = ops.apply_rope(k.reshape(-1, nkv, hd), seq_len, cfg.rope_theta).reshape(-1, nkv * hd)
        if q is not None:
            a = attn_ops.causal_attention(q.view(batch, seq_len, nh, hd), k.view(batch, seq_len, nkv, hd),
                                          v.view(batch, seq_len, nkv, hd))
        o = tp_ops.row_parallel_linear(a.reshape(batch * seq_len, nh * hd), _local(self.wo), self.group)
        x, resid = ops.add_rmsnorm(o, resid, ffn_norm, cfg.norm_eps)
        gu = tp_ops.column_parallel_linear(x, _local(self.w_gate_up), self.group)
        d = tp_ops.row_parallel_linear(ops.swiglu(gu), _local(self.w_down), self.group)
        return d, resid


class TPLlama(nn.Module):
    """``forward(tokens[B, S], targets[B, S])`` -> mean token loss; every tp rank gets the same batch."""

    def __init__(self, cfg: LlamaConfig, layout: Optional[Layout] = None, tp_axis: str = "tp", device=None,
                 dtype=torch.bfloat16, first_layer: int = 0, num_layers: Optional[int] = None,
                 with_embed: bool = True, with_head: bool = True):
        super().__init__()
        self.cfg = cfg
        mesh = layout.mesh if layout is not None else None
        self.group = mesh.get_group(tp_axis) if mesh is not None else None
        self.tp = mesh.size(tp_axis) if mesh is not None else 1
        self.tp_rank = mesh.get_local_rank(tp_axis) if mesh is not None else 0
        n = cfg.num_layers - first_layer if num_layers is None else num_layers
        self.with_embed, self.with_head = with_embed, with_head
        if with_embed:
            self.embed = _tp_param((cfg.vocab_size, cfg.hidden_size), layout, ("None", "None"), device, dtype)
        self.layers = nn.ModuleList(TPLlamaBlock(cfg, first_layer + i, layout, tp_axis, device, dtype) for i in range(n))
        if with_head:
            if cfg.vocab_size % self.tp:
                raise ValueError("vocab size must be divisible by the tensor-parallel size")
            self.final_norm = _tp_param((cfg.hidden_size,), layout, ("None",), device, dtype)
            self.lm_head = _tp_param((cfg.vocab_size, cfg.hidden_size), layout, (tp_axis, "None"), device, dtype)

    def reset_parameters(self):
        std = self.cfg.init_std
        with torch.no_grad():
            if self.with_embed:
                _local(self.embed).normal_(0.0, std)
            if self.with_head:
                _local(self.final_norm).fill_(1.0)
                p = self.lm_head
                shape = p.layout.get_global_shape(_local(p).shape) if isinstance(p, DTensor) else p.shape
                full = torch.empty(tuple(shape), dtype=torch.float32, device=_local(p).device).normal_(0.0, std)
                _local(p).copy_(full.chunk(self.tp, 0)[self.tp_rank])

    def init_weights(self):
        self.reset_parameters()
        for layer in self.layers:
            layer.reset_parameters()

    def forward(self, x, targets: Optional[torch.Tensor] = None, batch: Optional[int] = None,
                seq_len: Optional[int] = None, loss_denominator: Optional[float] = None):
        """First stage: ``x`` = tokens ``[B, S]``; later pipeline stages: ``x = (h, resid)`` token-sharded."""
        tp, r = self.tp, self.tp_rank
        if self.with_embed:
            B, S = x.shape
            flat = x.reshape(-1)
            mine = flat.chunk(tp)[r] if tp > 1 else flat            # sequence parallel: my slice of the tokens
            emb = tp_ops.copy_to_tensor_parallel(_local(self.embed), self.group)
            h, resid = F.embedding(mine, emb), None
        else:
            h, resid = x
            B, S = batch, seq_len
        for layer in self.layers:
            h, resid = layer(h, resid, B, S)
        if not self.with_head:
            return h, resid
        fn = tp_ops.copy_to_tensor_parallel(_local(self.final_norm), self.group)
        xn, _ = ops.add_rmsnorm(h, resid, fn, self.cfg.norm_eps)
        logits = tp_ops.column_parallel_linear(xn, _local(self.lm_head), self.group)      # [T, V / tp]
        if targets is None:
            return logits
        T = B * S
        return tp_ops.vocab_parallel_cross_entropy(logits, targets.reshape(-1), r * (self.cfg.vocab_size // tp),
                                                   self.group, float(loss_denominator or T))
