"""DeepSeek-V3-style decoder: MLA attention + MoE with sigmoid group-limited routing and expert parallelism.

The reference ships no model or expert-parallel code (its README lists EP as future work,
README.en.md:61-65); this module provides the architecture its MoE benchmark is quoted on:

* **MLA**: low-rank query (``q_lora``) and joint key/value (``kv_lora``) projections, decoupled
  RoPE key of ``qk_rope`` dims shared by all heads, per-head ``qk_nope`` + ``v_head`` dims;
* **router**: ``sigmoid(x W_g^T)``; selection score = score + aux-free bias; experts are split
  into ``n_group`` groups, each group scored by the sum of its top-2 selection scores, the best
  ``topk_group`` groups survive and the ``top_k`` best experts inside them are picked; gate
  weights are the *un-biased* scores, normalised to sum to 1 and multiplied by
  ``routed_scaling_factor``;
* **experts**: ``n_routed_experts`` SwiGLU experts sharded over the expert-parallel group
  (dispatch / combine all-to-all), plus ``n_shared_experts`` always-on shared experts.

On CUDA the routing, permutation and expert GEMMs use the kernels of ``hyper_parallel_b200.ops``;
on CPU the same functions run their PyTorch formulation, which is the oracle.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..collectives import cc
from ..ops import mla_attention as mla_ops
from ..ops import moe as moe_ops


@dataclass
class DeepSeekV3Config:
    vocab_size: int = 129280
    hidden_size: int = 7168
    num_layers: int = 4
    first_k_dense: int = 1
    num_heads: int = 128
    q_lora_rank: int = 1536
    kv_lora_rank: int = 512
    qk_nope_head_dim: int = 128
    qk_rope_head_dim: int = 64
    v_head_dim: int = 128
    dense_ffn_size: int = 18432
    moe_ffn_size: int = 2048
    n_routed_experts: int = 256
    n_shared_experts: int = 1
    top_k: int = 8
    n_group: int = 8
    topk_group: int = 4
    routed_scaling_factor: float = 2.5
    rope_theta: float = 10000.0
    norm_eps: float = 1e-6
    init_std: float = 0.006
    # block-scaled fp8 (e4m3; 1x128 activation tiles, 128x128 weight tiles) for the forward GEMMs of
    # the attention / dense / shared-expert projections and of the routed experts; master weights,
    # the backward GEMMs, the router and the lm head stay bf16 / fp32
    fp8: bool = False
    # receive capacity of the expert-parallel dispatch, in multiples of the balanced load; 0 = as large
    # as any routing can need (the expert-parallel size), capped at 4: group-limited routing of
    # correlated tokens can legitimately send most pairs to the ranks of a few groups
    ep_capacity: float = 0.0

    @staticmethod
    def tiny() -> "DeepSeekV3Config":
        return DeepSeekV3Config(vocab_size=512, hidden_size=128, num_layers=2, first_k_dense=1, num_heads=4,
                                q_lora_rank=64, kv_lora_rank=32, qk_nope_head_dim=32, qk_rope_head_dim=16,
                                v_head_dim=32, dense_ffn_size=256, moe_ffn_size=64, n_routed_experts=16,
                                n_shared_experts=1, top_k=4, n_group=4, topk_group=2)

    def flops_per_token(self, seq_len: int) -> float:
        h = self.hidden_size
        qk = self.qk_nope_head_dim + self.qk_rope_head_dim
        attn_p = h * self.q_lora_rank + self.q_lora_rank * self.num_heads * qk + \
            h * (self.kv_lora_rank + self.qk_rope_head_dim) + \
            self.kv_lora_rank * self.num_heads * (self.qk_nope_head_dim + self.v_head_dim) + \
            self.num_heads * self.v_head_dim * h
        dense = 3 * h * self.dense_ffn_size
        moe = 3 * h * self.moe_ffn_size * (self.top_k + self.n_shared_experts) + h * self.n_routed_experts
        n_moe = self.num_layers - self.first_k_dense
        mm = self.num_layers * attn_p + self.first_k_dense * dense + n_moe * moe + self.vocab_size * h
        attn = self.num_layers * 6 * self.num_heads * (qk + self.v_head_dim) * seq_len / 2
        return 6.0 * mm + attn


def _lin(x: torch.Tensor, w: torch.Tensor, fp8: bool) -> torch.Tensor:
    """Projection ``x @ w.T``: fp8 block-scaled forward GEMM when asked for (CUDA, K % 128 == 0)."""
    if fp8 and x.is_cuda and x.shape[-1] % 128 == 0:
        from ..ops import fp8 as f8
        return f8.fp8_linear(x, w)
    return ops.linear(x, w)


def _rope_last(x: torch.Tensor, seq_len: int, theta: float) -> torch.Tensor:
    """RoPE over ``x[T, NH, D]`` (rotate-half), positions t % seq_len."""
    return ops.apply_rope(x, seq_len, theta)


class MLA(nn.Module):
    def __init__(self, cfg: DeepSeekV3Config, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        h, nh = cfg.hidden_size, cfg.num_heads
        qk = cfg.qk_nope_head_dim + cfg.qk_rope_head_dim
        kw = dict(device=device, dtype=dtype)
        self.wq_a = nn.Parameter(torch.empty(cfg.q_lora_rank, h, **kw))
        self.q_norm = nn.Parameter(torch.empty(cfg.q_lora_rank, **kw))
        self.wq_b = nn.Parameter(torch.empty(nh * qk, cfg.q_lora_rank, **kw))
        self.wkv_a = nn.Parameter(torch.empty(cfg.kv_lora_rank + cfg.qk_rope_head_dim, h, **kw))
        self.kv_norm = nn.Parameter(torch.empty(cfg.kv_lora_rank, **kw))
        self.wkv_b = nn.Parameter(torch.empty(nh * (cfg.qk_nope_head_dim + cfg.v_head_dim), cfg.kv_lora_rank, **kw))
        self.wo = nn.Parameter(torch.empty(h, nh * cfg.v_head_dim, **kw))

    def reset_parameters(self):
        for w in (self.wq_a, self.wq_b, self.wkv_a, self.wkv_b, self.wo):
            nn.init.normal_(w, 0.0, self.cfg.init_std)
        nn.init.ones_(self.q_norm)
        nn.init.ones_(self.kv_norm)

    def forward(self, x: torch.Tensor, batch: int, seq_len: int) -> torch.Tensor:
        c = self.cfg
        nh, dn, dr, dv = c.num_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim
        T = x.shape[0]
        f8 = c.fp8
        # q stays one tensor: RoPE rotates the rotary tail of every head in place; kv is read by the
        # attention kernels as the up-projection left it (k_nope | v per head), the shared rotary key
        # as one vector per token -- no concatenation or expansion on either pass
        q = _lin(ops.rmsnorm(_lin(x, self.wq_a, f8), self.q_norm, c.norm_eps), self.wq_b, f8)
        q = mla_ops.rope_tail_(q.view(T, nh, dn + dr), dr, seq_len, c.rope_theta)
        kv_a = _lin(x, self.wkv_a, f8)
        kv_c, k_rope = kv_a.split([c.kv_lora_rank, dr], dim=-1)
        k_rope = _rope_last(k_rope.contiguous().view(T, 1, dr), seq_len, c.rope_theta)
        kv = _lin(ops.rmsnorm(kv_c.contiguous(), self.kv_norm, c.norm_eps), self.wkv_b, f8)
        o = mla_ops.mla_attention(q.view(batch, seq_len, nh, dn + dr), kv.view(batch, seq_len, nh, dn + dv),
                                  k_rope.view(batch, seq_len, dr), dn, dv)          # [B, S, nh, dv]
        return _lin(o.reshape(T, nh * dv), self.wo, f8)


class DenseFFN(nn.Module):
    def __init__(self, hidden: int, ffn: int, std: float, device=None, dtype=torch.bfloat16, fp8: bool = False):
        super().__init__()
        self.std = std
        self.fp8 = fp8
        self.w_gate_up = nn.Parameter(torch.empty(2 * ffn, hidden, device=device, dtype=dtype))
        self.w_down = nn.Parameter(torch.empty(hidden, ffn, device=device, dtype=dtype))

    def reset_parameters(self):
        nn.init.normal_(self.w_gate_up, 0.0, self.std)
        nn.init.normal_(self.w_down, 0.0, self.std)

    def forward(self, x):
        return _lin(ops.swiglu(_lin(x, self.w_gate_up, self.fp8)), self.w_down, self.fp8)


class MoE(nn.Module):
    """Routed experts (expert-parallel over ``ep_group``) + shared experts."""

    def __init__(self, cfg: DeepSeekV3Config, ep_group=None, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        self.ep_group = ep_group
        self.ep_size = cc.group_size(ep_group)
        self.ep_rank = cc.group_rank(ep_group)
        E = cfg.n_routed_experts
        if E % self.ep_size:
            raise ValueError(f"{E} experts are not divisible by the expert-parallel size {self.ep_size}")
        self.local_experts = E // self.ep_size
        h, f = cfg.hidden_size, cfg.moe_ffn_size
        kw = dict(device=device, dtype=dtype)
        self.gate = nn.Parameter(torch.empty(E, h, device=device, dtype=torch.float32))
        self.register_buffer("gate_bias", torch.zeros(E, device=device, dtype=torch.float32))   # aux-free bias
        self.w_gate_up = nn.Parameter(torch.empty(self.local_experts, 2 * f, h, **kw))
        self.w_down = nn.Parameter(torch.empty(self.local_experts, h, f, **kw))
        self.shared = DenseFFN(h, f * cfg.n_shared_experts, cfg.init_std, device, dtype, cfg.fp8) \
            if cfg.n_shared_experts else None
        # expert weights are expert-parallel, not data-parallel replicas: HSDP must not shard them
        self.w_gate_up.hsdp_shard_size = 1
        self.w_down.hsdp_shard_size = 1
        if self.ep_size > 1 and self.ep_size == cc.get_world_size():
            # every rank owns different experts: there is no data-parallel replica to synchronise with
            self.w_gate_up.hsdp_ignore = True
            self.w_down.hsdp_ignore = True

    def reset_parameters(self):
        # every EP rank draws the full expert tensor and keeps its slice, so that the global
        # initialisation does not depend on the expert-parallel size
        c = self.cfg
        nn.init.normal_(self.gate, 0.0, c.init_std)
        E, f, h = c.n_routed_experts, c.moe_ffn_size, c.hidden_size
        lo = self.ep_rank * self.local_experts
        for w, shape in ((self.w_gate_up, (E, 2 * f, h)), (self.w_down, (E, h, f))):
            if w.shape[0] == E:       # full tensor being initialised (deferred init materialises it)
                nn.init.normal_(w, 0.0, c.init_std)
            else:
                full = torch.empty(shape, dtype=torch.float32, device=w.device).normal_(0.0, c.init_std)
                with torch.no_grad():
                    w.copy_(full[lo:lo + self.local_experts].to(w.dtype))
        if self.gate_bias.device.type != "meta":
            self.gate_bias.zero_()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        topk_idx, topk_w = moe_ops.route(x, self.gate, self.gate_bias, c.top_k, c.n_group, c.topk_group,
                                         c.routed_scaling_factor)
        from ..parallel import ep_fused
        if ep_fused.usable(x, topk_idx, self.w_gate_up, c.n_routed_experts, self.ep_group):
            # dispatch / combine kernels over NVLink peer memory around the grouped expert GEMMs
            cap = c.ep_capacity if c.ep_capacity > 0 else float(min(max(self.ep_size, 2), 4))
            y = ep_fused.fused_expert_parallel_ffn(x, topk_idx, topk_w, self.w_gate_up, self.w_down,
                                                   c.n_routed_experts, self.ep_group, capacity=cap, fp8=c.fp8)
        else:
            y = moe_ops.expert_parallel_ffn(x, topk_idx, topk_w, self.w_gate_up, self.w_down, c.n_routed_experts,
                                            self.ep_group)
        if self.shared is not None:
            y = y + self.shared(x)
        return y


class DeepSeekBlock(nn.Module):
    def __init__(self, cfg: DeepSeekV3Config, layer_idx: int, ep_group=None, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        kw = dict(device=device, dtype=dtype)
        self.attn_norm = nn.Parameter(torch.empty(cfg.hidden_size, **kw))
        self.attn = MLA(cfg, device, dtype)
        self.ffn_norm = nn.Parameter(torch.empty(cfg.hidden_size, **kw))
        self.is_moe = layer_idx >= cfg.first_k_dense
        self.ffn = MoE(cfg, ep_group, device, dtype) if self.is_moe else \
            DenseFFN(cfg.hidden_size, cfg.dense_ffn_size, cfg.init_std, device, dtype, cfg.fp8)

    def reset_parameters(self):
        nn.init.ones_(self.attn_norm)
        nn.init.ones_(self.ffn_norm)

    def forward(self, h, resid, batch: int, seq_len: int):
        c = self.cfg
        if resid is None:
            resid = h
            x = ops.rmsnorm(h, self.attn_norm, c.norm_eps)
        else:
            x, resid = ops.add_rmsnorm(h, resid, self.attn_norm, c.norm_eps)
        a = self.attn(x, batch, seq_len)
        x, resid = ops.add_rmsnorm(a, resid, self.ffn_norm, c.norm_eps)
        return self.ffn(x), resid


class DeepSeekV3(nn.Module):
    def __init__(self, cfg: DeepSeekV3Config, ep_group=None, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        kw = dict(device=device, dtype=dtype)
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.layers = nn.ModuleList(DeepSeekBlock(cfg, i, ep_group, device, dtype) for i in range(cfg.num_layers))
        self.final_norm = nn.Parameter(torch.empty(cfg.hidden_size, **kw))
        self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))

    def reset_parameters(self):
        nn.init.normal_(self.embed, 0.0, self.cfg.init_std)
        nn.init.normal_(self.lm_head, 0.0, self.cfg.init_std)
        nn.init.ones_(self.final_norm)

    def init_weights(self):
        for m in self.modules():
            if hasattr(m, "reset_parameters"):
                m.reset_parameters()

    def forward(self, tokens: torch.Tensor, targets: Optional[torch.Tensor] = None,
                loss_denominator: Optional[float] = None, loss_is_final: bool = True):
        B, S = tokens.shape
        h = ops.embedding(tokens.reshape(-1), self.embed)
        resid = None
        for layer in self.layers:
            h, resid = layer(h, resid, B, S)
        x, _ = ops.add_rmsnorm(h, resid, self.final_norm, self.cfg.norm_eps)
        logits = ops.linear(x, self.lm_head)
        if targets is None:
            return logits.view(B, S, -1)
        return ops.fused_cross_entropy(logits, targets.reshape(-1), loss_denominator, unit_grad=loss_is_final)
