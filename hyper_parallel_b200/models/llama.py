"""Llama-family dense decoder (GQA, RoPE, SwiGLU, RMSNorm) built on the sm_100a kernels.

The reference ships no model code; this module provides the architectures its
benchmarks are quoted on (Llama-3-8B, Llama-2-13B shapes).  Projections are stored
fused (``wqkv``, ``w_gate_up``) so that each block runs four GEMMs; residual adds
are fused into the RMSNorm kernels; RoPE rotates q/k in place inside the fused QKV
buffer; the loss is a fused softmax-cross-entropy that produces dlogits in the
forward pass.  On CPU tensors every op falls back to its PyTorch formulation, which
is what the CPU tests (and the oracle) run.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..ops import attention as attn_ops


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    num_layers: int = 32
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    ffn_size: int = 14336
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    init_std: float = 0.02
    tie_embeddings: bool = False

    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama2_13b() -> "LlamaConfig":
        return LlamaConfig(vocab_size=32000, hidden_size=5120, num_layers=40, num_heads=40,
                           num_kv_heads=40, head_dim=128, ffn_size=13824, rope_theta=10000.0)

    @staticmethod
    def tiny(vocab_size=512, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2,
             head_dim=64, ffn_size=512) -> "LlamaConfig":
        return LlamaConfig(vocab_size, hidden_size, num_layers, num_heads, num_kv_heads, head_dim,
                           ffn_size)

    def num_params(self) -> int:
        h, L = self.hidden_size, self.num_layers
        qkv = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim * h
        per_layer = qkv + self.num_heads * self.head_dim * h + 3 * h * self.ffn_size + 2 * h
        emb = self.vocab_size * h * (1 if self.tie_embeddings else 2)
        return L * per_layer + emb + h

    def flops_per_token(self, seq_len: int) -> float:
        """Training FLOPs per token: 6 * matmul params + causal attention (fwd + bwd)."""
        h, L = self.hidden_size, self.num_layers
        qkv = (self.num_heads + 2 * self.num_kv_heads) * self.head_dim * h
        mm = L * (qkv + self.num_heads * self.head_dim * h + 3 * h * self.ffn_size) + self.vocab_size * h
        attn = L * 12 * self.num_heads * self.head_dim * seq_len / 2  # 4*S*d fwd, x3 with bwd, causal half
        return 6.0 * mm + attn


class _RopeQK(torch.autograd.Function):
    """Rotate the q and k column blocks of the fused ``qkv[T, (nh + 2 nkv) * hd]`` buffer in place."""

    @staticmethod
    def forward(ctx, qkv, nh, nkv, hd, seq_len, theta):
        ctx.meta = (nh, nkv, hd, seq_len, theta)
        T = qkv.shape[0]
        ops.rope_(qkv.as_strided((T, nh + nkv, hd), (qkv.stride(0), hd, 1)), seq_len, theta)
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, g):
        nh, nkv, hd, seq_len, theta = ctx.meta
        # the incoming gradient is the freshly concatenated (dq, dk, dv) buffer of the split that
        # is the only consumer of the rotated qkv: rotating it in place saves a 100 MB copy
        g = g.contiguous()
        T = g.shape[0]
        ops.rope_(g.as_strided((T, nh + nkv, hd), (g.stride(0), hd, 1)), seq_len, theta, inverse=True)
        return g, None, None, None, None, None


class LlamaBlock(nn.Module):
    """One pre-norm decoder block.  ``forward(h, resid)`` takes the previous block's un-added
    output ``h`` and the residual stream ``resid`` and returns the same pair."""

    def __init__(self, cfg: LlamaConfig, layer_idx: int, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        h, hd = cfg.hidden_size, cfg.head_dim
        kw = dict(device=device, dtype=dtype)
        self.attn_norm = nn.Parameter(torch.empty(h, **kw))
        self.wqkv = nn.Parameter(torch.empty((cfg.num_heads + 2 * cfg.num_kv_heads) * hd, h, **kw))
        self.wo = nn.Parameter(torch.empty(h, cfg.num_heads * hd, **kw))
        self.ffn_norm = nn.Parameter(torch.empty(h, **kw))
        self.w_gate_up = nn.Parameter(torch.empty(2 * cfg.ffn_size, h, **kw))
        self.w_down = nn.Parameter(torch.empty(h, cfg.ffn_size, **kw))
        # these matrices are only ever consumed by ops.linear: HSDP may gather them inside the GEMM
        for w in (self.wqkv, self.wo, self.w_gate_up, self.w_down):
            w._hpb_gemm_only = True

    def reset_parameters(self):
        std = self.cfg.init_std
        for w in (self.wqkv, self.wo, self.w_gate_up, self.w_down):
            nn.init.normal_(w, mean=0.0, std=std)
        nn.init.ones_(self.attn_norm)
        nn.init.ones_(self.ffn_norm)

    def forward(self, h: torch.Tensor, resid: Optional[torch.Tensor], batch: int, seq_len: int):
        cfg = self.cfg
        nh, nkv, hd = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim
        if resid is None:
            resid = h
            x = ops.rmsnorm(h, self.attn_norm, cfg.norm_eps)
        else:
            x, resid = ops.add_rmsnorm(h, resid, self.attn_norm, cfg.norm_eps)
        qkv = ops.linear(x, self.wqkv)                      # [T, (nh + 2 nkv) hd]
        if qkv.is_cuda:
            qkv = _RopeQK.apply(qkv, nh, nkv, hd, seq_len, cfg.rope_theta)
            # attention reads q / k / v as views of the packed projection output and returns one
            # packed gradient: no split / concatenation copies
            a = attn_ops.causal_attention_packed(qkv.view(batch, seq_len, -1), nh, nkv)
            q = None
        else:
            q, k, v = qkv.split([nh * hd, nkv * hd, nkv * hd], dim=-1)
            q = ops.apply_rope(q.reshape(-1, nh, hd), seq_len, cfg.rope_theta).reshape(-1, nh * hd)
            k = ops.apply_rope(k.reshape(-1, nkv, hd), seq_len, cfg.rope_theta).reshape(-1, nkv * hd)
        if q is not None:
            a = attn_ops.causal_attention(q.view(batch, seq_len, nh, hd), k.view(batch, seq_len, nkv, hd),
                                          v.view(batch, seq_len, nkv, hd))
        o = ops.linear(a.reshape(batch * seq_len, nh * hd), self.wo)
        x, resid = ops.add_rmsnorm(o, resid, self.ffn_norm, cfg.norm_eps)
        gu = ops.linear(x, self.w_gate_up)
        act = ops.swiglu(gu)
        d = ops.linear(act, self.w_down)
        return d, resid


class Llama(nn.Module):
    """Decoder-only LM.  ``forward(tokens[B, S], targets[B, S])`` returns the mean token loss;
    without targets it returns the logits."""

    def __init__(self, cfg: LlamaConfig, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.cfg = cfg
        kw = dict(device=device, dtype=dtype)
        self.embed = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
        self.layers = nn.ModuleList(LlamaBlock(cfg, i, device, dtype) for i in range(cfg.num_layers))
        self.final_norm = nn.Parameter(torch.empty(cfg.hidden_size, **kw))
        if cfg.tie_embeddings:
            self.lm_head = self.embed
        else:
            self.lm_head = nn.Parameter(torch.empty(cfg.vocab_size, cfg.hidden_size, **kw))
            self.lm_head._hpb_gemm_only = True
            self.lm_head._hpb_gather_late = True      # consumed at the very end of the forward pass

    def reset_parameters(self):
        nn.init.normal_(self.embed, mean=0.0, std=self.cfg.init_std)
        if not self.cfg.tie_embeddings:
            nn.init.normal_(self.lm_head, mean=0.0, std=self.cfg.init_std)
        nn.init.ones_(self.final_norm)

    def init_weights(self):
        """Initialise every parameter (N(0, init_std) matrices, unit norms)."""
        self.reset_parameters()
        for layer in self.layers:
            layer.reset_parameters()

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
