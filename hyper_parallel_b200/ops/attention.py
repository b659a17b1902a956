"""Causal self-attention entry point used by the models.

``causal_attention(q[B,S,H,D], k[B,S,Hkv,D], v[B,S,Hkv,D]) -> [B,S,H,D]`` with
grouped-query support.  The backend is chosen by ``HPB_ATTN``:

* ``cudnn`` (default on CUDA): the fused cuDNN flash-attention graph through
  ``torch.nn.functional.scaled_dot_product_attention``;
* ``flash``: the generic flash backend of the same call;
* ``math``: plain softmax(QK^T)V in fp32 (the CPU path and the test oracle).
"""
from __future__ import annotations

import math
import os

import torch
import torch.nn.functional as F


def _math_attention(q, k, v):
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    qf = q.float().transpose(1, 2)                       # [B,H,S,D]
    kf = k.float().transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    vf = v.float().transpose(1, 2).repeat_interleave(H // Hkv, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, dim=-1) @ vf
    return o.transpose(1, 2).to(q.dtype)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    backend = os.environ.get("HPB_ATTN", "cudnn" if q.is_cuda else "math")
    if backend == "math" or not q.is_cuda:
        return _math_attention(q, k, v)
    from torch.nn.attention import SDPBackend, sdpa_kernel
    H, Hkv = q.shape[2], k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    be = {"cudnn": [SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION],
          "flash": [SDPBackend.FLASH_ATTENTION],
          "efficient": [SDPBackend.EFFICIENT_ATTENTION]}[backend]
    with sdpa_kernel(be):
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=(H != Hkv))
    return o.transpose(1, 2)
