"""Multi-head latent attention (DeepSeek-V3 training form) on this library's tcgen05 kernels.

``mla_attention(q, kv, k_rope)`` takes the projections where the model leaves them --

* ``q``      ``[B, S, H, 192]``: 128 "nope" columns then 64 rotary columns per head (RoPE applied),
* ``kv``     ``[B, S, H, 256]``: ``k_nope | v`` per head (the output of the kv up-projection),
* ``k_rope`` ``[B, S, 64]``: the rotary key shared by all heads (RoPE applied)

-- and returns ``o [B, S, H, 128]``; neither the forward nor the backward concatenates or expands
anything: the backward returns ``dq``, ``dkv`` (``dk_nope | dv``, the gradient of the up-projection
output as one tensor) and ``dk_rope`` summed over the heads.  Kernels: ``attention_mla_sm100.cu``
and ``attention_mla_bwd_sm100.cu``.  The reference reaches this shape through
``hyper_parallel/core/shard/ops/parallel_scaled_dot_product_attention.py:32-376`` on library
attention kernels.

Other head widths, other dtypes and CPU tensors take ``mla_attention_reference`` (fp32 math), which
is also the oracle of the tests.  ``rope_tail_`` rotates the last ``D_r`` columns of every head of a
packed projection in place (with autograd), which is what keeps ``q`` one tensor.
"""
from __future__ import annotations

import ctypes
import math
import os
from typing import Optional, Tuple

import torch

DN, DR, DV = 128, 64, 128


def mla_attention_reference(q: torch.Tensor, kv: torch.Tensor, k_rope: torch.Tensor, dn: int, dv: int,
                            causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """fp32 softmax(Q K^T) V with K = k_nope | k_rope (broadcast over heads)."""
    B, S, H, dqk = q.shape
    dr = dqk - dn
    scale = scale if scale is not None else 1.0 / math.sqrt(dqk)
    qf = q.float().transpose(1, 2)                                      # [B, H, S, dqk]
    kn = kv[..., :dn].float().transpose(1, 2)                           # [B, H, S, dn]
    v = kv[..., dn:dn + dv].float().transpose(1, 2)
    kr = k_rope.float().view(B, 1, S, dr)
    s = (qf[..., :dn] @ kn.transpose(-1, -2) + qf[..., dn:] @ kr.transpose(-1, -2)) * scale
    if causal:
        mask = torch.ones(S, S, dtype=torch.bool, device=q.device).tril()
        s = s.masked_fill(~mask, float("-inf"))
    o = torch.softmax(s, dim=-1) @ v
    return o.transpose(1, 2).to(q.dtype)


def _bind(lib):
    if getattr(lib, "_hpb_mla_bound", False):
        return
    vp, ci, cll, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
    lib.hpb_mla_attn_fwd.argtypes = [vp, cll, cll, vp, cll, cll, vp, cll, cll, vp, vp, ci, ci, ci, cf, ci, vp, vp]
    lib.hpb_mla_attn_fwd.restype = ci
    lib.hpb_mla_attn_bwd.argtypes = [vp, cll, cll, vp, cll, cll, vp, cll, cll, vp, vp, vp, cll, cll, vp, vp, vp, vp, vp,
                                     vp, ci, ci, ci, cf, ci, vp, vp]
    lib.hpb_mla_attn_bwd.restype = ci
    lib._hpb_mla_bound = True


def _ok4(t: torch.Tensor) -> bool:
    return (t.stride(3) == 1 and t.stride(2) == t.shape[3] and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def _ok3(t: torch.Tensor) -> bool:
    return t.stride(2) == 1 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0


def native_shape(q: torch.Tensor, kv: torch.Tensor, k_rope: torch.Tensor) -> bool:
    from . import native
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == DN + DR and kv.shape[-1] == DN + DV
            and k_rope.shape[-1] == DR and native.available())


def mla_forward(q, kv, k_rope, causal: bool = True, scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(o [B,S,H,128] bf16, lse [B,H,S] fp32)`` from the tcgen05 forward kernel."""
    from . import native
    B, S, H, _ = q.shape
    q = q if _ok4(q) else q.contiguous()
    kv = kv if _ok4(kv) else kv.contiguous()
    k_rope = k_rope if _ok3(k_rope) else k_rope.contiguous()
    lib = native.lib()
    _bind(lib)
    out = torch.empty((B, S, H, DV), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    rc = lib.hpb_mla_attn_fwd(q.data_ptr(), q.stride(0), q.stride(1), kv.data_ptr(), kv.stride(0), kv.stride(1),
                              k_rope.data_ptr(), k_rope.stride(0), k_rope.stride(1), out.data_ptr(), lse.data_ptr(),
                              B, S, H, float(scale if scale is not None else 1.0 / math.sqrt(DN + DR)), int(causal),
                              native.status_word(q.device).data_ptr(), native.stream(q.device))
    native.check(rc, "hpb_mla_attn_fwd")
    return out, lse


def mla_backward(q, kv, k_rope, out, lse, do, causal: bool = True, scale: Optional[float] = None):
    """``(dq [B,S,H,192], dkv [B,S,H,256], dk_rope [B,S,64])`` bf16 from the tcgen05 backward kernel."""
    from . import native
    B, S, H, _ = q.shape
    q = q if _ok4(q) else q.contiguous()
    kv = kv if _ok4(kv) else kv.contiguous()
    do = do if _ok4(do) else do.contiguous()
    k_rope = k_rope if _ok3(k_rope) else k_rope.contiguous()
    out = out.contiguous()
    lib = native.lib()
    _bind(lib)
    dev = q.device
    dq = torch.empty((B, S, H, DN + DR), dtype=torch.bfloat16, device=dev)
    dkv = torch.empty((B, S, H, DN + DV), dtype=torch.bfloat16, device=dev)
    dkr = torch.empty((B, S, DR), dtype=torch.bfloat16, device=dev)
    dq_acc = torch.empty((B, S, H, DN + DR), dtype=torch.float32, device=dev)
    delta = torch.empty((B, H, S), dtype=torch.float32, device=dev)
    dkr_heads = torch.empty((B, S, H, DR), dtype=torch.bfloat16, device=dev)
    rc = lib.hpb_mla_attn_bwd(q.data_ptr(), q.stride(0), q.stride(1), kv.data_ptr(), kv.stride(0), kv.stride(1),
                              k_rope.data_ptr(), k_rope.stride(0), k_rope.stride(1), out.data_ptr(), lse.data_ptr(),
                              do.data_ptr(), do.stride(0), do.stride(1), dq.data_ptr(), dkv.data_ptr(),
                              dkr.data_ptr(), dq_acc.data_ptr(), delta.data_ptr(), dkr_heads.data_ptr(), B, S, H,
                              float(scale if scale is not None else 1.0 / math.sqrt(DN + DR)), int(causal),
                              native.status_word(dev).data_ptr(), native.stream(dev))
    native.check(rc, "hpb_mla_attn_bwd")
    return dq, dkv, dkr


class _MLAAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, kv, k_rope, causal, scale):
        out, lse = mla_forward(q, kv, k_rope, causal, scale)
        ctx.save_for_backward(q, kv, k_rope, out, lse)
        ctx.causal, ctx.scale = causal, scale
        return out

    @staticmethod
    def backward(ctx, do):
        q, kv, k_rope, out, lse = ctx.saved_tensors
        dq, dkv, dkr = mla_backward(q, kv, k_rope, out, lse, do, ctx.causal, ctx.scale)
        return dq, dkv, dkr, None, None


def mla_attention(q: torch.Tensor, kv: torch.Tensor, k_rope: torch.Tensor, dn: int = DN, dv: int = DV,
                  causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Attention over ``q [B,S,H,dn+dr]``, ``kv [B,S,H,dn+dv]``, ``k_rope [B,S,dr]`` -> ``[B,S,H,dv]``.

    ``HPB_MLA=ref`` forces the fp32 reference; the kernels serve dn = 128, dr = 64, dv = 128 in bf16.
    """
    mode = os.environ.get("HPB_MLA", "hpb")
    if mode == "hpb" and dn == DN and dv == DV and native_shape(q, kv, k_rope):
        return _MLAAttention.apply(q, kv, k_rope, causal, scale)
    if mode == "ref" or not causal or scale is not None:
        return mla_attention_reference(q, kv, k_rope, dn, dv, causal, scale)
    # other widths: the expanded form through the generic entry point (library attention on CUDA)
    from .attention import causal_attention
    B, S, H, dqk = q.shape
    kh = torch.cat([kv[..., :dn], k_rope.view(B, S, 1, dqk - dn).expand(B, S, H, dqk - dn)], dim=-1)
    return causal_attention(q, kh, kv[..., dn:dn + dv].contiguous())


class _RopeTail(torch.autograd.Function):
    """RoPE on the last ``dr`` columns of every head of ``x[T, NH, D]``, in place."""

    @staticmethod
    def forward(ctx, x, dr, seq_len, theta):
        from . import functional as Fn
        ctx.dr, ctx.seq_len, ctx.theta = dr, seq_len, theta
        ctx.mark_dirty(x)
        Fn.rope_(x[..., x.shape[-1] - dr:], seq_len, theta)
        return x

    @staticmethod
    def backward(ctx, dy):
        from . import functional as Fn
        dx = dy.clone(memory_format=torch.contiguous_format)
        Fn.rope_(dx[..., dx.shape[-1] - ctx.dr:], ctx.seq_len, ctx.theta, inverse=True)
        return dx, None, None, None


def rope_tail_(x: torch.Tensor, dr: int, seq_len: int, theta: float) -> torch.Tensor:
    """Rotate the last ``dr`` columns of every head of ``x[T, NH, D]`` (positions ``t % seq_len``) in
    place and return ``x``; differentiable (the input must not be needed by the op that produced it,
    which holds for a projection output)."""
    return _RopeTail.apply(x, dr, seq_len, theta)
