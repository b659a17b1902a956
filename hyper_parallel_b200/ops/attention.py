"""Causal self-attention entry point used by the models.

``causal_attention(q[B,S,H,D], k[B,S,Hkv,D], v[B,S,Hkv,D]) -> [B,S,H,D]`` with
grouped-query support.  The backend is chosen by ``HPB_ATTN``:

* ``hpb`` (default on CUDA for bf16 with head dimension 128): this library's tcgen05
  flash-attention kernels (``attention_sm100.cu``);
* ``cudnn`` (other shapes): the fused cuDNN flash-attention graph through
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


def _strides_ok(t: torch.Tensor) -> bool:
    return (t.stride(3) == 1 and t.stride(2) == t.shape[3] and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def set_forward_variant(p_in_tensor_memory: bool) -> None:
    """Forward kernel variant: P kept in tensor memory (default) or staged through shared memory."""
    from . import native
    native.lib().hpb_flash_attn_set_variant(int(bool(p_in_tensor_memory)))


def flash_attention_forward(q, k, v, causal: bool = True, scale: float = None):
    """tcgen05 flash attention forward: ``(out [B,S,H,128] bf16, lse [B,H,S] fp32)``.

    ``q/k/v`` may be views into a packed projection output (token and batch strides are free, the
    128 head elements must be contiguous and heads 128 elements apart).
    """
    import ctypes
    from . import native
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    assert D == 128 and q.dtype == torch.bfloat16 and k.shape[1] == S
    q, k, v = [t if _strides_ok(t) else t.contiguous() for t in (q, k, v)]
    lib = native.lib()
    if not getattr(lib, "_hpb_fa_bound", False):
        vp, ci, cll, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.hpb_flash_attn_fwd.argtypes = [vp, cll, cll, vp, cll, cll, vp, cll, cll, vp, vp, ci, ci, ci, ci, cf, ci,
                                           vp, vp]
        lib.hpb_flash_attn_fwd.restype = ci
        lib._hpb_fa_bound = True
    out = torch.empty((B, S, H, D), dtype=torch.bfloat16, device=q.device)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    rc = lib.hpb_flash_attn_fwd(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1),
                                v.data_ptr(), v.stride(0), v.stride(1), out.data_ptr(), lse.data_ptr(), B, S, H, Hkv,
                                float(scale if scale is not None else 1.0 / math.sqrt(D)), int(causal),
                                native.status_word(q.device).data_ptr(), native.stream(q.device))
    native.check(rc, "hpb_flash_attn_fwd")
    return out, lse


def _default_backend(q: torch.Tensor) -> str:
    if not q.is_cuda:
        return "math"
    from . import native
    if q.shape[-1] == 128 and q.dtype == torch.bfloat16 and native.available():
        return "hpb"
    return "cudnn"


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    backend = os.environ.get("HPB_ATTN") or _default_backend(q)
    if backend == "math" or not q.is_cuda:
        return _math_attention(q, k, v)
    if backend == "hpb" and q.shape[-1] == 128 and q.dtype == torch.bfloat16:
        return _FlashAttention.apply(q, k, v)
    from torch.nn.attention import SDPBackend, sdpa_kernel
    H, Hkv = q.shape[2], k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    be = {"cudnn": [SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION],
          "flash": [SDPBackend.FLASH_ATTENTION],
          "efficient": [SDPBackend.EFFICIENT_ATTENTION]}[backend]
    with sdpa_kernel(be):
        o = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=(H != Hkv))
    return o.transpose(1, 2)


def flash_attention_backward(q, k, v, out, lse, do, causal: bool = True, scale: float = None, packed: bool = False):
    """tcgen05 flash attention backward: ``(dq, dk, dv)`` bf16 ``[B,S,H,128]``.

    With ``packed=True`` the three gradients are the column ranges ``[dq | dk | dv]`` of ONE
    ``[B, S, (H + 2 Hkv) * 128]`` tensor (returned as a fourth value), which is the gradient of a
    fused qkv projection output without any concatenation copy.
    """
    import ctypes
    from . import native
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    q, k, v, do = [t if _strides_ok(t) else t.contiguous() for t in (q, k, v, do)]
    out = out.contiguous()
    lib = native.lib()
    if not getattr(lib, "_hpb_fa_bwd_bound", False):
        vp, ci, cll, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
        lib.hpb_flash_attn_bwd.argtypes = [vp, cll, cll, vp, cll, cll, vp, cll, cll, vp, vp, vp, cll, cll, vp, vp, vp,
                                           cll, cll, vp, vp, ci, ci, ci, ci, cf, ci, vp, vp]
        lib.hpb_flash_attn_bwd.restype = ci
        lib._hpb_fa_bwd_bound = True
    dev = q.device
    if packed:
        W = (H + 2 * Hkv) * D
        dqkv = torch.empty((B, S, W), dtype=torch.bfloat16, device=dev)
        dq = dqkv[..., :H * D].view(B, S, H, D)
        dk = dqkv[..., H * D:(H + Hkv) * D].view(B, S, Hkv, D)
        dv = dqkv[..., (H + Hkv) * D:].view(B, S, Hkv, D)
        dq_stride = dkv_stride = W
    else:
        dqkv = None
        dq = torch.empty((B, S, H, D), dtype=torch.bfloat16, device=dev)
        dk = torch.empty((B, S, Hkv, D), dtype=torch.bfloat16, device=dev)
        dv = torch.empty((B, S, Hkv, D), dtype=torch.bfloat16, device=dev)
        dq_stride, dkv_stride = H * D, Hkv * D
    dq_acc = torch.empty((B, S, H, D), dtype=torch.float32, device=dev)
    delta = torch.empty((B, H, S), dtype=torch.float32, device=dev)
    rc = lib.hpb_flash_attn_bwd(q.data_ptr(), q.stride(0), q.stride(1), k.data_ptr(), k.stride(0), k.stride(1),
                                v.data_ptr(), v.stride(0), v.stride(1), out.data_ptr(), lse.data_ptr(),
                                do.data_ptr(), do.stride(0), do.stride(1), dq.data_ptr(), dk.data_ptr(),
                                dv.data_ptr(), dq_stride, dkv_stride, dq_acc.data_ptr(), delta.data_ptr(), B, S, H,
                                Hkv, float(scale if scale is not None else 1.0 / math.sqrt(D)), int(causal),
                                native.status_word(dev).data_ptr(), native.stream(dev))
    native.check(rc, "hpb_flash_attn_bwd")
    if packed:
        return dq, dk, dv, dqkv
    return dq, dk, dv


class _FlashAttentionPacked(torch.autograd.Function):
    """Attention on a fused projection output ``qkv[B, S, (H + 2 Hkv) * 128]``: q / k / v are read as
    strided views and the backward writes one packed gradient, so no split / concat copy exists."""

    @staticmethod
    def forward(ctx, qkv, H, Hkv):
        B, S, W = qkv.shape
        D = W // (H + 2 * Hkv)
        q = qkv[..., :H * D].view(B, S, H, D)
        k = qkv[..., H * D:(H + Hkv) * D].view(B, S, Hkv, D)
        v = qkv[..., (H + Hkv) * D:].view(B, S, Hkv, D)
        out, lse = flash_attention_forward(q, k, v, causal=True)
        ctx.save_for_backward(qkv, out, lse)
        ctx.heads = (H, Hkv, D)
        return out

    @staticmethod
    def backward(ctx, do):
        qkv, out, lse = ctx.saved_tensors
        H, Hkv, D = ctx.heads
        B, S, W = qkv.shape
        q = qkv[..., :H * D].view(B, S, H, D)
        k = qkv[..., H * D:(H + Hkv) * D].view(B, S, Hkv, D)
        v = qkv[..., (H + Hkv) * D:].view(B, S, Hkv, D)
        dqkv = flash_attention_backward(q, k, v, out, lse, do, causal=True, packed=True)[3]
        return dqkv, None, None


def causal_attention_packed(qkv: torch.Tensor, num_heads: int, num_kv_heads: int) -> torch.Tensor:
    """``qkv[B, S, (H + 2 Hkv) * D]`` (q heads, then k heads, then v heads) -> ``[B, S, H, D]``."""
    B, S, W = qkv.shape
    D = W // (num_heads + 2 * num_kv_heads)
    backend = os.environ.get("HPB_ATTN") or _default_backend(qkv.view(B, S, -1, D))
    if backend == "hpb" and D == 128 and qkv.dtype == torch.bfloat16 and qkv.is_cuda and qkv.stride(2) == 1 \
            and qkv.stride(1) % 8 == 0 and qkv.stride(0) % 8 == 0 and qkv.data_ptr() % 16 == 0 \
            and os.environ.get("HPB_ATTN_BWD", "hpb") == "hpb":
        return _FlashAttentionPacked.apply(qkv, num_heads, num_kv_heads)
    q, k, v = qkv.split([num_heads * D, num_kv_heads * D, num_kv_heads * D], dim=-1)
    return causal_attention(q.reshape(B, S, num_heads, D) if not q.is_contiguous() else q.view(B, S, num_heads, D),
                            k.reshape(B, S, num_kv_heads, D), v.reshape(B, S, num_kv_heads, D))


class _FlashAttention(torch.autograd.Function):
    """Forward and backward on this library's kernels (``HPB_ATTN_BWD=lib`` recomputes the backward
    through the library call instead)."""

    @staticmethod
    def forward(ctx, q, k, v):
        out, lse = flash_attention_forward(q, k, v, causal=True)
        ctx.save_for_backward(q, k, v, out, lse)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse = ctx.saved_tensors
        if os.environ.get("HPB_ATTN_BWD", "hpb") == "hpb":
            return flash_attention_backward(q, k, v, out, lse, do, causal=True)
        from torch.nn.attention import SDPBackend, sdpa_kernel
        with torch.enable_grad():
            qd, kd, vd = [t.detach().requires_grad_() for t in (q, k, v)]
            with sdpa_kernel([SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION]):
                o = F.scaled_dot_product_attention(qd.transpose(1, 2), kd.transpose(1, 2), vd.transpose(1, 2),
                                                   is_causal=True, enable_gqa=(q.shape[2] != k.shape[2]))
            dq, dk, dv = torch.autograd.grad(o, (qd, kd, vd), do.transpose(1, 2))
        return dq, dk, dv
