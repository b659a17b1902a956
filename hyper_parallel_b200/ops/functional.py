"""Autograd-aware operators backed by the hand-written sm_100a kernels.

Each operator has two paths: CUDA tensors run the native kernels in
``libhpb200.so`` (tcgen05 GEMM, fused norm / activation / loss / optimizer
kernels); CPU tensors run an equivalent plain-PyTorch formulation, which is also
the oracle the GPU tests compare against.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import native

__all__ = [
    "gemm", "linear", "matmul", "rmsnorm", "add_rmsnorm", "swiglu", "rope_", "apply_rope",
    "cross_entropy_fwd_bwd", "fused_cross_entropy", "adamw_step_", "embedding",
]


# --------------------------------------------------------------------- GEMM --
import os as _os

_PAIR_MODE = _os.environ.get("HPB_GEMM_PAIR", "auto")     # "0" single-CTA kernel, "1" CTA pairs, "auto" by size


def set_gemm_pair_mode(mode: str) -> None:
    """Select the GEMM kernel: ``"0"`` 128x256 single-CTA, ``"1"`` 256x256 CTA pairs, ``"auto"``."""
    global _PAIR_MODE
    _PAIR_MODE = mode


_RIDE_PROVIDER = None      # callable(device, flops) -> gather spec that this GEMM should carry, or None
_RIDE_ORDERS = {(False, False), (False, True), (True, True)}


def set_ride_provider(fn) -> None:
    """HSDP over symmetric memory registers the source of weight gathers that ride on GEMM launches
    (the communication warps of the GEMM kernel copy a later GEMM's weight while the tensor cores
    work on this one)."""
    global _RIDE_PROVIDER
    _RIDE_PROVIDER = fn


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
         accumulate: bool = False) -> torch.Tensor:
    """``C[M,N] (+)= opA @ opB^T`` on the tcgen05 tensor cores.

    ``a`` is stored ``[M,K]`` (``a_mn=False``) or ``[K,M]`` (``a_mn=True``); ``b``
    is stored ``[N,K]`` or ``[K,N]`` likewise.  Inputs are 2-D bf16 with unit
    inner stride; the result is bf16 or fp32.
    """
    assert a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        assert not accumulate
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if not native.use_native(a):
        fa = (a.t() if a_mn else a).float()
        fb = (b if b_mn else b.t()).float()
        res = fa @ fb
        if accumulate:
            res = res + out.float()
        out.copy_(res.to(out.dtype))
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    if a.stride(-1) != 1 or (a.stride(0) % 8) or (a.data_ptr() % 16):
        a = a.contiguous()
    if b.stride(-1) != 1 or (b.stride(0) % 8) or (b.data_ptr() % 16):
        b = b.contiguous()
    assert out.stride(-1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    if M == 0 or N == 0:
        return out
    if K == 0:
        if not accumulate:
            out.zero_()
        return out
    dev = a.device
    lib = native.lib()
    # CTA-pair (256x256, cta_group::2) kernel for large problems, single-CTA 128x256 otherwise
    use_pair = _PAIR_MODE == "1" or (_PAIR_MODE == "auto" and M >= 512 and N >= 512 and hasattr(lib, "hpb_gemm2_bf16"))
    if (use_pair and _RIDE_PROVIDER is not None and out.dtype == torch.bfloat16 and (a_mn, b_mn) in _RIDE_ORDERS
            and (not accumulate or (a_mn and b_mn))):
        ride = _RIDE_PROVIDER(dev, 2.0 * M * N * K)
        if ride is not None:
            import ctypes
            rc = lib.hpb_gemm2_gather(a.data_ptr(), int(a_mn), a.stride(0), b.data_ptr(), int(b_mn), b.stride(0),
                                      out.data_ptr(), out.stride(0), int(accumulate), M, N, K, None, 0,
                                      ctypes.byref(ride), 2_000_000_000, native.status_word(dev).data_ptr(),
                                      native.sm_count(dev), native.stream(dev))
            native.check(rc, "hpb_gemm2_gather")
            return out
    fn = lib.hpb_gemm2_bf16 if use_pair else lib.hpb_gemm_bf16
    rc = fn(a.data_ptr(), int(a_mn), a.stride(0), b.data_ptr(), int(b_mn), b.stride(0),
            out.data_ptr(), out.stride(0), int(out.dtype == torch.float32), int(accumulate),
            M, N, K, native.status_word(dev).data_ptr(), native.sm_count(dev), native.stream(dev))
    native.check(rc, "hpb_gemm2_bf16" if use_pair else "hpb_gemm_bf16")
    return out


class _Linear(torch.autograd.Function):
    """y = x W^T with all three GEMMs on the tcgen05 kernel (no transposes)."""

    @staticmethod
    def forward(ctx, x, w, wgrad_into, symm):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        ctx.wgrad_into = wgrad_into
        ctx.symm = symm
        # allocate with the final shape: the result must not be a view created inside the Function
        # (callers may update it in place, e.g. RoPE on the fused QKV buffer)
        y = torch.empty(*x.shape[:-1], w.shape[0], dtype=torch.bfloat16, device=x.device)
        hs = getattr(w, "_hpb_symm", None)
        if hs is not None and hs[0].gather_pending(hs[1]):
            # HSDP: the weight has not been gathered yet -- this product gathers it from the peers
            # inside the GEMM kernel (the all-gather is fused into its first consumer)
            hs[0].gather_gemm(hs[1], x2, y.view(-1, w.shape[0]), w_mn=False)
        else:
            gemm(x2, w, out=y.view(-1, w.shape[0]))
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = dw = None
        hs = getattr(w, "_hpb_symm", None)
        if ctx.needs_input_grad[0]:
            if hs is not None and hs[0].gather_pending(hs[1]):
                # level-3 backward: the input-gradient product is the first consumer of the
                # re-gathered weight
                dx = torch.empty((dy2.shape[0], w.shape[1]), dtype=torch.bfloat16, device=dy2.device)
                hs[0].gather_gemm(hs[1], dy2, dx, w_mn=True)
                dx = dx.view(ctx.x_shape)
            else:
                dx = gemm(dy2, w, b_mn=True).view(ctx.x_shape)
        if ctx.needs_input_grad[1] and ctx.symm is not None:
            # HSDP over symmetric memory: the epilogue writes dW into the flat gradient buffer that
            # the fused reduce-scatter + AdamW kernel of every peer reads
            buf, i = ctx.symm
            view, acc = buf.wgrad_target(i)
            gemm(dy2, x2, a_mn=True, b_mn=True, out=view, accumulate=acc)
            if buf.mark_ready(i):
                buf.on_all_ready()
        elif ctx.needs_input_grad[1]:
            tgt = ctx.wgrad_into
            if tgt is not None:
                # fused gradient accumulation: dW is added straight into the
                # (fp32 or bf16) main-grad buffer by the GEMM epilogue
                gemm(dy2, x2, a_mn=True, b_mn=True, out=tgt, accumulate=True)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw, None, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None,
           wgrad_into: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)``; bf16 CUDA inputs use the tcgen05 GEMM for fwd/dgrad/wgrad."""
    if native.use_native(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        symm = getattr(w, "_hpb_symm", None) if (w.requires_grad and torch.is_grad_enabled()) else None
        y = _Linear.apply(x, w, wgrad_into, symm)
        return y if bias is None else y + bias
    hs = getattr(w, "_hpb_symm", None)
    if hs is not None and hs[0].gather_pending(hs[1]):
        hs[0].materialize(hs[1])
    return F.linear(x, w, bias)


class _MatMul(torch.autograd.Function):
    """y = x W with W stored [K, N]: forward, dgrad and wgrad on the tcgen05 GEMM, no transposes."""

    @staticmethod
    def forward(ctx, x, w):
        x2 = x.reshape(-1, x.shape[-1])
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        y = torch.empty(*x.shape[:-1], w.shape[1], dtype=torch.bfloat16, device=x.device)
        gemm(x2, w, b_mn=True, out=y.view(-1, w.shape[1]))
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dx = gemm(dy2, w).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = gemm(x2, dy2, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, dw


def matmul(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w`` for ``x[..., K]`` and a 2-D ``w[K, N]``; bf16 CUDA operands use the tcgen05 GEMM."""
    if (native.use_native(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2
            and x.dim() >= 2 and w.is_contiguous()):
        return _MatMul.apply(x, w)
    return torch.matmul(x, w)


# ------------------------------------------------------------------ RMSNorm --
def _rmsnorm_ref(x, w, eps, res=None):
    h = x if res is None else (x.float() + res.float()).to(x.dtype)
    hf = h.float()
    rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    y = (hf * rstd * w.float()).to(x.dtype)
    return y, h


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, res, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H).contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, dtype=torch.float32, device=x.device)
        h = None
        r2 = None
        if res is not None:
            r2 = res.reshape(-1, H).contiguous()
            h = torch.empty_like(x2)
        rc = native.lib().hpb_rmsnorm_fwd(x2.data_ptr(), native.ptr(r2), w.data_ptr(), y.data_ptr(),
                                          native.ptr(h), rstd.data_ptr(), T, H, eps,
                                          native.stream(x.device))
        native.check(rc, "hpb_rmsnorm_fwd")
        src = h if h is not None else x2
        ctx.save_for_backward(src, w, rstd)
        ctx.has_res = res is not None
        ctx.shape = x.shape
        if res is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        src, w, rstd = ctx.saved_tensors
        T, H = src.shape
        dy2 = dy.reshape(T, H).contiguous()
        dh2 = dh.reshape(T, H).contiguous() if (ctx.has_res and dh is not None) else None
        dx = torch.empty_like(src)
        P = min(T, native.sm_count(src.device) * 8)
        part = torch.empty((P, H), dtype=torch.float32, device=src.device)
        dw = torch.empty_like(w)
        rc = native.lib().hpb_rmsnorm_bwd(dy2.data_ptr(), src.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                          native.ptr(dh2), dx.data_ptr(), part.data_ptr(), P,
                                          dw.data_ptr(), int(dw.dtype == torch.float32), 0, T, H,
                                          native.stream(src.device))
        native.check(rc, "hpb_rmsnorm_bwd")
        dx = dx.view(ctx.shape)
        return dx, dw, (dx if ctx.has_res else None), None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """RMSNorm over the last dim: ``x * rsqrt(mean(x^2) + eps) * w``."""
    if native.use_native(x) and x.dtype == torch.bfloat16:
        return _RMSNorm.apply(x, w, None, eps)[0]
    return _rmsnorm_ref(x, w, eps)[0]


def add_rmsnorm(x: torch.Tensor, res: torch.Tensor, w: torch.Tensor,
                eps: float = 1e-5) -> Tuple[torch.Tensor, torch.Tensor]:
    """Fused residual add + RMSNorm.  Returns ``(norm(x + res), x + res)``."""
    if native.use_native(x) and x.dtype == torch.bfloat16:
        return _RMSNorm.apply(x, w, res, eps)
    return _rmsnorm_ref(x, w, eps, res)


# ------------------------------------------------------------------- SwiGLU --
class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        F2 = gu.shape[-1]
        g2 = gu.reshape(-1, F2).contiguous()
        T = g2.shape[0]
        out = torch.empty((T, F2 // 2), dtype=gu.dtype, device=gu.device)
        rc = native.lib().hpb_swiglu_fwd(g2.data_ptr(), out.data_ptr(), T, F2 // 2,
                                         native.sm_count(gu.device), native.stream(gu.device))
        native.check(rc, "hpb_swiglu_fwd")
        ctx.save_for_backward(g2)
        ctx.shape = gu.shape
        return out.view(*gu.shape[:-1], F2 // 2)

    @staticmethod
    def backward(ctx, dout):
        (g2,) = ctx.saved_tensors
        T, F2 = g2.shape
        d2 = dout.reshape(T, F2 // 2).contiguous()
        dgu = torch.empty_like(g2)
        rc = native.lib().hpb_swiglu_bwd(g2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), T, F2 // 2,
                                         native.sm_count(g2.device), native.stream(g2.device))
        native.check(rc, "hpb_swiglu_bwd")
        return dgu.view(ctx.shape)


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` where ``gate_up[..., :F]`` is the gate and ``[..., F:]`` is up."""
    if native.use_native(gate_up) and gate_up.dtype == torch.bfloat16:
        return _SwiGLU.apply(gate_up)
    g, u = gate_up.chunk(2, dim=-1)
    return (F.silu(g.float()) * u.float()).to(gate_up.dtype)


# --------------------------------------------------------------------- RoPE --
def _rope_ref(x, seq_len, theta, positions=None, inverse=False):
    # x: [T, NH, D]; pairs (i, i + D/2)
    T, NH, D = x.shape
    half = D // 2
    pos = (torch.arange(T, device=x.device) % seq_len) if positions is None else positions
    inv = torch.exp2(-math.log2(theta) * (2.0 * torch.arange(half, device=x.device, dtype=torch.float32)) / D)
    ang = pos.float()[:, None] * inv[None, :]
    cs, sn = ang.cos()[:, None, :], ang.sin()[:, None, :]
    if inverse:
        sn = -sn
    a, b = x[..., :half].float(), x[..., half:].float()
    return torch.cat([a * cs - b * sn, b * cs + a * sn], dim=-1).to(x.dtype)


_ROPE_TABLES = {}


def _rope_table(seq_len: int, D: int, theta: float, device) -> torch.Tensor:
    """(cos, sin) of every (position, frequency) pair, built once per configuration on the device."""
    key = (seq_len, D, theta, str(device))
    t = _ROPE_TABLES.get(key)
    if t is None:
        t = torch.empty(seq_len * (D // 2) * 2, dtype=torch.float32, device=device)
        rc = native.lib().hpb_rope_table(t.data_ptr(), seq_len, D, theta, native.stream(device))
        native.check(rc, "hpb_rope_table")
        _ROPE_TABLES[key] = t
    return t


def rope_(x: torch.Tensor, seq_len: int, theta: float, positions: Optional[torch.Tensor] = None,
          inverse: bool = False) -> torch.Tensor:
    """In-place rotary embedding of ``x[T, NH, D]`` (token stride may exceed ``NH*D``; the heads may be
    further apart than ``D``, e.g. the rotary tail of every head of a packed projection)."""
    T, NH, D = x.shape
    if not native.use_native(x):
        x.copy_(_rope_ref(x, seq_len, theta, positions, inverse))
        return x
    if x.dtype != torch.bfloat16 or x.stride(2) != 1:
        x.copy_(_rope_ref(x, seq_len, theta, positions, inverse))     # other dtypes / layouts: reference math
        return x
    if x.stride(1) != D:
        if not (D % 16 == 0 and x.stride(0) % 8 == 0 and x.stride(1) % 8 == 0 and x.data_ptr() % 16 == 0
                and positions is None):
            x.copy_(_rope_ref(x, seq_len, theta, positions, inverse))
            return x
        table = _rope_table(seq_len, D, float(theta), x.device)
        rc = native.lib().hpb_rope_vec_strided(x.data_ptr(), table.data_ptr(), None, T, seq_len, NH, D, x.stride(0),
                                               x.stride(1), int(inverse), native.sm_count(x.device),
                                               native.stream(x.device))
        native.check(rc, "hpb_rope_vec_strided")
        return x
    pos_ptr = None
    if positions is not None:
        positions = positions.to(torch.int32).contiguous()
        pos_ptr = positions.data_ptr()
    if D % 16 == 0 and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and positions is None:
        table = _rope_table(seq_len, D, float(theta), x.device)
        rc = native.lib().hpb_rope_vec(x.data_ptr(), table.data_ptr(), None, T, seq_len, NH, D, x.stride(0),
                                       int(inverse), native.sm_count(x.device), native.stream(x.device))
        native.check(rc, "hpb_rope_vec")
        return x
    rc = native.lib().hpb_rope(x.data_ptr(), pos_ptr, T, seq_len, NH, D, x.stride(0), float(theta),
                               int(inverse), native.sm_count(x.device), native.stream(x.device))
    native.check(rc, "hpb_rope")
    return x


class _RoPE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_len, theta):
        ctx.seq_len, ctx.theta = seq_len, theta
        y = x.clone()
        rope_(y, seq_len, theta)
        return y

    @staticmethod
    def backward(ctx, dy):
        dx = dy.clone(memory_format=torch.contiguous_format)
        rope_(dx, ctx.seq_len, ctx.theta, inverse=True)
        return dx, None, None


def apply_rope(x: torch.Tensor, seq_len: int, theta: float) -> torch.Tensor:
    """Out-of-place rotary embedding with autograd; ``x`` is ``[T, NH, D]``, position = t % seq_len."""
    if native.use_native(x):
        return _RoPE.apply(x.contiguous(), seq_len, theta)
    return _rope_ref(x, seq_len, theta)


# ---------------------------------------------------------------- embedding --
class _Embedding(torch.autograd.Function):
    """Row gather forward; deterministic dense weight gradient backward (``embedding.cu``)."""

    @staticmethod
    def forward(ctx, tokens, weight):
        T = tokens.numel()
        V, H = weight.shape
        idx = tokens.reshape(-1).to(torch.int64).contiguous()
        out = torch.empty((T, H), dtype=weight.dtype, device=weight.device)
        dev = weight.device
        rc = native.lib().hpb_embedding_fwd(idx.data_ptr(), weight.data_ptr(), out.data_ptr(), T, V, H,
                                            native.status_word(dev).data_ptr(), native.sm_count(dev), native.stream(dev))
        native.check(rc, "hpb_embedding_fwd")
        ctx.save_for_backward(idx)
        ctx.shape = (V, H)
        return out.view(*tokens.shape, H)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        V, H = ctx.shape
        dy2 = dy.reshape(-1, H).contiguous()
        dev = dy2.device
        T = idx.numel()
        dw = torch.empty((V, H), dtype=dy2.dtype, device=dev)
        scratch = torch.empty(3 * V + T, dtype=torch.int32, device=dev)
        rc = native.lib().hpb_embedding_bwd(idx.data_ptr(), dy2.data_ptr(), dw.data_ptr(), scratch.data_ptr(), T, V, H,
                                            native.status_word(dev).data_ptr(), native.sm_count(dev), native.stream(dev))
        native.check(rc, "hpb_embedding_bwd")
        return None, dw


def embedding(tokens: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``weight[tokens]`` -> ``[*tokens.shape, H]``.  bf16 CUDA weights with ``H % 8 == 0`` take this
    library's kernels (the weight gradient is dense, written once per row, and bit-identical from
    run to run); everything else takes ``torch.nn.functional.embedding``."""
    if (native.use_native(weight) and weight.dtype == torch.bfloat16 and weight.dim() == 2 and weight.is_contiguous()
            and weight.shape[1] % 8 == 0 and type(weight) in (torch.Tensor, torch.nn.Parameter)):
        return _Embedding.apply(tokens, weight)
    return F.embedding(tokens, weight)


# ------------------------------------------------------------ cross entropy --
def cross_entropy_fwd_bwd(logits: torch.Tensor, target: torch.Tensor,
                          grad_scale: float) -> torch.Tensor:
    """Per-token loss; overwrites ``logits`` in place with ``grad_scale * dloss/dlogits``."""
    T, V = logits.shape
    if not native.use_native(logits):
        lf = logits.float()
        lse = torch.logsumexp(lf, dim=-1)
        valid = (target >= 0) & (target < V)
        safe = target.clamp(0, V - 1)
        loss = torch.where(valid, lse - lf.gather(1, safe[:, None])[:, 0], torch.zeros_like(lse))
        p = torch.exp(lf - lse[:, None])
        p[torch.arange(T), safe] -= 1.0
        p = p * torch.where(valid, grad_scale, 0.0)[:, None]
        logits.copy_(p.to(logits.dtype))
        return loss
    assert logits.dtype == torch.bfloat16 and logits.stride(1) == 1
    target = target.to(torch.int64).contiguous()
    loss = torch.empty(T, dtype=torch.float32, device=logits.device)
    rc = native.lib().hpb_cross_entropy(logits.data_ptr(), target.data_ptr(), loss.data_ptr(), T, V,
                                        logits.stride(0), float(grad_scale),
                                        native.stream(logits.device))
    native.check(rc, "hpb_cross_entropy")
    return loss


class _FusedCE(torch.autograd.Function):
    """Mean token cross-entropy whose backward was already computed in the forward kernel."""

    @staticmethod
    def forward(ctx, logits, target, denom, unit_grad):
        loss = cross_entropy_fwd_bwd(logits, target, 1.0 / denom)
        ctx.save_for_backward(logits)  # now holds dlogits (for grad_out == 1)
        ctx.unit_grad = unit_grad
        return loss.sum() / denom

    @staticmethod
    def backward(ctx, g):
        (dlogits,) = ctx.saved_tensors
        if ctx.unit_grad:
            # the caller promised that this loss is what backward() is called on (upstream
            # gradient 1): the stored dlogits are final and a 2 GB rescale pass is skipped
            return dlogits, None, None, None
        return dlogits * g.to(dlogits.dtype), None, None, None


def fused_cross_entropy(logits: torch.Tensor, target: torch.Tensor, denom: Optional[float] = None,
                        unit_grad: bool = False) -> torch.Tensor:
    """``sum(CE(logits, target)) / denom``; consumes (overwrites) ``logits``.

    ``unit_grad=True`` states that ``backward()`` will be called on this very value (upstream
    gradient exactly 1; scale the loss through ``denom`` instead of multiplying it afterwards).
    """
    T = logits.shape[0]
    return _FusedCE.apply(logits, target, float(denom if denom is not None else T), unit_grad)


# -------------------------------------------------------------------- AdamW --
def adamw_step_(param_bf16: Optional[torch.Tensor], master: torch.Tensor, exp_avg: torch.Tensor,
                exp_avg_sq: torch.Tensor, grad: torch.Tensor, *, lr: float, beta1: float,
                beta2: float, eps: float, weight_decay: float, step: int,
                grad_scale: float = 1.0) -> None:
    """Fused AdamW on flat buffers: fp32 master / moments, optional bf16 model copy."""
    n = master.numel()
    if not native.use_native(master):
        g = grad.float().reshape(-1) * grad_scale
        exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
        exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        upd = (exp_avg / bc1) / ((exp_avg_sq / bc2).sqrt() + eps)
        master.mul_(1 - lr * weight_decay).add_(upd, alpha=-lr)
        if param_bf16 is not None:
            param_bf16.copy_(master.to(param_bf16.dtype))
        return
    assert master.dtype == torch.float32 and grad.dtype in (torch.bfloat16, torch.float32)
    assert master.is_contiguous() and exp_avg.is_contiguous() and exp_avg_sq.is_contiguous()
    assert grad.is_contiguous() and grad.numel() == n
    rc = native.lib().hpb_adamw(grad.data_ptr(), int(grad.dtype == torch.float32), master.data_ptr(),
                                exp_avg.data_ptr(), exp_avg_sq.data_ptr(), native.ptr(param_bf16), n,
                                lr, beta1, beta2, eps, weight_decay, step, grad_scale,
                                native.sm_count(master.device), native.stream(master.device))
    native.check(rc, "hpb_adamw")
