"""Block-scaled FP8 (e4m3) linear algebra: quantisers and the tcgen05 fp8 GEMM.

Scaling follows the DeepSeek-V3 recipe named by the benchmark configuration: activations carry
one fp32 scale per 1x128 tile, weights one per 128x128 tile; products are accumulated in fp32
and promoted block by block (see gemm_fp8_sm100.cu).  The reference has no FP8 path.

``fp8_linear(x, w)`` runs the forward GEMM in fp8 and both backward GEMMs in bf16 on the
master weights (straight-through for the quantisation).
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import functional as Fn
from . import native

_bound = False
E4M3_MAX = 448.0


def _lib():
    global _bound
    lib = native.lib()
    if not _bound:
        vp, ci, cll = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.hpb_gemm_fp8_blockscale.argtypes = [vp, vp, vp, vp, vp, cll, ci, ci, ci, vp, ci, vp]
        lib.hpb_gemm_fp8_blockscale.restype = ci
        lib.hpb_gemm_fp8_blockscale_grouped.argtypes = [vp, vp, vp, vp, vp, cll, ci, ci, ci, ci, vp, vp, ci, vp]
        lib.hpb_gemm_fp8_blockscale_grouped.restype = ci
        lib.hpb_quant_act_1x128.argtypes = [vp, vp, vp, ci, ci, vp]
        lib.hpb_quant_act_1x128.restype = ci
        lib.hpb_quant_weight_128x128.argtypes = [vp, vp, vp, ci, ci, vp]
        lib.hpb_quant_weight_128x128.restype = ci
        _bound = True
    return lib


def quantize_act_1x128(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``x[M, K]`` bf16 -> (e4m3 ``[M, K]``, scales ``[K/128, M]`` fp32)."""
    M, K = x.shape
    assert K % 128 == 0
    if not x.is_cuda:
        xb = x.float().view(M, K // 128, 128)
        scale = xb.abs().amax(-1).clamp_min(1e-10) / E4M3_MAX
        q = (xb / scale[..., None]).to(torch.float8_e4m3fn).view(M, K)
        return q, scale.t().contiguous()
    x = x.contiguous()
    q = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=x.device)
    s = torch.empty((K // 128, M), dtype=torch.float32, device=x.device)
    native.check(_lib().hpb_quant_act_1x128(x.data_ptr(), q.data_ptr(), s.data_ptr(), M, K, native.stream(x.device)),
                 "hpb_quant_act_1x128")
    return q, s


def quantize_weight_128x128(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``w[N, K]`` bf16 -> (e4m3 ``[N, K]``, scales ``[ceil(N/128), K/128]`` fp32)."""
    N, K = w.shape
    assert K % 128 == 0
    nb = (N + 127) // 128
    if not w.is_cuda:
        pad = nb * 128 - N
        wp = torch.nn.functional.pad(w.float(), (0, 0, 0, pad)).view(nb, 128, K // 128, 128)
        scale = wp.abs().amax(dim=(1, 3)).clamp_min(1e-10) / E4M3_MAX
        q = (wp / scale[:, None, :, None]).to(torch.float8_e4m3fn).view(nb * 128, K)[:N]
        return q.contiguous(), scale
    w = w.contiguous()
    q = torch.empty((N, K), dtype=torch.float8_e4m3fn, device=w.device)
    s = torch.empty((nb, K // 128), dtype=torch.float32, device=w.device)
    native.check(_lib().hpb_quant_weight_128x128(w.data_ptr(), q.data_ptr(), s.data_ptr(), N, K,
                                                 native.stream(w.device)), "hpb_quant_weight_128x128")
    return q, s


def dequantize(q, scale_act=None, scale_w=None) -> torch.Tensor:
    """fp32 reconstruction (oracle for the tests)."""
    f = q.float()
    if scale_act is not None:
        M, K = f.shape
        return (f.view(M, K // 128, 128) * scale_act.t()[..., None]).view(M, K)
    N, K = f.shape
    nb = scale_w.shape[0]
    pad = nb * 128 - N
    fp = torch.nn.functional.pad(f, (0, 0, 0, pad)).view(nb, 128, K // 128, 128)
    return (fp * scale_w[:, None, :, None]).view(nb * 128, K)[:N]


def gemm_fp8(aq, sa, bq, sb) -> torch.Tensor:
    """``C[M, N] = dequant(aq, sa) @ dequant(bq, sb).T`` in bf16, computed on the fp8 tensor cores."""
    M, K = aq.shape
    N = bq.shape[0]
    if not aq.is_cuda:
        return (dequantize(aq, scale_act=sa) @ dequantize(bq, scale_w=sb).t()).to(torch.bfloat16)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=aq.device)
    dev = aq.device
    rc = _lib().hpb_gemm_fp8_blockscale(aq.data_ptr(), sa.data_ptr(), bq.data_ptr(), sb.data_ptr(), out.data_ptr(),
                                        out.stride(0), M, N, K, native.status_word(dev).data_ptr(),
                                        native.sm_count(dev), native.stream(dev))
    native.check(rc, "hpb_gemm_fp8_blockscale")
    return out


def gemm_fp8_grouped(aq, sa, bq, sb, block_group, num_experts: int, out=None) -> torch.Tensor:
    """Grouped (expert) fp8 GEMM: rows of ``aq[M, K]`` are grouped by expert in 128-row blocks
    (``block_group[M/128]``, ``-1`` = unused block, left untouched in the output); ``bq[E*N, K]``
    stacks the experts' weights, ``sb[E*N/128, K/128]`` their scale tiles.  Returns ``[M, N]`` bf16."""
    M, K = aq.shape
    N = bq.shape[0] // num_experts
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=aq.device)
    if not aq.is_cuda:
        a = dequantize(aq, scale_act=sa)
        b = dequantize(bq, scale_w=sb).view(num_experts, N, K)
        for blk, e in enumerate(block_group.tolist()):
            if e >= 0:
                out[blk * 128:(blk + 1) * 128] = (a[blk * 128:(blk + 1) * 128] @ b[e].t()).to(torch.bfloat16)
        return out
    dev = aq.device
    rc = _lib().hpb_gemm_fp8_blockscale_grouped(aq.data_ptr(), sa.data_ptr(), bq.data_ptr(), sb.data_ptr(),
                                                out.data_ptr(), out.stride(0), M, N, K, num_experts,
                                                block_group.data_ptr(), native.status_word(dev).data_ptr(),
                                                native.sm_count(dev), native.stream(dev))
    native.check(rc, "hpb_gemm_fp8_blockscale_grouped")
    return out


class _Fp8Linear(torch.autograd.Function):
    """2-D in, 2-D out: nothing it returns is a view created inside the Function, so callers may
    modify (part of) the result in place."""

    @staticmethod
    def forward(ctx, x2, w):
        ctx.save_for_backward(x2, w)
        aq, sa = quantize_act_1x128(x2)
        bq, sb = quantize_weight_128x128(w)
        return gemm_fp8(aq, sa, bq, sb)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.contiguous()
        dx = Fn.gemm(dy2, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = Fn.gemm(dy2, x2, a_mn=True, b_mn=True) if ctx.needs_input_grad[1] else None
        return dx, dw


def fp8_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` with an fp8 block-scaled forward GEMM (K must be a multiple of 128)."""
    if x.shape[-1] % 128:
        return Fn.linear(x, w)
    y = _Fp8Linear.apply(x.reshape(-1, x.shape[-1]), w)
    return y if x.dim() == 2 else y.view(*x.shape[:-1], w.shape[0])
