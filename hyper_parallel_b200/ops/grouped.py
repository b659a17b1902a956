"""Grouped (per-expert) linear layers on the tcgen05 GEMM kernel.

``grouped_linear(x, w[E, N, K], counts)``: rows of ``x`` are grouped by expert (``counts[e]`` rows
for expert ``e``); returns ``y`` with ``y_e = x_e @ w[e].T`` in the same row order.

The kernel works on a *padded* layout in which every expert's rows start at a multiple of 128
(the M tile) so that no output tile straddles two experts: rows are scattered into that layout
(padding rows are zero), the three GEMMs of forward / dgrad / wgrad run as single grouped
launches, and the result is gathered back.  Padding costs at most 127 rows per expert.
"""
from __future__ import annotations

import ctypes
from typing import List, Sequence, Tuple

import torch

from . import native

_BLOCK_M = 128
_bound = False


def _lib():
    global _bound
    lib = native.lib()
    if not _bound:
        vp, ci, c64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
        lib.hpb_gemm_bf16_grouped.argtypes = [vp, ci, c64, c64, vp, ci, c64, c64, vp, c64, ci, ci, ci, ci, ci, ci,
                                              vp, vp, ci, ci, vp, ci, vp]
        lib.hpb_gemm_bf16_grouped.restype = ci
        _bound = True
    return lib


def padded_layout(counts: Sequence[int], device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, int]:
    """``(row map [sum counts] -> padded row, block_group [blocks], group_offsets [E+1], padded rows)``."""
    offs = [0]
    blocks: List[int] = []
    rows: List[torch.Tensor] = []
    for e, c in enumerate(counts):
        pad = (c + _BLOCK_M - 1) // _BLOCK_M * _BLOCK_M
        rows.append(torch.arange(offs[-1], offs[-1] + c))
        blocks += [e] * (pad // _BLOCK_M)
        offs.append(offs[-1] + pad)
    row_map = torch.cat(rows).to(device) if rows else torch.zeros(0, dtype=torch.long, device=device)
    return (row_map, torch.tensor(blocks, dtype=torch.int32, device=device),
            torch.tensor(offs, dtype=torch.int32, device=device), offs[-1])


def _grouped(a, a_mn, a_rows, b, b_mn, b_rows, out, M, N, K, mode, block_group, group_offsets, E, b_group_rows,
             accumulate=False):
    dev = a.device
    rc = _lib().hpb_gemm_bf16_grouped(
        a.data_ptr(), int(a_mn), a.stride(0), a_rows, b.data_ptr(), int(b_mn), b.stride(0), b_rows,
        out.data_ptr(), out.stride(-2), int(out.dtype == torch.float32), int(accumulate), M, N, K, mode,
        native.ptr(block_group), native.ptr(group_offsets), E, b_group_rows,
        native.status_word(dev).data_ptr(), native.sm_count(dev), native.stream(dev))
    native.check(rc, "hpb_gemm_bf16_grouped")
    return out


class _GroupedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, counts):
        E, N, K = w.shape
        row_map, block_group, offsets, Mp = padded_layout(counts, x.device)
        xp = torch.zeros((Mp, K), dtype=x.dtype, device=x.device)
        xp.index_copy_(0, row_map, x)
        yp = torch.empty((Mp, N), dtype=x.dtype, device=x.device)
        if Mp > 0:
            _grouped(xp, False, Mp, w.view(E * N, K), False, E * N, yp, Mp, N, K, 1, block_group, None, E, N)
        ctx.save_for_backward(xp, w, row_map, block_group, offsets)
        ctx.dims = (E, N, K, Mp)
        return yp.index_select(0, row_map)

    @staticmethod
    def backward(ctx, dy):
        xp, w, row_map, block_group, offsets = ctx.saved_tensors
        E, N, K, Mp = ctx.dims
        dyp = torch.zeros((Mp, N), dtype=dy.dtype, device=dy.device)
        dyp.index_copy_(0, row_map, dy.contiguous())
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dxp = torch.empty((Mp, K), dtype=dy.dtype, device=dy.device)
            if Mp > 0:
                # dx = dy @ W_e : B = W stacked [E*N, K], MN-major with the contraction along its rows
                _grouped(dyp, False, Mp, w.view(E * N, K), True, E * N, dxp, Mp, K, N, 1, block_group, None, E, N)
            dx = dxp.index_select(0, row_map)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(w)
            # dW_e[N, K] = dy_e^T x_e : contraction over the expert's (padded, zero-filled) rows
            _grouped(dyp, True, Mp, xp, True, Mp, dw.view(E * N, K), N, K, 0, 2, None, offsets, E, 0)
        return dx, dw, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts: Sequence[int]) -> torch.Tensor:
    """``y_e = x_e @ w[e].T`` for rows grouped by expert; bf16 CUDA tensors."""
    assert x.dim() == 2 and w.dim() == 3 and x.shape[1] == w.shape[2]
    assert sum(counts) == x.shape[0] and len(counts) == w.shape[0]
    return _GroupedLinear.apply(x.contiguous(), w.contiguous(), list(int(c) for c in counts))
