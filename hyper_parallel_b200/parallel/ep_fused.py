"""Expert parallelism over symmetric memory: pull-model dispatch / combine kernels around the
grouped tcgen05 expert GEMMs, with no host round trip between routing and the expert output.

The reference has no expert-parallel path (its only related primitive is the generic all-to-all
of ``redistribute``, hyper_parallel/core/tensor_redistribution.py:84-151); the NCCL formulation
of this layer (``ops.moe.expert_parallel_ffn``: count exchange, two ``all_to_all_single`` and
host-side split lists) is kept as the baseline and as the oracle of the tests.

One :class:`EPWorkspace` per (group, shape) owns a symmetric region with the staged tokens, the
sorted pair lists, the per-expert counts and the expert-output matrix that peers pull from.  The
receive matrix of a dispatch is an ordinary tensor sized for ``capacity`` x the balanced load
(it is saved for the backward of the expert GEMMs); unused 128-row blocks are skipped by the
GEMM kernel through a device-side block table, so no size ever returns to the host.  A router so
imbalanced that one rank receives more than ``capacity`` x the balanced load is an ERROR: the
dispatch kernel records status code 6, leaves empty tables (the expert GEMMs then do nothing) and
``native.check_status()`` raises at the end of the step; raise ``capacity`` in that case.  The
DeepSeek-V3 model passes the expert-parallel size (capped at 4) unless told otherwise: with
group-limited routing, correlated tokens all prefer the same few groups and the ranks that host
them receive far more than twice the balanced load -- seen after a handful of steps on random
tokens (2.4 x at EP = 4), which is why 2.0 is only the default of the bare function.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict

import torch

from ..collectives import cc
from ..ops import native
from ..ops.grouped import _grouped
from .symm import DEFAULT_WAIT_NS, SymmetricMemory

_WS: Dict[tuple, "EPWorkspace"] = {}
_bound = False


def _lib():
    global _bound
    lib = native.lib()
    if not _bound:
        vp, ci, cu, cull = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_ulonglong
        pp = ctypes.POINTER(vp)
        lib.hpb_ep_dispatch.argtypes = [pp, pp, pp, pp, pp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cu, cull,
                                        vp, ci, vp]
        lib.hpb_ep_dispatch.restype = ci
        lib.hpb_ep_combine.argtypes = [pp, vp, pp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cu, cull, vp, ci,
                                       vp]
        lib.hpb_ep_combine.restype = ci
        _bound = True
    return lib


def enabled() -> bool:
    return os.environ.get("HPB_FUSED_EP", "1") != "0"


def _al(b: int) -> int:
    return (int(b) + 255) // 256 * 256


class EPWorkspace:
    def __init__(self, group, T: int, k: int, H: int, E: int, capacity: float = 2.0, device=None):
        self.group = group
        self.n = cc.group_size(group)
        self.rank = cc.group_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.T, self.k, self.H, self.E = T, k, H, E
        self.e_local = E // self.n
        self.cap_rows = (int(T * k * capacity) + 127) // 128 * 128 + self.e_local * 128
        self.off_x = 0
        self.off_tok = _al(T * H * 2)
        self.off_scale = self.off_tok + _al(T * k * 4)
        self.off_cnt = self.off_scale + _al(T * k * 4)
        self.off_out = self.off_cnt + _al(E * 4)
        self.symm = SymmetricMemory(group, self.off_out + self.cap_rows * H * 2, self.device)
        s = self.symm
        self.x_stage = s.tensor(torch.bfloat16, T * H, self.off_x).view(T, H)
        self.sorted_token = s.tensor(torch.int32, T * k, self.off_tok)
        self.sorted_scale = s.tensor(torch.float32, T * k, self.off_scale)
        self.counts = s.tensor(torch.int32, E, self.off_cnt)
        self.out = s.tensor(torch.bfloat16, self.cap_rows * H, self.off_out).view(self.cap_rows, H)
        self.p_x, self.p_tok, self.p_scale = s.ptr_table(self.off_x), s.ptr_table(self.off_tok), s.ptr_table(self.off_scale)
        self.p_cnt, self.p_out = s.ptr_table(self.off_cnt), s.ptr_table(self.off_out)
        self.null_table = (ctypes.c_void_p * max(self.n, 1))()
        self.meta = torch.zeros(4, dtype=torch.int32, device=self.device)
        # every rank's counts as seen by the last dispatch on this rank (local: the combine kernel of
        # the same layer reads them from here, not from a peer that may have moved on)
        self.counts_all = torch.zeros(self.n * E, dtype=torch.int32, device=self.device)
        self.status = native.status_word(self.device)
        self.ctas = 2 * native.sm_count(self.device)

    @staticmethod
    def get(group, T, k, H, E, capacity: float = 2.0) -> "EPWorkspace":
        key = (id(group), torch.cuda.current_device(), T, k, H, E, capacity)
        if key not in _WS:
            _WS[key] = EPWorkspace(group, T, k, H, E, capacity)
        return _WS[key]

    def dispatch(self, x, sorted_token, counts, scale=None, limit_ns: int = DEFAULT_WAIT_NS):
        """Stage ``x`` and the pair lists, pull my experts' rows: ``(recv [cap, H], block_group, group_offsets)``."""
        self.x_stage.copy_(x)
        self.sorted_token.copy_(sorted_token)
        self.counts.copy_(counts)
        if scale is not None:
            self.sorted_scale.copy_(scale)
        recv = torch.empty((self.cap_rows, self.H), dtype=torch.bfloat16, device=self.device)
        block_group = torch.empty(self.cap_rows // 128, dtype=torch.int32, device=self.device)
        offsets = torch.empty(self.e_local + 1, dtype=torch.int32, device=self.device)
        rc = _lib().hpb_ep_dispatch(self.p_x, self.p_tok, self.p_scale if scale is not None else self.null_table,
                                    self.p_cnt, self.symm.pad_ptrs, recv.data_ptr(), block_group.data_ptr(),
                                    offsets.data_ptr(), self.meta.data_ptr(), self.counts_all.data_ptr(), self.T,
                                    self.k, self.H, self.E, self.n, self.rank, self.cap_rows, self.symm.next_epoch(), limit_ns,
                                    self.status.data_ptr(), self.ctas, native.stream(self.device))
        native.check(rc, "hpb_ep_dispatch")
        return recv, block_group, offsets

    def combine(self, topk_idx, sorted_pos, weights, save_rows: bool, limit_ns: int = DEFAULT_WAIT_NS):
        """Pull the k expert-output rows of every token out of the owners' ``out`` matrices."""
        y = torch.empty((self.T, self.H), dtype=torch.bfloat16, device=self.device)
        rows = torch.empty((self.T * self.k, self.H), dtype=torch.bfloat16, device=self.device) if save_rows else None
        rc = _lib().hpb_ep_combine(self.p_out, self.counts_all.data_ptr(), self.symm.pad_ptrs, topk_idx.data_ptr(),
                                   sorted_pos.data_ptr(), native.ptr(weights), y.data_ptr(), native.ptr(rows),
                                   self.T, self.k, self.H, self.E, self.n, self.rank, self.cap_rows,
                                   self.symm.next_epoch(), limit_ns, self.status.data_ptr(), self.ctas, native.stream(self.device))
        native.check(rc, "hpb_ep_combine")
        return y, rows


def _swiglu_raw(h: torch.Tensor) -> torch.Tensor:
    rows, f2 = h.shape
    out = torch.empty((rows, f2 // 2), dtype=h.dtype, device=h.device)
    native.check(native.lib().hpb_swiglu_fwd(h.data_ptr(), out.data_ptr(), rows, f2 // 2, native.sm_count(h.device),
                                             native.stream(h.device)), "hpb_swiglu_fwd")
    return out


def _swiglu_bwd_raw(h: torch.Tensor, dact: torch.Tensor) -> torch.Tensor:
    rows, f2 = h.shape
    dh = torch.empty_like(h)
    native.check(native.lib().hpb_swiglu_bwd(h.data_ptr(), dact.data_ptr(), dh.data_ptr(), rows, f2 // 2,
                                             native.sm_count(h.device), native.stream(h.device)), "hpb_swiglu_bwd")
    return dh


class _FusedExperts(torch.autograd.Function):
    """dispatch -> grouped SwiGLU FFN -> combine, forward and backward, on the kernels above."""

    @staticmethod
    def forward(ctx, x, topk_idx, topk_w, w_gate_up, w_down, ws: EPWorkspace, fp8: bool = False):
        T, k = topk_idx.shape
        E, El, H, cap = ws.E, ws.e_local, ws.H, ws.cap_rows
        F2 = w_gate_up.shape[1]
        # expert ids index device-side tables: keep them inside [0, E) whatever the router produced
        topk_idx = topk_idx.clamp(0, E - 1)
        flat_e = topk_idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        sorted_token = (order // k).to(torch.int32)
        counts = torch.bincount(flat_e, minlength=E).to(torch.int32)
        sorted_pos = torch.empty(T * k, dtype=torch.int32, device=x.device)
        sorted_pos[order] = torch.arange(T * k, dtype=torch.int32, device=x.device)
        topk_idx = topk_idx.contiguous()
        recv, block_group, offsets = ws.dispatch(x, sorted_token, counts)
        h = torch.empty((cap, F2), dtype=x.dtype, device=x.device)
        if fp8:
            # forward expert GEMMs on the fp8 tensor cores: 1x128 activation scales, 128x128 weight
            # scales, fp32 promotion per 128-deep block; the backward runs in bf16 on the master weights
            from ..ops import fp8 as f8
            aq, sa = f8.quantize_act_1x128(recv)
            wq, wsc = f8.quantize_weight_128x128(w_gate_up.view(El * F2, H))
            f8.gemm_fp8_grouped(aq, sa, wq, wsc, block_group, El, out=h)
            act = _swiglu_raw(h)
            aq, sa = f8.quantize_act_1x128(act)
            wq, wsc = f8.quantize_weight_128x128(w_down.view(El * H, F2 // 2))
            f8.gemm_fp8_grouped(aq, sa, wq, wsc, block_group, El, out=ws.out)
        else:
            _grouped(recv, False, cap, w_gate_up.view(El * F2, H), False, El * F2, h, cap, F2, H, 1, block_group,
                     None, El, F2)
            act = _swiglu_raw(h)
            _grouped(act, False, cap, w_down.view(El * H, F2 // 2), False, El * H, ws.out, cap, H, F2 // 2, 1,
                     block_group, None, El, H)
        y, rows = ws.combine(topk_idx, sorted_pos, topk_w.float().contiguous(), save_rows=True)
        ctx.save_for_backward(recv, h, block_group, offsets, topk_idx, topk_w, order, sorted_token, counts,
                              sorted_pos, rows, w_gate_up, w_down)
        ctx.ws = ws
        return y

    @staticmethod
    def backward(ctx, dy):
        (recv, h, block_group, offsets, topk_idx, topk_w, order, sorted_token, counts, sorted_pos, rows, w_gate_up,
         w_down) = ctx.saved_tensors
        ws: EPWorkspace = ctx.ws
        T, k = topk_idx.shape
        El, H, cap = ws.e_local, ws.H, ws.cap_rows
        F2 = w_gate_up.shape[1]
        Fh = F2 // 2
        dy = dy.contiguous()
        # gate weights: d w[t, j] = <expert output row (t, j), dy[t]>
        dw_topk = torch.bmm(rows.view(T, k, H), dy.view(T, H, 1)).view(T, k).to(topk_w.dtype)
        # d(expert output) = gate weight x dy, delivered in the expert layout
        scale = topk_w.reshape(-1).float().index_select(0, order)
        d_out, _, _ = ws.dispatch(dy, sorted_token, counts, scale=scale)
        act = _swiglu_raw(h)
        d_act = torch.empty((cap, Fh), dtype=dy.dtype, device=dy.device)
        _grouped(d_out, False, cap, w_down.view(El * H, Fh), True, El * H, d_act, cap, Fh, H, 1, block_group, None,
                 El, H)
        dw_down = torch.empty_like(w_down)
        _grouped(d_out, True, cap, act, True, cap, dw_down.view(El * H, Fh), H, Fh, 0, 2, None, offsets, El, 0)
        del act
        d_h = _swiglu_bwd_raw(h, d_act)
        del d_act
        _grouped(d_h, False, cap, w_gate_up.view(El * F2, H), True, El * F2, ws.out, cap, H, F2, 1, block_group, None,
                 El, F2)
        dw_gate_up = torch.empty_like(w_gate_up)
        _grouped(d_h, True, cap, recv, True, cap, dw_gate_up.view(El * F2, H), F2, H, 0, 2, None, offsets, El, 0)
        dx, _ = ws.combine(topk_idx, sorted_pos, None, save_rows=False)
        return dx, None, dw_topk, dw_gate_up, dw_down, None, None


def fused_expert_parallel_ffn(x, topk_idx, topk_w, w_gate_up, w_down, num_experts: int, ep_group,
                              capacity: float = 2.0, fp8: bool = False):
    """``y[t] = sum_k topk_w[t,k] * expert_{topk_idx[t,k]}(x[t])`` with experts sharded over ``ep_group``.
    ``fp8``: the two forward expert GEMMs run block-scaled in e4m3 (hidden and expert width must be
    multiples of 128; otherwise bf16 is used)."""
    T, k = topk_idx.shape
    ws = EPWorkspace.get(ep_group, T, k, x.shape[-1], num_experts, capacity)
    fp8 = bool(fp8) and x.shape[-1] % 128 == 0 and w_down.shape[-1] % 128 == 0
    return _FusedExperts.apply(x.contiguous(), topk_idx, topk_w, w_gate_up.contiguous(), w_down.contiguous(), ws,
                               fp8)


def usable(x, topk_idx, w_gate_up, num_experts: int, ep_group) -> bool:
    if not (enabled() and x.is_cuda and x.dtype == torch.bfloat16 and native.available()):
        return False
    n = cc.group_size(ep_group)
    if n > 8 or topk_idx.shape[1] > 8 or num_experts > 512 or num_experts % n or num_experts // n > 64:
        return False
    if x.shape[-1] % 8 or (n > 1 and cc.get_backend(ep_group) != "nccl"):
        return False
    return True
