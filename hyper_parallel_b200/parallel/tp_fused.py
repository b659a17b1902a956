"""Workspace and launchers of the fused tensor-parallel kernels (all-gather->GEMM, GEMM->reduce-scatter).

A :class:`TPWorkspace` owns, per tensor-parallel group, one symmetric-memory region with two
activation-shard buffers (alternated call by call) and two receive areas for the reduce-scatter,
plus the local staging matrix and counters the kernels need.  Alternating buffers is what makes a
"done reading" handshake unnecessary (see gemm_comm_sm100.cu).
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional

import torch

from ..collectives import cc
from ..ops import native
from .symm import DEFAULT_WAIT_NS, SymmetricMemory

_WORKSPACES: Dict[tuple, "TPWorkspace"] = {}
_bound = False


def _lib():
    global _bound
    lib = native.lib()
    if not _bound:
        vp, ci, cu, cull, cll = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_ulonglong, ctypes.c_longlong
        pp = ctypes.POINTER(vp)
        lib.hpb_ag_gemm.argtypes = [pp, pp, vp, vp, vp, vp, cll, ci, ci, ci, ci, ci, cu, cull, vp, ci, vp]
        lib.hpb_ag_gemm.restype = ci
        lib.hpb_gemm_rs.argtypes = [vp, vp, pp, pp, vp, vp, ci, ci, ci, ci, ci, cu, cull, vp, ci, vp]
        lib.hpb_gemm_rs.restype = ci
        lib.hpb_p2p_allgather.argtypes = [pp, pp, vp, ci, vp, ci, ci, cu, cull, vp, vp, ci, vp]
        lib.hpb_p2p_allgather.restype = ci
        _bound = True
    return lib


class TPWorkspace:
    def __init__(self, group, shard_bytes: int, recv_bytes: int, device=None):
        self.group = group
        self.n = cc.group_size(group)
        self.rank = cc.group_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        al = lambda b: (int(b) + 255) // 256 * 256  # noqa: E731
        self.shard_bytes, self.recv_bytes = al(shard_bytes), al(recv_bytes)
        self.symm = SymmetricMemory(group, 2 * self.shard_bytes + 2 * self.recv_bytes, self.device)
        self.staging = torch.empty(self.n * self.shard_bytes // 2, dtype=torch.bfloat16, device=self.device)
        self.counters = torch.zeros(32, dtype=torch.int32, device=self.device)
        self.status = native.status_word(self.device)
        self.ag_calls = 0
        self.rs_calls = 0

    @staticmethod
    def get(group, shard_bytes: int, recv_bytes: int) -> "TPWorkspace":
        key = (id(group), torch.cuda.current_device())
        ws = _WORKSPACES.get(key)
        if ws is None or ws.shard_bytes < shard_bytes or ws.recv_bytes < recv_bytes:
            ws = TPWorkspace(group, max(shard_bytes, ws.shard_bytes if ws else 0),
                             max(recv_bytes, ws.recv_bytes if ws else 0))
            _WORKSPACES[key] = ws
        return ws

    # -------------------------------------------------------------------------------
    def ag_gemm(self, x_shard: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None,
                limit_ns: int = DEFAULT_WAIT_NS) -> torch.Tensor:
        """``concat_r(x_r)[n*Ms, K] @ w[N, K].T`` with the gather fused into the GEMM kernel."""
        Ms, K = x_shard.shape
        N = w.shape[0]
        nbytes = Ms * K * 2
        assert nbytes <= self.shard_bytes and x_shard.dtype == torch.bfloat16 and w.is_contiguous()
        off = (self.ag_calls & 1) * self.shard_bytes
        self.ag_calls += 1
        slot = self.symm.tensor(torch.bfloat16, Ms * K, off).view(Ms, K)
        slot.copy_(x_shard)                                   # my shard into this call's symmetric buffer
        if out is None:
            out = torch.empty((self.n * Ms, N), dtype=torch.bfloat16, device=self.device)
        cnt = self.counters[:8]
        cnt.zero_()
        rc = _lib().hpb_ag_gemm(self.symm.ptr_table(off), self.symm.pad_ptrs, self.staging.data_ptr(),
                                cnt.data_ptr(), w.data_ptr(), out.data_ptr(), out.stride(0), Ms, N, K, self.n,
                                self.rank, self.symm.next_epoch(), limit_ns, self.status.data_ptr(),
                                native.sm_count(self.device), native.stream(self.device))
        native.check(rc, "hpb_ag_gemm")
        return out

    def gathered(self, rows: int, cols: int) -> torch.Tensor:
        """The ``[rows, cols]`` matrix that the last :meth:`ag_gemm` / :meth:`gather` call assembled in
        the local staging buffer (valid until the next such call on this workspace)."""
        return self.staging[:rows * cols].view(rows, cols)

    def gather(self, x_shard: torch.Tensor, limit_ns: int = DEFAULT_WAIT_NS) -> torch.Tensor:
        """``concat_r(x_r)`` by peer pulls over NVLink (no product attached): the operand of a
        weight-gradient GEMM whose contraction runs over the gathered rows."""
        Ms, K = x_shard.shape
        assert Ms * K * 2 <= self.shard_bytes and x_shard.dtype == torch.bfloat16 and (Ms * K) % 8 == 0
        off = (self.ag_calls & 1) * self.shard_bytes
        self.ag_calls += 1
        self.symm.tensor(torch.bfloat16, Ms * K, off).view(Ms, K).copy_(x_shard)
        seg = torch.tensor([[0, 0, Ms * K, 0]], dtype=torch.int64, device=self.device)
        rc = _lib().hpb_p2p_allgather(self.symm.ptr_table(off), self.symm.pad_ptrs, seg.data_ptr(), 1,
                                      self.staging.data_ptr(), self.rank, self.n, self.symm.next_epoch(), limit_ns,
                                      self.status.data_ptr(), self.symm.done_counter.data_ptr(), 96,
                                      native.stream(self.device))
        native.check(rc, "hpb_p2p_allgather")
        return self.gathered(self.n * Ms, K)

    def gemm_rs(self, a: torch.Tensor, w: torch.Tensor, limit_ns: int = DEFAULT_WAIT_NS) -> torch.Tensor:
        """``reduce_scatter_rows(a[n*Ms, K] @ w[N, K].T)`` with the scatter fused into the GEMM epilogue."""
        M, K = a.shape
        N = w.shape[0]
        Ms = M // self.n
        assert M % self.n == 0 and self.n * Ms * N * 2 <= self.recv_bytes and a.is_contiguous() and w.is_contiguous()
        off = 2 * self.shard_bytes + (self.rs_calls & 1) * self.recv_bytes
        self.rs_calls += 1
        out = torch.empty((Ms, N), dtype=torch.bfloat16, device=self.device)
        cnt = self.counters[8:16]
        cnt.zero_()
        rc = _lib().hpb_gemm_rs(a.data_ptr(), w.data_ptr(), self.symm.ptr_table(off), self.symm.pad_ptrs,
                                cnt.data_ptr(), out.data_ptr(), Ms, N, K, self.n, self.rank, self.symm.next_epoch(),
                                limit_ns, self.status.data_ptr(), native.sm_count(self.device),
                                native.stream(self.device))
        native.check(rc, "hpb_gemm_rs")
        return out
