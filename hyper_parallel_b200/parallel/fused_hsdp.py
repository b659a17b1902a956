"""HSDP over symmetric memory: P2P all-gather into place and fused reduce-scatter + AdamW.

This is the B200-native replacement of the two hot collectives of an HSDP step (the reference
issues them as separate NCCL calls followed by cast / scale / optimizer kernels,
hyper_parallel/core/hsdp/hsdp_param_buffer.py:74-97, hsdp_grad_buffer.py:95-135):

* the bf16 parameter shards of one wrapped module live in ONE flat buffer inside a
  :class:`SymmetricMemory` region; unsharding is a single kernel in which every rank pulls all
  peers' shard segments over NVLink straight into the per-parameter full tensors (no gather
  buffer, no copy-out);
* weight gradients are written by the wgrad GEMM epilogue directly into a flat gradient buffer
  in symmetric memory; when the module's backward is done ONE kernel reads this rank's slice of
  every peer's gradient buffer, sums in fp32, scales, and applies AdamW to the fp32 master /
  moments and the bf16 shard -- reduce-scatter, cast, scale and optimizer in a single pass over
  the data, overlapped with the backward of the next module on a side stream.

Synchronisation between ranks is inside the kernels (signal pads, bounded waits); between the
compute stream and the communication stream it is CUDA events.  The path is used when the group
is a full-shard group of CUDA ranks on one node and the parameters are bf16; anything else falls
back to the ``torch.distributed`` buffers.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional

import torch

from ..collectives import cc
from ..ops import native
from .symm import DEFAULT_WAIT_NS, SymmetricMemory

_COMM_STREAMS: Dict[int, torch.cuda.Stream] = {}
# CTAs of the communication kernels.  Both are bandwidth kernels (the fused reduce-scatter + AdamW
# moves 26 B of optimizer state per parameter through HBM on top of the NVLink reads), so they
# need most of the machine's memory-level parallelism; they co-reside with the GEMM CTAs.
_NUM_COMM_CTAS = int(os.environ.get("HPB_COMM_CTAS", "96"))
_NUM_RS_CTAS = int(os.environ.get("HPB_RS_CTAS", os.environ.get("HPB_COMM_CTAS", "148")))


def comm_stream(device: torch.device) -> torch.cuda.Stream:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _COMM_STREAMS:
        _COMM_STREAMS[idx] = torch.cuda.Stream(device=idx, priority=-1)
    return _COMM_STREAMS[idx]


def symm_path_enabled() -> bool:
    return os.environ.get("HPB_FUSED_COMM", "1") != "0"


def can_use(params) -> bool:
    """All parameters: CUDA, bf16, plain tensors, fully sharded over one group of this node."""
    if not symm_path_enabled() or not params or not torch.cuda.is_available():
        return False
    if not cc.is_initialized() or cc.get_backend() != "nccl":
        return False
    p0 = params[0]
    if p0.dp_size != 1 or p0.shard_size > 16 or p0.shard_size > torch.cuda.device_count():
        return False
    for p in params:
        if p.is_dtensor or p.shard.dtype != torch.bfloat16 or not p.shard.is_cuda:
            return False
        if p.shard.numel() % 8:
            return False
    return True


def _bind(lib):
    vp, ci, cu, cull = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_ulonglong
    pp = ctypes.POINTER(vp)
    lib.hpb_p2p_allgather.argtypes = [pp, pp, vp, ci, vp, ci, ci, cu, cull, vp, vp, ci, vp]
    lib.hpb_p2p_allgather.restype = ci
    cf = ctypes.c_float
    lib.hpb_fused_rs_adamw.argtypes = [pp, pp, vp, ci, vp, vp, vp, vp, cf, cf, cf, cf, cf, ci, cf, ci, ci, cu,
                                       cull, vp, vp, ci, vp]
    lib.hpb_fused_rs_adamw.restype = ci
    return lib


class SymmParamBuffer:
    """Flat shard + flat gradient buffers of one HSDP state in symmetric memory."""

    def __init__(self, params, level3: bool):
        self.params = params
        p0 = params[0]
        self.group = p0.sharded_group_info.group
        self.n = p0.shard_size
        self.rank = p0.sharded_group_info.index
        self.device = p0.shard.device
        self.lib = _bind(native.lib())
        numels = [p.shard.numel() for p in params]
        self.shard_off, self.full_off = [], []
        so = fo = 0
        for k in numels:
            self.shard_off.append(so)
            self.full_off.append(fo)
            so += k
            fo += k * self.n
        self.shard_numel, self.full_numel = so, fo
        # symmetric region: [flat shard | flat full gradients]
        self.grad_byte_off = (so * 2 + 255) // 256 * 256
        self.symm = SymmetricMemory(self.group, self.grad_byte_off + fo * 2, self.device)
        self.flat_shard = self.symm.tensor(torch.bfloat16, so, 0)
        self.flat_grad = self.symm.tensor(torch.bfloat16, fo, self.grad_byte_off)
        self.shard_ptrs = self.symm.ptr_table(0)
        self.grad_ptrs = self.symm.ptr_table(self.grad_byte_off)
        segs = torch.tensor([[f, s, k] for f, s, k in zip(self.full_off, self.shard_off, numels)],
                            dtype=torch.int64, device=self.device)
        self.segs = segs.contiguous()
        self.full = torch.empty(fo, dtype=torch.bfloat16, device=self.device)
        for p, s, k in zip(params, self.shard_off, numels):
            view = self.flat_shard[s:s + k].view(p.shard_shape)
            view.copy_(p.shard)
            p.rebind_shard(view)
        self.full_views = [self.full[f:f + k * self.n].view(p.full_shape)
                           for p, f, k in zip(params, self.full_off, numels)]
        self.grad_views = [self.flat_grad[f:f + k * self.n].view(p.full_shape)
                           for p, f, k in zip(params, self.full_off, numels)]
        self.status = native.status_word(self.device)
        self.gather_event: Optional[torch.cuda.Event] = None
        self.reduce_event: Optional[torch.cuda.Event] = None
        self.free_event: Optional[torch.cuda.Event] = None     # compute finished with `full`
        self.grad_fresh = True        # nothing accumulated in flat_grad yet in this window
        self.ready = set()
        self.optimizer = None         # set by FusedAdamW.fuse_into_backward
        self.opt_state = None
        self.handle = None
        for i, p in enumerate(params):
            p._symm = (self, i)

    # ------------------------------------------------------------- all-gather --
    def prefetch(self) -> None:
        if self.gather_event is not None or not self.params[0].is_sharded_now:
            return
        cs = comm_stream(self.device)
        cur = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(cur)
        cs.wait_event(ev)                       # everything that read `full` before is finished
        with torch.cuda.stream(cs):
            ep = self.symm.next_epoch()
            rc = self.lib.hpb_p2p_allgather(self.shard_ptrs, self.symm.pad_ptrs, self.segs.data_ptr(),
                                            len(self.params), self.full.data_ptr(), self.rank, self.n, ep,
                                            DEFAULT_WAIT_NS, self.status.data_ptr(),
                                            self.symm.done_counter.data_ptr(), _NUM_COMM_CTAS, cs.cuda_stream)
            native.check(rc, "hpb_p2p_allgather")
            self.gather_event = torch.cuda.Event()
            self.gather_event.record(cs)

    def unshard(self) -> None:
        if not self.params[0].is_sharded_now:
            return
        if self.gather_event is None:
            self.prefetch()
        torch.cuda.current_stream(self.device).wait_event(self.gather_event)
        self.gather_event = None
        for p, v in zip(self.params, self.full_views):
            p.leaf.data = v
            p.is_sharded_now = False

    def reshard(self) -> None:
        for p in self.params:
            p.to_sharded()

    # ------------------------------------------------------------------ grads --
    def wgrad_target(self, i: int):
        """(buffer view, accumulate?) for the weight-gradient GEMM of parameter ``i``."""
        if self.reduce_event is not None:
            # the previous reduction must have finished reading the buffer (on every rank)
            torch.cuda.current_stream(self.device).wait_event(self.reduce_event)
            self.reduce_event = None
        return self.grad_views[i], (not self.grad_fresh) or (i in self.ready)

    def mark_ready(self, i: int) -> bool:
        self.ready.add(i)
        return len(self.ready) == sum(1 for p in self.params if p.param.requires_grad)

    def store_grad(self, i: int, grad: torch.Tensor) -> bool:
        """Copy (or accumulate) an autograd-produced gradient into the flat buffer."""
        view, acc = self.wgrad_target(i)
        if acc:
            view.add_(grad.view_as(view))
        else:
            view.copy_(grad.view_as(view))
        return self.mark_ready(i)

    def reduce_and_step(self, sync: bool, grad_scale: float) -> bool:
        """All gradients of this state are in ``flat_grad``.  On a sync step launch the fused
        reduce-scatter + AdamW; returns True when the optimizer consumed the gradients."""
        self.ready = set()
        if not sync:
            self.grad_fresh = False
            return True
        opt = self.optimizer
        if opt is None:
            return False
        st = opt.flat_state_for(self)
        g = opt.group_for(self)
        cs = comm_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        cs.wait_event(ev)
        with torch.cuda.stream(cs):
            ep = self.symm.next_epoch()
            rc = self.lib.hpb_fused_rs_adamw(
                self.grad_ptrs, self.symm.pad_ptrs, self.segs.data_ptr(), len(self.params),
                st["master"].data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(),
                self.flat_shard.data_ptr(), g["lr"], g["betas"][0], g["betas"][1], g["eps"], g["weight_decay"],
                opt._step_count + 1, grad_scale, self.rank, self.n, ep, DEFAULT_WAIT_NS, self.status.data_ptr(),
                self.symm.done_counter.data_ptr() + 8, _NUM_RS_CTAS, cs.cuda_stream)
            native.check(rc, "hpb_fused_rs_adamw")
            self.reduce_event = torch.cuda.Event()
            self.reduce_event.record(cs)
        self.grad_fresh = True
        return True

    def wait(self) -> None:
        if self.reduce_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self.reduce_event)
            self.reduce_event = None
