"""HSDP over symmetric memory: weight all-gather fused into the consumer GEMM, fused
reduce-scatter + AdamW.

This is the B200-native replacement of the two hot collectives of an HSDP step (the reference
issues them as separate NCCL calls followed by cast / scale / optimizer kernels,
hyper_parallel/platform/torch/hsdp/param.py:43-53, hyper_parallel/core/hsdp/hsdp_param_buffer.py:74-97,
hsdp_grad_buffer.py:95-135):

* the bf16 parameter shards of one wrapped module live in ONE flat buffer inside a
  :class:`SymmetricMemory` region.  Unsharding a matrix that is only consumed by ``ops.linear``
  costs no kernel of its own: the parameter receives a *ticket*, and the first GEMM that consumes
  it (the forward product, or the input-gradient product of the level-3 backward) runs the
  all-gather inside the GEMM kernel -- communication warps pull the peers' row panels over NVLink
  into a staging matrix while the tensor cores already multiply the panels that have arrived.
  The staging matrix comes from a small pool and goes back at reshard, so a gathered weight never
  outlives its consumers (the semantics of the reference's only native component, the graph pass
  platform/mindspore/custom_pass/passes/duplicate_on_multi_users/duplicate_on_multi_users.cc:287-353).
  Everything else of the module (norm weights, embedding tables, matrices whose shape the fused
  kernel does not take) is gathered by one peer-pull copy kernel on a side stream;
* weight gradients are written by the wgrad GEMM epilogue directly into a flat gradient buffer
  in symmetric memory; when the module's backward is done ONE kernel reads this rank's slice of
  every peer's gradient buffer -- through one ``multimem.ld_reduce`` per vector where the NVSwitch
  supports multicast, else with N peer loads --, scales, and applies AdamW to the fp32 master /
  moments and the bf16 shard: reduce-scatter, cast, scale and optimizer in a single pass over
  the data, overlapped with the backward of the next module on a side stream.

Synchronisation between ranks is inside the kernels (signal pads, bounded waits).  A rank publishes
a *shard version* whenever its parameter shards have been rewritten (by the fused optimizer kernel,
or after any optimizer step); the fused gather waits for the peers' version of the current step,
which has normally been published long before.  A shard is only rewritten after every peer's
gradients of that module have arrived, i.e. after every peer has finished reading it.

The path is used when the group is a full-shard group of CUDA ranks on one node and the parameters
are bf16 -- plain parameters, or the local shards of tensor-parallel DTensor parameters (TP x HSDP:
the HSDP group of such a parameter is the set of ranks that hold the same tensor-parallel slice);
parameters of other kinds in the same module go through the ``torch.distributed`` buffers.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..collectives import cc
from ..ops import native
from ..utils import tracing
from .symm import DEFAULT_WAIT_NS, SLOT_SHARD_VERSION, SymmetricMemory

_COMM_STREAMS: Dict[int, torch.cuda.Stream] = {}
# CTAs of the communication kernels.  Both are bandwidth kernels (the fused reduce-scatter + AdamW
# moves 26 B of optimizer state per parameter through HBM on top of the NVLink reads), so they
# need most of the machine's memory-level parallelism; they co-reside with the GEMM CTAs.
_NUM_COMM_CTAS = int(os.environ.get("HPB_COMM_CTAS", "96"))
_NUM_RS_CTAS = int(os.environ.get("HPB_RS_CTAS", os.environ.get("HPB_COMM_CTAS", "148")))
_MAX_GROUPS = 4            # optimizer parameter groups per flat buffer (kernel table size)
_LIVE: "weakref.WeakSet[SymmParamBuffer]" = weakref.WeakSet()
_STEP_HOOK = None


def comm_stream(device: torch.device) -> torch.cuda.Stream:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _COMM_STREAMS:
        _COMM_STREAMS[idx] = torch.cuda.Stream(device=idx, priority=-1)
    return _COMM_STREAMS[idx]


def symm_path_enabled() -> bool:
    return os.environ.get("HPB_FUSED_COMM", "1") != "0"


def fused_gather_enabled() -> bool:
    """``HPB_FUSED_AG=1`` gathers GEMM-only weights inside the GEMMs (own gather in the consumer,
    riding gathers on the GEMMs before it).  Default off: end to end the stand-alone peer-pull copy
    kernel on its side stream was faster on the Llama-3-8B step (2 GPUs: 402.8 against 414.9 ms,
    4 GPUs: 424.7 against 437.6 ms) -- the copy hides completely behind the compute of the layer
    before, while a GEMM that carries a gather gives four warps per CTA and part of its L2 / HBM
    bandwidth to it.  Kernel against kernel the fused GEMM beats NCCL all-gather + GEMM."""
    return os.environ.get("HPB_FUSED_AG", "0") != "0"


def group_ok(params) -> bool:
    """The group as a whole can use symmetric memory (which parameters join is decided per parameter)."""
    if not symm_path_enabled() or not params or not torch.cuda.is_available():
        return False
    if not cc.is_initialized() or cc.get_backend() != "nccl":
        return False
    p0 = params[0]
    return p0.dp_size == 1 and 1 < p0.shard_size <= 16 and p0.shard_size <= torch.cuda.device_count()


def eligible(p) -> bool:
    """One parameter: a CUDA bf16 tensor (a plain parameter, or the local shard of a tensor-parallel
    DTensor parameter: HSDP shards dim 0 of the local tensor over the ranks that replicate it) whose
    HSDP shard is a whole number of 16-byte vectors.  ``HPB_SYMM_DTENSOR=0`` keeps DTensor parameters
    on the NCCL buffers."""
    if p.is_dtensor and os.environ.get("HPB_SYMM_DTENSOR", "1") == "0":
        return False
    return p.shard.dtype == torch.bfloat16 and p.shard.is_cuda and p.shard.numel() % 8 == 0


def split_eligible(params):
    """``(symmetric-memory parameters, the rest)`` of one (group, dtype, device) parameter list."""
    if not group_ok(params):
        return [], list(params)
    yes = [p for p in params if eligible(p)]
    no = [p for p in params if not eligible(p)]
    return yes, no


def can_use(params) -> bool:
    """Every parameter of the list can live in one symmetric buffer."""
    yes, no = split_eligible(params)
    return bool(yes) and not no


def _bind(lib):
    if getattr(lib, "_hpb_fused_hsdp_bound", False):
        return lib
    vp, ci, cu, cull, c64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint, ctypes.c_ulonglong, ctypes.c_int64
    pp = ctypes.POINTER(vp)
    cf = ctypes.c_float
    lib.hpb_p2p_allgather.argtypes = [pp, pp, vp, ci, vp, ci, ci, cu, cull, vp, vp, ci, vp]
    lib.hpb_p2p_allgather.restype = ci
    lib.hpb_fused_rs_adamw.argtypes = [pp, vp, pp, vp, ci, vp, vp, vp, vp, ctypes.POINTER(cf), ci, ci, cf, ci, ci,
                                       cu, cu, cull, vp, vp, ci, vp]
    lib.hpb_fused_rs_adamw.restype = ci
    lib.hpb_gemm2_agw.argtypes = [vp, c64, pp, vp, ci, c64, c64, vp, c64, ci, ci, ci, vp, cu, vp, ci, cu, cull,
                                  vp, ci, vp]
    lib.hpb_gemm2_agw.restype = ci
    pg = ctypes.POINTER(HpbGather)
    lib.hpb_gemm2_gather.argtypes = [vp, ci, c64, vp, ci, c64, vp, c64, ci, ci, ci, ci, pg, ci, pg, cull, vp, ci, vp]
    lib.hpb_gemm2_gather.restype = ci
    lib.hpb_gather_shape_ok.argtypes = [c64, c64, ci]
    lib.hpb_gather_shape_ok.restype = ci
    lib._hpb_fused_hsdp_bound = True
    return lib


class HpbGather(ctypes.Structure):
    """One weight to gather (mirror of the C struct of the same name)."""
    _fields_ = [("shard_ptrs", ctypes.POINTER(ctypes.c_void_p)), ("staging", ctypes.c_void_p),
                ("rows", ctypes.c_int64), ("cols", ctypes.c_int64), ("n", ctypes.c_int), ("rank", ctypes.c_int),
                ("counters", ctypes.c_void_p), ("seq", ctypes.c_uint), ("my_pad", ctypes.c_void_p),
                ("version_slot", ctypes.c_int), ("version", ctypes.c_uint)]


def rides_enabled() -> bool:
    """``HPB_RIDE=0``: a weight is gathered only by the GEMM that consumes it."""
    return os.environ.get("HPB_RIDE", "1") != "0"


class _Ticket:
    """A weight whose gather has been requested: it rides on the GEMMs that run before its consumer."""
    __slots__ = ("buf", "i", "spec", "left", "late")

    def __init__(self, buf, i, spec, nbytes, late):
        self.buf, self.i, self.spec, self.left, self.late = buf, i, spec, float(nbytes), late


# per device: tickets in the order in which their consumers will run
_RIDE_QUEUE: Dict[int, List[_Ticket]] = {}
_RIDE_GBS = 500.0         # bytes a host GEMM is assumed to move per second of its own duration (x 1e9)
_GEMM_TFLOPS = 1400.0


_RIDE_STATS = [] if os.environ.get("HPB_RIDE_STATS", "0") == "1" else None


def ride_stats():
    """``[(parameter, is_dgrad, fraction gathered before the consumer started)]`` (HPB_RIDE_STATS=1)."""
    return _RIDE_STATS


def _queue(device) -> List[_Ticket]:
    return _RIDE_QUEUE.setdefault(device.index, [])


def next_ride(device, flops: float, exclude=None):
    """The gather that a GEMM of ``flops`` floating-point operations should carry: the first ticket of
    the queue (tickets marked ``late`` only when nothing else waits).  The ticket's estimate of what
    is left shrinks by what this host can be expected to move; a ticket estimated complete leaves
    the queue (its consumer finishes whatever is really left)."""
    q = _RIDE_QUEUE.get(device.index)
    if not q:
        return None
    pick = None
    for t in q:
        if t is not exclude and not t.late:
            pick = t
            break
    if pick is None:
        for t in q:
            if t is not exclude:
                pick = t
                break
    if pick is None:
        return None
    pick.left -= flops / (_GEMM_TFLOPS * 1e12) * _RIDE_GBS * 1e9
    if pick.left <= 0:
        q.remove(pick)
    return pick.spec


class _StagingPool:
    """Full-size weight staging buffers, shared by all wrapped modules of a device: a module takes
    one at unshard and gives it back at reshard.  Reuse is ordered by the streams: a buffer is next
    written either by a GEMM on the compute stream or by the gather kernel, whose stream first waits
    for the compute stream."""

    def __init__(self):
        self.free: Dict[tuple, List[torch.Tensor]] = {}

    def take(self, numel: int, device) -> torch.Tensor:
        lst = self.free.get((device, numel))
        if lst:
            return lst.pop()
        return torch.empty(numel, dtype=torch.bfloat16, device=device)

    def give(self, t: torch.Tensor) -> None:
        self.free.setdefault((t.device, t.numel()), []).append(t)


_POOL = _StagingPool()


def _on_optimizer_step(optimizer, args, kwargs) -> None:
    """After ANY optimizer step: parameter shards that were rewritten outside the fused kernel get
    their new version published."""
    for buf in list(_LIVE):
        buf.after_optimizer_step()


def _install_step_hook() -> None:
    global _STEP_HOOK
    if _STEP_HOOK is None:
        from torch.optim.optimizer import register_optimizer_step_post_hook
        _STEP_HOOK = register_optimizer_step_post_hook(_on_optimizer_step)


class SymmParamBuffer:
    """Flat shard + flat gradient buffers of one HSDP state in symmetric memory."""

    def __init__(self, params, level3: bool):
        self.params = params
        p0 = params[0]
        self.group = p0.sharded_group_info.group
        self.n = p0.shard_size
        self.rank = p0.sharded_group_info.index
        self.device = p0.shard.device
        self.level3 = level3
        self.lib = _bind(native.lib())
        numels = [p.shard.numel() for p in params]
        self.numels = numels
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
        self.symm = SymmetricMemory(self.group, self.grad_byte_off + fo * 2, self.device, multicast=True)
        self.flat_shard = self.symm.tensor(torch.bfloat16, so, 0)
        self.flat_grad = self.symm.tensor(torch.bfloat16, fo, self.grad_byte_off)
        self.shard_ptrs = self.symm.ptr_table(0)
        self.grad_ptrs = self.symm.ptr_table(self.grad_byte_off)
        self.mc_grad = None if self.symm.mc_base is None else self.symm.mc_base + self.grad_byte_off
        for p, s, k in zip(params, self.shard_off, numels):
            view = self.flat_shard[s:s + k].view(p.shard_shape)
            view.copy_(p.shard)
            p.rebind_shard(view)
        self.grad_views = [self.flat_grad[f:f + k * self.n].view(p.full_shape)
                           for p, f, k in zip(params, self.full_off, numels)]
        # which parameters get their all-gather inside the consumer GEMM
        self.fusable = [self._fusable(p) for p in params]
        self.param_shard_ptrs = [self.symm.ptr_table(s * 2) for s in self.shard_off]
        self.panel_cnt: List[Optional[torch.Tensor]] = []
        for p, f in zip(params, self.fusable):
            rows = p.full_shape[0]
            # per-panel chunk counters, then the total, then the work-queue head
            self.panel_cnt.append(torch.zeros((rows + 127) // 128 + 2, dtype=torch.int32, device=self.device)
                                  if f else None)
        self.gather_seq = [0] * len(params)
        self.pending = [False] * len(params)
        self.tickets: List[Optional[_Ticket]] = [None] * len(params)
        self.specs: List[Optional[HpbGather]] = [None] * len(params)
        self._build_segments(None)
        self.status = native.status_word(self.device)
        self.staged_round = False     # tickets of the current unshard have been opened
        self.full: Optional[torch.Tensor] = None          # staging buffer while unsharded
        self.full_views: List[Optional[torch.Tensor]] = [None] * len(params)
        self.gather_event: Optional[torch.cuda.Event] = None
        self.reduce_event: Optional[torch.cuda.Event] = None
        self.grad_fresh = True        # nothing accumulated in flat_grad yet in this window
        self.ready = set()
        self.optimizer = None         # set by FusedAdamW.fuse_into_backward
        self.opt_state = None
        self.handle = None
        self.version = 0              # parameter-shard version published to the peers
        self._fused_step_done = False
        for i, p in enumerate(params):
            p._symm = (self, i)
        self.closed = False
        _LIVE.add(self)
        _install_step_hook()
        from ..ops import functional as _fn
        _fn.set_ride_provider(next_ride)
        if self.n > 1:
            # every rank's shards are in place before anybody gathers them
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)

    # ------------------------------------------------------------------ set-up --
    def _fusable(self, p) -> bool:
        """The fused gather takes 2-D weights that are only consumed by ``ops.linear`` (the model
        marks them ``_hpb_gemm_only``) and whose shape fits the kernel's granularity."""
        if not fused_gather_enabled() or self.n < 2 or not getattr(p.param, "_hpb_gemm_only", False):
            return False
        shape = p.full_shape
        if len(shape) != 2 or shape[1] % 64 or shape[0] % self.n:
            return False
        return shape[0] >= 256 and self.lib.hpb_gather_shape_ok(shape[0], shape[1], self.n) == 0

    def _build_segments(self, group_index) -> None:
        """Segment tables: all parameters (optimizer kernel) and the non-fusable ones (copy kernel)."""
        gi = group_index or [0] * len(self.params)
        rows = [[f, s, k, g] for f, s, k, g in zip(self.full_off, self.shard_off, self.numels, gi)]
        self.segs = torch.tensor(rows, dtype=torch.int64, device=self.device).contiguous()
        rest = [r for r, fz in zip(rows, self.fusable) if not fz]
        self.num_rest = len(rest)
        self.segs_rest = (torch.tensor(rest, dtype=torch.int64, device=self.device).contiguous()
                          if rest else None)

    def set_param_groups(self, group_index: List[int]) -> None:
        """``group_index[i]``: row of the hyper-parameter table used for parameter ``i``."""
        self._build_segments(group_index)

    # ------------------------------------------------------------- all-gather --
    def _take_staging(self) -> None:
        if self.full is None:
            self.full = _POOL.take(self.full_numel, self.device)
            self.full_views = [self.full[f:f + k * self.n].view(p.full_shape)
                               for p, f, k in zip(self.params, self.full_off, self.numels)]

    def prefetch(self) -> None:
        """Start gathering what the consumer GEMMs will not gather themselves."""
        if self.gather_event is not None or not self.params[0].is_sharded_now:
            return
        self._take_staging()
        self._open_tickets()
        if self.num_rest == 0:
            return
        cs = comm_stream(self.device)
        cur = torch.cuda.current_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(cur)
        cs.wait_event(ev)                       # everything that read the staging buffer before is finished
        with torch.cuda.stream(cs), tracing.nvtx_range("hpb.hsdp.allgather"):
            ep = self.symm.next_epoch()
            rc = self.lib.hpb_p2p_allgather(self.shard_ptrs, self.symm.pad_ptrs, self.segs_rest.data_ptr(),
                                            self.num_rest, self.full.data_ptr(), self.rank, self.n, ep,
                                            DEFAULT_WAIT_NS, self.status.data_ptr(),
                                            self.symm.done_counter.data_ptr(), _NUM_COMM_CTAS, cs.cuda_stream)
            native.check(rc, "hpb_p2p_allgather")
            self.gather_event = torch.cuda.Event()
            self.gather_event.record(cs)

    def _open_tickets(self) -> None:
        """Start a gather round for every weight that its consumer GEMM gathers: from now on the
        GEMMs that run before the consumer carry it (in consumption order: parameter order in a
        forward pass, the reverse inside a backward pass)."""
        if self.staged_round:
            return
        self.staged_round = True
        order = [i for i, f in enumerate(self.fusable) if f]
        if torch._C._current_graph_task_id() != -1:
            order.reverse()
        q = _queue(self.device)
        for i in order:
            p = self.params[i]
            rows, cols = p.full_shape
            self.gather_seq[i] += 1
            spec = self.specs[i]
            if spec is None:
                spec = HpbGather(ctypes.cast(self.param_shard_ptrs[i], ctypes.POINTER(ctypes.c_void_p)), 0, rows, cols, self.n, self.rank,
                                 self.panel_cnt[i].data_ptr(), 0, self.symm.pad_ptrs[self.rank],
                                 SLOT_SHARD_VERSION, 0)
                self.specs[i] = spec
            spec.staging = self.full_views[i].data_ptr()
            spec.seq = self.gather_seq[i]
            spec.version = self.version
            t = _Ticket(self, i, spec, rows * cols * 2, bool(getattr(p.param, "_hpb_gather_late", False)))
            self.tickets[i] = t
            if rides_enabled():
                q.append(t)

    def unshard(self) -> None:
        if not self.params[0].is_sharded_now:
            return
        if self.gather_event is None:
            self.prefetch()
        if self.gather_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self.gather_event)
            self.gather_event = None
        for i, (p, v) in enumerate(zip(self.params, self.full_views)):
            p.leaf.data = v
            p.is_sharded_now = False
            self.pending[i] = self.fusable[i]

    def reshard(self) -> None:
        for p in self.params:
            p.to_sharded()
        self.release_staging()

    def release_staging(self) -> None:
        """Hand the staging buffer back (the parameters point at their shards again)."""
        if self.full is not None and self.gather_event is None and all(p.is_sharded_now for p in self.params):
            for i, t in enumerate(self.tickets):
                if t is not None:
                    self._abandon(i)         # requested but never consumed
            _POOL.give(self.full)
            self.full = None
            self.full_views = [None] * len(self.params)
            self.pending = [False] * len(self.params)
            self.staged_round = False

    def gather_pending(self, i: int) -> bool:
        return self.pending[i]

    def _close_ticket(self, i: int):
        t = self.tickets[i]
        self.tickets[i] = None
        if t is not None:
            q = _RIDE_QUEUE.get(self.device.index)
            if q and t in q:
                q.remove(t)
        return t

    def _abandon(self, i: int) -> None:
        """A gather round that will not be completed by a consumer: forget it and zero the weight's
        counters (stream ordered), so that the next round starts from a clean queue."""
        self._close_ticket(i)
        self.panel_cnt[i].zero_()
        self.gather_seq[i] = 0

    def gather_gemm(self, i: int, a: torch.Tensor, out: torch.Tensor, w_mn: bool) -> None:
        """``out = a @ W_i^T`` (``w_mn=False``) or ``out = a @ W_i`` (``w_mn=True``).  This launch is
        the consumer of ``W_i``: its communication warps finish whatever part of the gather the
        earlier GEMMs have not done, its tiles wait for the panels they need; afterwards the
        parameter's full view holds the whole weight for any later consumer.  The launch also
        carries the gather of the next weight in the queue."""
        if a.stride(-1) != 1 or (a.stride(0) % 8) or (a.data_ptr() % 16):
            a = a.contiguous()
        t = self._close_ticket(i)
        spec = t.spec
        rows, cols = self.params[i].full_shape
        if _RIDE_STATS is not None:
            # diagnostic (HPB_RIDE_STATS=1, synchronises): how much of the weight the earlier GEMMs had
            # brought in by the time its consumer is launched
            torch.cuda.current_stream(self.device).synchronize()
            items = (rows * cols // 8 + (2047 if cols % 128 == 0 else 1023)) // (2048 if cols % 128 == 0 else 1024)
            done = int(self.panel_cnt[i][-2].item()) - (spec.seq - 1) * items
            _RIDE_STATS.append((self.params[i].name, int(w_mn), done / max(items, 1)))
        ride = next_ride(self.device, 2.0 * a.shape[0] * rows * cols)
        with tracing.nvtx_range("hpb.hsdp.allgather_gemm"):
            rc = self.lib.hpb_gemm2_gather(
                a.data_ptr(), 0, a.stride(0), None, 0, 0, out.data_ptr(), out.stride(0), 0, a.shape[0], 0, 0,
                ctypes.byref(spec), int(w_mn), ctypes.byref(ride) if ride is not None else None, DEFAULT_WAIT_NS,
                self.status.data_ptr(), native.sm_count(self.device), native.stream(self.device))
        native.check(rc, "hpb_gemm2_gather")
        self.pending[i] = False

    def materialize(self, i: int) -> None:
        """Gather parameter ``i`` now with the copy kernel (a consumer that is not ``ops.linear``)."""
        if not self.pending[i]:
            return
        self._abandon(i)
        seg = self.segs[i:i + 1].contiguous()
        ep = self.symm.next_epoch()
        rc = self.lib.hpb_p2p_allgather(self.shard_ptrs, self.symm.pad_ptrs, seg.data_ptr(), 1,
                                        self.full.data_ptr(), self.rank, self.n, ep, DEFAULT_WAIT_NS,
                                        self.status.data_ptr(), self.symm.done_counter.data_ptr(),
                                        _NUM_COMM_CTAS, native.stream(self.device))
        native.check(rc, "hpb_p2p_allgather")
        self.pending[i] = False

    # ------------------------------------------------------------------ grads --
    def wgrad_target(self, i: int):
        """(buffer view, accumulate?) for the weight-gradient GEMM of parameter ``i``."""
        if self.reduce_event is not None:
            # the previous reduction must have finished reading the buffer (on every rank)
            torch.cuda.current_stream(self.device).wait_event(self.reduce_event)
            self.reduce_event = None
        return self.grad_views[i], (not self.grad_fresh) or (i in self.ready)

    def num_grad_params(self) -> int:
        return sum(1 for p in self.params if p.param.requires_grad)

    def mark_ready(self, i: int) -> bool:
        self.ready.add(i)
        return len(self.ready) == self.num_grad_params()

    def store_grad(self, i: int, grad: torch.Tensor) -> bool:
        """Copy (or accumulate) an autograd-produced gradient into the flat buffer."""
        view, acc = self.wgrad_target(i)
        if acc:
            view.add_(grad.view_as(view))
        else:
            view.copy_(grad.view_as(view))
        return self.mark_ready(i)

    def flush_missing(self) -> bool:
        """End of a backward pass in which some parameters of this buffer received no gradient (an
        unused branch): their slots are zero-filled -- on every rank alike, so the ranks' kernels
        stay matched -- and the buffer counts as complete.  Returns True when there was anything to
        flush."""
        if not self.ready or len(self.ready) == self.num_grad_params():
            return False
        for i, p in enumerate(self.params):
            if p.param.requires_grad and i not in self.ready:
                view, acc = self.wgrad_target(i)
                if not acc:
                    view.zero_()
                self.ready.add(i)
        return True

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
        hyper = opt.hyper_table_for(self)
        cs = comm_stream(self.device)
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        cs.wait_event(ev)
        with torch.cuda.stream(cs), tracing.nvtx_range("hpb.hsdp.reduce_scatter_adamw"):
            ep = self.symm.next_epoch()
            self.version += 1
            self._fused_step_done = True
            rc = self.lib.hpb_fused_rs_adamw(
                self.grad_ptrs, self.mc_grad, self.symm.pad_ptrs, self.segs.data_ptr(), len(self.params),
                st["master"].data_ptr(), st["exp_avg"].data_ptr(), st["exp_avg_sq"].data_ptr(),
                self.flat_shard.data_ptr(), hyper, len(hyper) // 5, opt._step_count + 1, grad_scale, self.rank,
                self.n, ep, self.version, DEFAULT_WAIT_NS, self.status.data_ptr(),
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

    # --------------------------------------------------------------- versions --
    def close(self) -> None:
        """Give the symmetric region back (collective over the shard group; see
        ``SymmetricMemory.close``).  The buffer leaves the set that the optimizer post-step hook
        walks, so no later optimizer step -- of this or of any other model -- signals through pads
        that are no longer mapped."""
        if self.closed:
            return
        self.closed = True
        _LIVE.discard(self)
        self.release_staging()
        self.tickets = [None] * len(self.params)
        self.symm.close()

    def after_optimizer_step(self) -> None:
        """Runs after every optimizer step.  If the fused kernel rewrote the shards in this step it
        has published the new version itself; otherwise (an optimizer that writes the shards with
        its own kernels) publish it now, ordered after those kernels on the current stream."""
        if self.closed:
            return
        if self._fused_step_done:
            self._fused_step_done = False
            return
        self.params_written()

    def params_written(self) -> None:
        """The shards of this buffer were rewritten on the current stream (optimizer step, state-dict
        load): publish a new version.  Every rank must call it the same number of times."""
        if self.closed:
            raise RuntimeError("this HSDP buffer was closed (teardown_hsdp); its model cannot be stepped any more")
        self.version += 1
        if self.n > 1:
            self.symm.signal(SLOT_SHARD_VERSION, self.version)
