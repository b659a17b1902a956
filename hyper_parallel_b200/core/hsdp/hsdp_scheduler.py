"""Hook scheduler that drives an :class:`HSDPState` through forward and backward.

State machine and hook placement follow hyper_parallel/core/hsdp/hsdp_scheduler.py:40-174
and hyper_parallel/platform/torch/hsdp/scheduler.py:51-106 of the reference:

* forward-pre  : unshard (consume a prefetch if one is in flight) + start the forward
  prefetch of the configured cells;
* forward-post : level3 only -- reshard; install backward hooks: a tensor hook on the
  outputs (backward-pre: unshard again + backward prefetch) and an identity
  ``autograd.Function`` on the inputs (backward-post: reshard);
* per-parameter post-accumulate hooks reduce the gradient (see ``hsdp_grad_hook``);
* one engine callback per backward pass reshards what is left, and -- in synchronous
  mode -- installs the reduced gradients as ``param.grad``; in asynchronous mode that
  happens in :func:`hsdp_sync_stream`.
"""
from __future__ import annotations

import enum
from typing import List

import torch
from torch.autograd import Variable

from .hsdp_grad_hook import PendingReduce
from .hsdp_state import HSDPState
from .hsdp_utils import HSDPConfig, OptimizerLevel

_ALL_SCHEDULERS: List["HSDPScheduler"] = []
_PENDING: List[PendingReduce] = []
_ROOT_CALLBACK_QUEUED = False


class FwdBwdState(enum.Enum):
    PRE_FORWARD = 0
    FORWARD = 1
    PRE_BACKWARD = 2
    BACKWARD = 3


class _PostBackward(torch.autograd.Function):
    """Identity on the module inputs; its backward runs after the module's backward."""

    @staticmethod
    def forward(ctx, scheduler, *inputs):
        ctx.scheduler = scheduler
        return inputs if len(inputs) > 1 else inputs[0]

    @staticmethod
    def backward(ctx, *grads):
        ctx.scheduler._backward_post()
        return (None,) + grads


def _tree_tensors(obj, fn):
    if isinstance(obj, torch.Tensor):
        return fn(obj)
    if isinstance(obj, (list, tuple)):
        return type(obj)(_tree_tensors(o, fn) for o in obj)
    if isinstance(obj, dict):
        return {k: _tree_tensors(v, fn) for k, v in obj.items()}
    return obj


def _drain_pending() -> None:
    while _PENDING:
        _PENDING.pop(0).wait()


def _install_grads(state: HSDPState) -> None:
    for hp in state.hsdp_params:
        if hp.reduced_grad is not None:
            g = hp.reduced_grad
            hp.reduced_grad = None
            if g.shape != hp.leaf.shape:
                g = g.reshape(hp.leaf.shape)
            hp.leaf.grad = g
    if state.config.requires_acc_grad and not state.grad_hook.requires_grad_sync:
        # A micro-step without synchronisation: ``param.grad`` shows the running accumulator (this
        # rank's rows of it where the accumulator is kept at full size), as the reference's hooks do by
        # returning it (core/hsdp/hsdp_grad_hook.py:60-150 there).  It is a view, valid until the next
        # forward of the cell, which takes it away again so that autograd never adds into it.
        for hp in state.hsdp_params:
            acc = hp.acc_grad
            if acc is None or hp.leaf.grad is not None:
                continue
            if acc.shape != hp.leaf.shape:
                if not hp.sharded or acc.shape != hp.full_shape:
                    continue
                acc = acc.chunk(hp.shard_size, dim=0)[hp.sharded_group_info.index]
                if acc.shape != hp.leaf.shape:
                    continue
            hp.leaf.grad = acc.detach()
            hp._acc_exposed = True


def _root_backward_callback() -> None:
    global _ROOT_CALLBACK_QUEUED
    _ROOT_CALLBACK_QUEUED = False
    for sch in _ALL_SCHEDULERS:
        # buckets that are only partly filled (a parameter got no gradient in this pass) are
        # completed with zeros and reduced now; afterwards no bucket keeps stale entries
        _PENDING.extend(sch.hsdp_state.flush_partial_buckets())
        sch.hsdp_state.reset_buckets()
    for sch in _ALL_SCHEDULERS:
        if sch.state in (FwdBwdState.PRE_BACKWARD, FwdBwdState.BACKWARD) or not sch.hsdp_state.is_sharded:
            sch.hsdp_state.shard()
        sch.state = FwdBwdState.PRE_FORWARD
        for hp in sch.hsdp_state.hsdp_params:
            hp.grad_ready = False
        if not sch.config.comm_async:
            _install_grads(sch.hsdp_state)
    if not any(s.config.comm_async for s in _ALL_SCHEDULERS):
        _drain_pending()


def hsdp_sync_stream() -> None:
    """Wait for every in-flight gradient reduction and install the reduced gradients.

    Call it after ``backward()`` and before ``optimizer.step()`` when ``comm_async=True``
    (hyper_parallel/core/hsdp/api.py:268-272 of the reference).  Harmless otherwise.
    """
    _drain_pending()
    for sch in _ALL_SCHEDULERS:
        for buf in sch.hsdp_state.symm_buffers:
            buf.wait()
        _install_grads(sch.hsdp_state)


class HSDPScheduler:
    def __init__(self, cell, config: HSDPConfig, params):
        self.cell = cell
        self.config = config
        self.hsdp_state = HSDPState(cell, config, params)
        self.state = FwdBwdState.PRE_FORWARD
        self.forward_prefetch_cells: List = []
        self.backward_prefetch_cells: List = []
        self.level3 = config.shard_level == OptimizerLevel.SHARD_OPT_GRAD_PARAM
        self._bind_symm_buffers()
        self._register_hooks()
        _ALL_SCHEDULERS.append(self)

    def _bind_symm_buffers(self) -> None:
        """Let the wgrad GEMM write straight into the symmetric gradient buffers."""
        for buf in self.hsdp_state.symm_buffers:
            buf.on_all_ready = (lambda b=buf: self._symm_ready(b))
            for i, hp in enumerate(buf.params):
                hp.param._hpb_symm = (buf, i)
                if hp.leaf is not hp.param:
                    # tensor-parallel layers hand the local tensor of a DTensor parameter to the GEMMs
                    hp.leaf._hpb_symm = (buf, i)

    def _symm_ready(self, buf) -> None:
        for hp in buf.params:
            hp.grad_ready = True
        self._queue_root_callback()
        self.hsdp_state.symm_bucket_done(buf)

    # ---------------------------------------------------------------- hooks --
    def _register_hooks(self) -> None:
        self.cell.register_forward_pre_hook(self._forward_pre, with_kwargs=True)
        self.cell.register_forward_hook(self._forward_post)
        for hp in self.hsdp_state.hsdp_params:
            if hp.param.requires_grad:
                hp._grad_hook_fn = self._make_grad_hook(hp)
                hp.leaf.register_post_accumulate_grad_hook(hp._grad_hook_fn)

    def _make_grad_hook(self, hp):
        def hook(leaf):
            grad = leaf.grad
            leaf.grad = None
            if grad is None:
                return
            hp.grad_ready = True
            self._queue_root_callback()
            symm = getattr(hp, "_symm", None)
            if symm is not None:
                buf, i = symm
                if buf.store_grad(i, grad):
                    self.hsdp_state.symm_bucket_done(buf)
                return
            pending = self.hsdp_state.reduce_grad(hp, grad)
            if pending is not None:
                _PENDING.append(pending)
            elif hp.reduced_grad is not None and hp.grad_consumer is not None:
                # e.g. the optimizer fused into backward: use the shard gradient now, then drop it
                g, hp.reduced_grad = hp.reduced_grad, None
                hp.grad_consumer(hp, g)
        return hook

    @staticmethod
    def _queue_root_callback() -> None:
        global _ROOT_CALLBACK_QUEUED
        if not _ROOT_CALLBACK_QUEUED:
            _ROOT_CALLBACK_QUEUED = True
            Variable._execution_engine.queue_callback(_root_backward_callback)

    def _forward_pre(self, cell, args, kwargs):
        if self.config.requires_acc_grad:
            for hp in self.hsdp_state.hsdp_params:
                if getattr(hp, "_acc_exposed", False):
                    hp.leaf.grad = None
                    hp._acc_exposed = False
        self.hsdp_state.unshard()
        self.state = FwdBwdState.FORWARD
        for c in self.forward_prefetch_cells:
            sch = getattr(c, "hsdp_scheduler", None)
            if sch is not None:
                sch.hsdp_state.prefetch()
        if not torch.is_grad_enabled():
            return args, kwargs
        tensors = [a for a in args if isinstance(a, torch.Tensor) and a.requires_grad]
        if not tensors:
            return args, kwargs
        wrapped = _PostBackward.apply(self, *tensors)
        if not isinstance(wrapped, tuple):
            wrapped = (wrapped,)
        it = iter(wrapped)
        new_args = tuple(next(it) if (isinstance(a, torch.Tensor) and a.requires_grad) else a for a in args)
        return new_args, kwargs

    def _forward_post(self, cell, args, output):
        if self.level3:
            self.hsdp_state.shard()
        self.state = FwdBwdState.PRE_BACKWARD
        if torch.is_grad_enabled():
            def reg(t):
                if t.requires_grad:
                    t.register_hook(self._backward_pre)
                return t
            _tree_tensors(output, reg)
        return output

    def _backward_pre(self, grad):
        self._queue_root_callback()
        if self.state != FwdBwdState.BACKWARD:
            self.hsdp_state.unshard()
            self.state = FwdBwdState.BACKWARD
            for c in self.backward_prefetch_cells:
                sch = getattr(c, "hsdp_scheduler", None)
                if sch is not None:
                    sch.hsdp_state.prefetch()
        return grad

    def _backward_post(self) -> None:
        # reshard now only when every gradient of this cell has been produced; otherwise the
        # end-of-backward callback does it
        if all(hp.grad_ready or not hp.param.requires_grad for hp in self.hsdp_state.hsdp_params):
            self.hsdp_state.shard()
            self.state = FwdBwdState.PRE_FORWARD

    # ------------------------------------------------------------- controls --
    def set_requires_grad_sync(self, flag: bool) -> None:
        self.hsdp_state.set_requires_grad_sync(flag)

    def zero_grads(self) -> None:
        self.hsdp_state.zero_grads()

    def set_forward_prefetch_cells(self, cells) -> None:
        self.forward_prefetch_cells = list(cells)

    def set_backward_prefetch_cells(self, cells) -> None:
        self.backward_prefetch_cells = list(cells)


def reset_hsdp_registry() -> None:
    """Forget every scheduler (tests build many models in one process)."""
    _ALL_SCHEDULERS.clear()
    _PENDING.clear()


def teardown_hsdp(root) -> None:
    """Give back what ``hsdp()`` allocated outside the caching allocator for the modules below
    ``root``: the symmetric-memory regions (flat shards and gradient buffers, mapped by the peers)
    are closed, the staging buffers and the queue of pending weight gathers dropped, the registry
    forgotten.  Collective -- every rank calls it, with no kernel of the model in flight -- and the
    model must not be used afterwards."""
    import torch
    from ...parallel import fused_hsdp
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    for mod in root.modules():
        sch = mod.__dict__.get("hsdp_scheduler")
        if sch is None:
            continue
        for buf in list(getattr(sch.hsdp_state, "symm_buffers", [])):
            buf.close()
        sch.hsdp_state.symm_buffers = []
    fused_hsdp._RIDE_QUEUE.clear()
    fused_hsdp._POOL.free.clear()
    reset_hsdp_registry()
