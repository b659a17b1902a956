"""Per-wrapped-module HSDP state: its parameters, fused parameter buffers and gradient buckets.

Mirrors the roles of hyper_parallel/core/hsdp/hsdp_state.py:20-161,
hsdp_param_buffer.py:18-105 and hsdp_grad_buffer.py:19-236 of the reference.

* ``HSDPParamBuffer`` (``comm_fusion``): all sharded parameters of one (shard group, dtype)
  live in ONE flat shard buffer; unsharding is one all-gather of that buffer followed by a
  copy-out into the per-parameter full tensors (the asynchronous gather is waited before
  the copy-out).
* ``HSDPGradBuffer`` (``comm_fusion`` and ``bucket_size != 0``): gradients of a bucket are
  packed as ``(shard_size, numel / shard_size)`` once all of them are ready, reduced with one
  reduce-scatter (+ one all-reduce across replicas) and handed back as per-parameter views.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ...collectives import cc
from .hsdp_grad_hook import HSDPGradHook, PendingReduce
from .hsdp_param import HSDPParam
from .hsdp_utils import HSDPConfig, OptimizerLevel


class HSDPParamBuffer:
    """Flat shard buffer + one all-gather for every parameter of a (shard group, dtype)."""

    def __init__(self, params: List[HSDPParam]):
        self.params = params
        p0 = params[0]
        self.group = p0.sharded_group_info.group
        self.shard_size = p0.shard_size
        numels = [p.shard.numel() for p in params]
        self.offsets = [0]
        for n in numels:
            self.offsets.append(self.offsets[-1] + n)
        total = self.offsets[-1]
        self.flat_shard = torch.empty(total, dtype=p0.shard.dtype, device=p0.shard.device)
        for p, o, n in zip(params, self.offsets, numels):
            view = self.flat_shard[o:o + n].view(p.shard_shape)
            if p.shard.device.type != "meta":
                view.copy_(p.shard)
            p.rebind_shard(view)
        self.handle = None
        self.gathered: Optional[torch.Tensor] = None

    def prefetch(self) -> None:
        if self.handle is not None or not self.params[0].is_sharded_now:
            return
        self.gathered = torch.empty(self.shard_size * self.flat_shard.numel(),
                                    dtype=self.flat_shard.dtype, device=self.flat_shard.device)
        work = cc.all_gather_into(self.gathered, self.flat_shard, self.group, async_op=True)
        self.handle = work if work is not None else True

    def unshard(self) -> None:
        if not self.params[0].is_sharded_now:
            return
        if self.handle is None:
            self.prefetch()
        if self.handle is not True:
            self.handle.wait()
        self.handle = None
        g = self.gathered.view(self.shard_size, -1)
        for p, o in zip(self.params, self.offsets):
            n = p.shard.numel()
            full = p._full_buffer()
            full.view(self.shard_size, -1).copy_(g[:, o:o + n])
            p.leaf.data = full
            p.is_sharded_now = False
        self.gathered = None

    def reshard(self) -> None:
        for p in self.params:
            p.to_sharded()


class HSDPGradBuffer:
    """One gradient bucket: pack -> one reduce-scatter / all-reduce -> per-parameter views."""

    def __init__(self, params: List[HSDPParam], config: HSDPConfig):
        self.params = params
        self.config = config
        self.ready: Dict[int, torch.Tensor] = {}

    def add(self, hp: HSDPParam, grad: torch.Tensor) -> bool:
        self.ready[id(hp)] = grad
        return len(self.ready) == len(self.params)

    def reduce(self, sync: bool) -> Optional[PendingReduce]:
        cfg = self.config
        p0 = self.params[0]
        ss = p0.shard_size
        grads = [self.ready[id(p)] for p in self.params]
        self.ready = {}
        orig_dtype = grads[0].dtype
        rd = cfg.reduce_dtype or orig_dtype
        level1 = cfg.shard_level == OptimizerLevel.SHARD_OPT
        acc = cfg.requires_acc_grad
        for p in self.params:
            p.reduced_grad = None
        if acc and level1:
            for p, g in zip(self.params, grads):
                p.ensure_acc_grad(g).add_(g)
            if not sync:
                return None
            grads = [p.acc_grad for p in self.params]
        packed = torch.cat([g.reshape(ss, -1).to(rd) for g in grads], dim=1).contiguous()
        works: list = []
        if ss > 1:
            out = torch.empty(packed.shape[1], dtype=rd, device=packed.device)
            works.append(cc.reduce_scatter_into(out, packed.view(-1), p0.sharded_group_info.group, "sum",
                                                async_op=cfg.comm_async))
        else:
            out = packed.view(-1)

        def views(flat):
            res, o = [], 0
            for p in self.params:
                n = p.shard.numel() if p.sharded else p.leaf.numel()
                res.append(flat[o:o + n].view(p.shard_shape))
                o += n
            return res

        if acc and not level1:
            for w in works:
                if w is not None:
                    w.wait()
            works = []
            for p, v in zip(self.params, views(out)):
                p.ensure_acc_grad(v).add_(v)
            if not sync:
                return None
            out = torch.cat([p.acc_grad.reshape(-1) for p in self.params])
        if p0.dp_size > 1:
            for w in works:
                if w is not None:
                    w.wait()
            works = [cc.all_reduce_(out, "sum", p0.unsharded_group_info.group, async_op=cfg.comm_async)]

        def post():
            flat = out.to(orig_dtype) if out.dtype != orig_dtype else out
            if cfg.grad_scale != 1.0:
                flat = flat * cfg.grad_scale
            for p, v in zip(self.params, views(flat)):
                p.reduced_grad = v

        if any(w is not None for w in works):
            return PendingReduce(works, post)
        post()
        return None


class HSDPState:
    """All HSDP-managed parameters of one wrapped module."""

    def __init__(self, cell, config: HSDPConfig, params: List[Tuple[str, torch.nn.Parameter]]):
        self.cell = cell
        self.config = config
        self.hsdp_params: List[HSDPParam] = [HSDPParam(n, p, config) for n, p in params]
        self.sharded_params = [p for p in self.hsdp_params if p.sharded]
        self.grad_hook = HSDPGradHook(config)
        self.param_buffers: List[HSDPParamBuffer] = []
        self.symm_buffers: list = []
        self.grad_buffers: List[HSDPGradBuffer] = []
        self._bucket_of: Dict[int, HSDPGradBuffer] = {}
        self.is_sharded = True
        if config.comm_fusion:
            self._init_param_buffers()
        if config.grad_fusion:
            self._init_grad_buffers()

    def _init_param_buffers(self) -> None:
        groups: Dict[tuple, List[HSDPParam]] = {}
        for p in self.sharded_params:
            groups.setdefault((p.sharded_group_info.ranks, p.shard.dtype, p.shard.device), []).append(p)
        self._in_buffer = set()
        from ...parallel import fused_hsdp
        level3 = self.config.shard_level == OptimizerLevel.SHARD_OPT_GRAD_PARAM
        for plist in groups.values():
            rest = plist
            if plist[0].shard.device.type == "cuda":
                # the parameters that can live in symmetric memory do; one odd parameter (fp32, a
                # DTensor, a shard that is not a whole number of vectors) no longer sends its whole
                # group to the NCCL buffers
                symm, rest = fused_hsdp.split_eligible(plist)
                if symm:
                    buf = fused_hsdp.SymmParamBuffer(symm, level3)   # NVLink gather + fused RS/AdamW
                    self.symm_buffers.append(buf)
                    self.param_buffers.append(buf)
                    self._in_buffer.update(id(p) for p in symm)
            if len(rest) > 1:
                self.param_buffers.append(HSDPParamBuffer(rest))
                self._in_buffer.update(id(p) for p in rest)

    def rebuild_param_buffers(self) -> None:
        """Re-create the flat parameter buffers from the current shards (after materialisation)."""
        if self.config.comm_fusion:
            for b in self.symm_buffers:
                b.symm.close()
            self.param_buffers, self.symm_buffers = [], []
            self._init_param_buffers()
            if self.config.grad_fusion:
                self.grad_buffers, self._bucket_of = [], {}
                self._init_grad_buffers()

    def _init_grad_buffers(self) -> None:
        groups: Dict[tuple, List[HSDPParam]] = {}
        for p in self.hsdp_params:
            if not p.param.requires_grad or getattr(p, "_symm", None) is not None:
                continue
            key = (p.sharded_group_info.ranks, p.unsharded_group_info.ranks, p.leaf.dtype, p.shard_size)
            groups.setdefault(key, []).append(p)
        limit = self.config.bucket_size
        for plist in groups.values():
            bucket, size = [], 0
            for p in plist:
                nbytes = p.leaf.element_size() * int(torch.Size(p.full_shape).numel())
                if bucket and limit > 0 and size + nbytes > limit:
                    self._add_bucket(bucket)
                    bucket, size = [], 0
                bucket.append(p)
                size += nbytes
            if bucket:
                self._add_bucket(bucket)

    def _add_bucket(self, plist: List[HSDPParam]) -> None:
        b = HSDPGradBuffer(plist, self.config)
        self.grad_buffers.append(b)
        for p in plist:
            self._bucket_of[id(p)] = b

    # ------------------------------------------------------------- (un)shard --
    def unshard(self) -> None:
        if not self.is_sharded:
            return
        in_buf = getattr(self, "_in_buffer", set())
        for b in self.param_buffers:
            b.unshard()
        # launch every gather first, then wait: the collectives overlap each other
        rest = [p for p in self.sharded_params if id(p) not in in_buf]
        for p in rest:
            p.prefetch_unsharded()
        for p in rest:
            p.to_unsharded()
        self.is_sharded = False

    def prefetch(self) -> None:
        if not self.is_sharded:
            return
        in_buf = getattr(self, "_in_buffer", set())
        for b in self.param_buffers:
            b.prefetch()
        for p in self.sharded_params:
            if id(p) not in in_buf:
                p.prefetch_unsharded()

    def shard(self) -> None:
        if self.is_sharded:
            return
        for p in self.sharded_params:
            p.to_sharded()
        for b in self.symm_buffers:
            b.release_staging()          # the gathered weights do not outlive their consumers
        self.is_sharded = True

    # ----------------------------------------------------------------- grads --
    def reduce_grad(self, hp: HSDPParam, grad: torch.Tensor) -> Optional[PendingReduce]:
        bucket = self._bucket_of.get(id(hp))
        if bucket is None:
            return self.grad_hook.process(hp, grad)
        if bucket.add(hp, grad):
            return bucket.reduce(self.grad_hook.requires_grad_sync)
        return None

    def symm_bucket_done(self, buf) -> None:
        """Every gradient of a symmetric buffer has been written: reduce (and step) it."""
        sync = self.grad_hook.requires_grad_sync
        if buf.reduce_and_step(sync, self.config.grad_scale):
            return
        # no fused optimizer attached: reduce-scatter each parameter's gradient with NCCL
        for hp, view in zip(buf.params, buf.grad_views):
            if hp.param.requires_grad:
                self.grad_hook.process(hp, view)
        buf.grad_fresh = True

    def flush_partial_buckets(self):
        """End of a backward pass: buckets in which some parameters produced no gradient (an unused
        branch, an expert without tokens) are completed with zeros -- every rank does the same, so
        the collectives stay matched -- and reduced.  Returns the pending reductions."""
        pending = []
        sync = self.grad_hook.requires_grad_sync
        for b in self.grad_buffers:
            if not b.ready or len(b.ready) == len(b.params):
                continue
            for p in b.params:
                if id(p) not in b.ready:
                    b.ready[id(p)] = torch.zeros(p.full_shape, dtype=p.leaf.dtype, device=p.leaf.device)
            r = b.reduce(sync)
            if r is not None:
                pending.append(r)
        for buf in self.symm_buffers:
            if buf.flush_missing():
                self.symm_bucket_done(buf)
        return pending

    def reset_buckets(self) -> None:
        """Nothing of one backward pass leaks into the next."""
        for b in self.grad_buffers:
            b.ready = {}
        for buf in self.symm_buffers:
            buf.ready = set()

    def zero_grads(self) -> None:
        for b in self.symm_buffers:
            b.grad_fresh = True
            b.ready = set()
        for p in self.hsdp_params:
            p.zero_acc_grad()
            p.reduced_grad = None
            p.leaf.grad = None

    def set_requires_grad_sync(self, flag: bool) -> None:
        self.grad_hook.set_requires_grad_sync(flag)
