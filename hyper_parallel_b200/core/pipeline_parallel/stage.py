"""``PipelineStage``: one (virtual) pipeline stage -- its module, peers and p2p transfers.

Behaviour follows hyper_parallel/core/pipeline_parallel/stage.py:58-345 and
hyper_parallel/platform/torch/pipeline_parallel/stage.py:21-130 of the reference:

* ``stage_num`` counts **virtual** stages; with ``v`` chunks per rank there are
  ``stage_num / v`` real stages, each owning ``world / real_stages`` consecutive ranks; virtual
  stage ``s`` lives on real stage ``s % real_stages`` (loop placement);
* the peer of this rank for another stage is the rank at the same offset inside that stage;
* the first transfer on a link (every transfer with ``dyn_shape``) sends a small metadata list
  (shape, dtype, DTensor placements) with ``send_object_list``; tensors go with ``isend/irecv``;
  a received DTensor is re-based onto this stage's own mesh;
* the backward of the last stage is seeded with ``1 / repeat_num`` per output;
* tied ("shared") parameters are broadcast from their first stage at init and their gradients
  are all-reduced after the schedule.

Stage boundaries stay on NCCL p2p by design; the receive of micro-batch ``i+1`` is posted
while micro-batch ``i`` computes (``overlap_p2p``).
"""
from __future__ import annotations

import os

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ...collectives import cc
from ..device_mesh import init_device_mesh
from ..dtensor import DTensor, _build_layout


@dataclass
class SharedParameterInfo:
    """A parameter tied across pipeline stages (e.g. input embedding and output head)."""
    parameter: torch.nn.Parameter
    shared_stage: Sequence[int]


class _Pending:
    """An in-flight p2p receive: buffers + handles + how to rebuild the values."""

    def __init__(self, works, buffers, metas):
        self.works, self.buffers, self.metas = works, buffers, metas

    def wait(self):
        for w in self.works:
            w.wait()
        self.works = []


class PipelineStage:
    def __init__(self, submodule: torch.nn.Module, stage_index: int, stage_num: int, device=None,
                 group=None, src_stage: Optional[int] = None, dst_stage: Optional[int] = None,
                 dyn_shape: bool = False, has_backward: bool = True,
                 shared_parameters: Optional[List[SharedParameterInfo]] = None):
        if not 0 <= stage_index < stage_num:
            raise ValueError(f"stage_index {stage_index} out of range for {stage_num} stages")
        self.submodule = submodule
        self.stage_index = stage_index
        self.stage_num = stage_num
        self.device = device
        self.group = group
        self.dyn_shape = dyn_shape
        self.has_backward = has_backward
        self.shared_parameters = list(shared_parameters or [])
        self.is_first = stage_index == 0
        self.is_last = stage_index == stage_num - 1
        self.src_stage = src_stage if src_stage is not None else (None if self.is_first else stage_index - 1)
        self.dst_stage = dst_stage if dst_stage is not None else (None if self.is_last else stage_index + 1)
        self._inited = False
        self.clear_cache()

    # --------------------------------------------------------------- set-up --
    def init(self, virtual_chunk_num: int = 1) -> None:
        if self._inited:
            return
        self.rank = cc.get_rank()
        self.world = cc.get_world_size()
        if self.stage_num % virtual_chunk_num:
            raise ValueError(f"{self.stage_num} stages cannot be split into {virtual_chunk_num} chunks per rank")
        self.real_stage_num = self.stage_num // virtual_chunk_num
        if self.world % self.real_stage_num:
            raise ValueError(f"world size {self.world} is not divisible by {self.real_stage_num} pipeline stages")
        self.device_num_per_stage = self.world // self.real_stage_num
        self.real_stage_index = self.stage_index % self.real_stage_num
        if self.rank // self.device_num_per_stage != self.real_stage_index:
            raise ValueError(f"rank {self.rank} does not belong to pipeline stage {self.stage_index} "
                             f"(real stage {self.real_stage_index} owns ranks "
                             f"[{self.real_stage_index * self.device_num_per_stage}, "
                             f"{(self.real_stage_index + 1) * self.device_num_per_stage}))")
        self.pp_ranks = [self.rank + self.device_num_per_stage * (i - self.real_stage_index)
                         for i in range(self.real_stage_num)]
        # One process group (communicator + stream) per ordered neighbour pair and traffic
        # direction: activations and gradients then do not queue behind each other, which a single
        # communicator would force.  The groups of all pipeline rings are created by all ranks of
        # the world in the same order (every rank builds its stage with the same configuration).
        self._p2p_groups = {}
        if self.real_stage_num > 1 and os.environ.get("HPB_PP_SPLIT_GROUPS", "1") != "0":
            links = [(i, i + 1) for i in range(self.real_stage_num - 1)]
            if virtual_chunk_num > 1:
                links.append((self.real_stage_num - 1, 0))
            specs, meaning = [], {}
            for ring in range(self.device_num_per_stage):
                ring_ranks = [ring + self.device_num_per_stage * i for i in range(self.real_stage_num)]
                for a, b in links:
                    for src, dst, kind in ((a, b, "f"), (b, a, "b")):
                        rs, rd = ring_ranks[src], ring_ranks[dst]
                        spec = (tuple(sorted((rs, rd))), f"pp-{rs}-{rd}-{kind}")
                        specs.append(spec)
                        meaning[spec] = (rs, rd, kind)
            for spec, grp in cc.world_collective_groups(specs).items():
                self._p2p_groups[meaning[spec]] = grp
        self._shared_groups = []
        for info in self.shared_parameters:
            ranks = sorted({self.peer_rank(s) for s in info.shared_stage})
            grp = cc.group_for_ranks(ranks) if len(ranks) > 1 else None
            self._shared_groups.append((info, ranks, grp))
            if grp is not None:
                leaf = info.parameter.to_local() if isinstance(info.parameter, DTensor) else info.parameter
                cc.broadcast(leaf.data, src=ranks[0], group=grp)
        self._inited = True

    def peer_rank(self, stage: int) -> int:
        """Global rank that plays my role inside (virtual) stage ``stage``."""
        real = stage % self.real_stage_num
        return self.rank + self.device_num_per_stage * (real - self.real_stage_index)

    def clear_cache(self) -> None:
        self.fwd_cache: Dict[int, Tuple[tuple, Any]] = {}
        self.meta_cache: Dict[Tuple[str, int], list] = {}
        self._sent_meta: set = set()
        self.input_grads: Dict[int, list] = {}
        self._pending_sends: list = []

    # ------------------------------------------------------------------ p2p --
    clear_states = clear_cache          # the reference's name (core/pipeline_parallel/stage.py:115-118)

    def _dev(self):
        if self.device is not None:
            return torch.device(self.device)
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")

    @staticmethod
    def _describe(t) -> list:
        if isinstance(t, DTensor):
            lay = t.layout
            return [tuple(t.to_local().shape), t.dtype, (lay.mesh_shape, lay.alias_name, lay.placements)]
        return [tuple(t.shape), t.dtype, None]

    def _rebuild(self, buf: torch.Tensor, meta) -> torch.Tensor:
        lay = meta[2]
        if lay is None:
            return buf
        mesh_shape, names, placements = lay
        mesh = init_device_mesh("cuda", mesh_shape, mesh_dim_names=names)   # this stage's own block of ranks
        return DTensor._wrap(buf, _build_layout(mesh, placements, buf.dim()))

    def _send(self, tensors: Sequence[torch.Tensor], dst_rank: int, key: Tuple[str, int]) -> None:
        grp = self._p2p_groups.get((self.rank, dst_rank, key[0]))
        need_meta = self.dyn_shape or key not in self._sent_meta
        if need_meta:
            dist.send_object_list([[self._describe(t) for t in tensors]], dst=dst_rank, group=grp)
            self._sent_meta.add(key)
        for t in tensors:
            local = t.to_local() if isinstance(t, DTensor) else t
            self._pending_sends.append((dist.isend(local.detach().contiguous(), dst=dst_rank, group=grp), local))

    def _post_recv(self, src_rank: int, key: Tuple[str, int]) -> _Pending:
        grp = self._p2p_groups.get((src_rank, self.rank, key[0]))
        metas = None if self.dyn_shape else self.meta_cache.get(key)
        if metas is None:
            box = [None]
            dist.recv_object_list(box, src=src_rank, group=grp)
            metas = box[0]
            self.meta_cache[key] = metas
        dev = self._dev()
        bufs = [torch.empty(m[0], dtype=m[1], device=dev) for m in metas]
        works = [dist.irecv(b, src=src_rank, group=grp) for b in bufs]
        return _Pending(works, bufs, metas)

    def wait_sends(self) -> None:
        for w, _keep in self._pending_sends:
            w.wait()
        self._pending_sends = []

    # forward direction ---------------------------------------------------
    def post_forward_recv(self) -> _Pending:
        return self._post_recv(self.peer_rank(self.src_stage), ("f", self.src_stage))

    def finish_forward_recv(self, pending: _Pending) -> tuple:
        pending.wait()
        vals = []
        for b, m in zip(pending.buffers, pending.metas):
            v = self._rebuild(b, m)
            if self.has_backward and b.is_floating_point():
                (v.to_local() if isinstance(v, DTensor) else v).requires_grad_(True)
            vals.append(v)
        return tuple(vals)

    def send_forward(self, micro: int) -> None:
        _, outputs = self.fwd_cache[micro]
        outs = outputs if isinstance(outputs, (tuple, list)) else (outputs,)
        self._send([o for o in outs if isinstance(o, torch.Tensor)], self.peer_rank(self.dst_stage),
                   ("f", self.dst_stage))

    # backward direction --------------------------------------------------
    def post_backward_recv(self) -> _Pending:
        return self._post_recv(self.peer_rank(self.dst_stage), ("b", self.dst_stage))

    def send_backward(self, micro: int) -> None:
        grads = self.input_grads.pop(micro)
        self._send(grads, self.peer_rank(self.src_stage), ("b", self.src_stage))

    # ---------------------------------------------------------------- compute --
    def forward_one_chunk(self, micro: int, args: tuple, kwargs: Optional[dict] = None):
        out = self.submodule(*args, **(kwargs or {}))
        self.fwd_cache[micro] = (args, out)
        return out

    def get_last_stage_sens(self, outputs) -> list:
        """Backward seeds of the last stage: ``1 / repeat_num`` for every output element."""
        sens = []
        for o in outputs:
            rep = o.layout.repeat_num() if isinstance(o, DTensor) else 1
            local = o.to_local() if isinstance(o, DTensor) else o
            sens.append(torch.full_like(local, 1.0 / rep))
        return sens

    def backward_one_chunk(self, micro: int, grads: Optional[Sequence[torch.Tensor]], last_micro: bool) -> None:
        args, outputs = self.fwd_cache.pop(micro)
        outs = outputs if isinstance(outputs, (tuple, list)) else (outputs,)
        outs = [o for o in outs if isinstance(o, torch.Tensor)]
        if hasattr(self.submodule, "set_requires_grad_sync"):
            self.submodule.set_requires_grad_sync(bool(last_micro))
        if grads is None:
            grads = self.get_last_stage_sens(outs)
        locals_, seeds = [], []
        for o, g in zip(outs, grads):
            lo = o.to_local() if isinstance(o, DTensor) else o
            if lo.requires_grad:
                locals_.append(lo)
                seeds.append(g.to_local() if isinstance(g, DTensor) else g)
        if locals_:
            torch.autograd.backward(locals_, grad_tensors=seeds)
        if not self.is_first:
            gl = []
            for a in args:
                if isinstance(a, torch.Tensor):
                    la = a.to_local() if isinstance(a, DTensor) else a
                    if la.requires_grad:
                        g = la.grad if la.grad is not None else torch.zeros_like(la)
                        gl.append(DTensor._wrap(g, a.layout) if isinstance(a, DTensor) else g)
                        la.grad = None
            self.input_grads[micro] = gl

    def sync_shared_parameters_grad(self) -> None:
        for info, ranks, grp in self._shared_groups:
            if grp is None:
                continue
            leaf = info.parameter.to_local() if isinstance(info.parameter, DTensor) else info.parameter
            if leaf.grad is None:
                leaf.grad = torch.zeros_like(leaf)
            cc.all_reduce_(leaf.grad, "sum", grp)
