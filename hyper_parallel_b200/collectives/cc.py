"""Process-group helpers and the communication primitives the framework is built on.

Public helpers mirror hyper_parallel/collectives/cc.py:24-106 of the reference
(``init_process_group``, ``destroy_process_group``, ``get_process_group_ranks``,
``get_backend``, ``split_group``).  The backend is whatever ``torch.distributed``
supports on the machine: ``nccl`` when CUDA is available, ``gloo`` otherwise.

Groups are cached by their rank tuple so that a mesh dimension, an HSDP shard
group and a pipeline group over the same ranks share one communicator.  New
groups are created with *local* synchronisation: only member ranks have to make
the call, which is what lets per-pipeline-stage meshes create their own groups.
"""
from __future__ import annotations

import datetime
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

_GROUP_CACHE: Dict[Tuple[int, ...], "dist.ProcessGroup"] = {}


# ------------------------------------------------------------------ basics --
def is_initialized() -> bool:
    return dist.is_available() and dist.is_initialized()


def get_rank() -> int:
    if is_initialized():
        return dist.get_rank()
    return int(os.environ.get("HPB_FAKE_RANK", "0"))


def get_world_size() -> int:
    if is_initialized():
        return dist.get_world_size()
    return int(os.environ.get("HPB_FAKE_WORLD_SIZE", "1"))


def default_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


def init_process_group(backend: Optional[str] = None, *, init_method: Optional[str] = None,
                       timeout: Optional[datetime.timedelta] = None, world_size: int = -1,
                       rank: int = -1, store=None, pg_options=None, device_id=None) -> None:
    """Initialise the default process group (no-op when already initialised)."""
    if is_initialized():
        return
    backend = backend or default_backend()
    kwargs = {}
    if timeout is not None:
        kwargs["timeout"] = timeout
    if pg_options is not None:
        kwargs["pg_options"] = pg_options
    if device_id is not None:
        kwargs["device_id"] = device_id
    if store is not None:
        kwargs["store"] = store
    if init_method is not None:
        kwargs["init_method"] = init_method
    if world_size >= 0:
        kwargs["world_size"] = world_size
    if rank >= 0:
        kwargs["rank"] = rank
    dist.init_process_group(backend, **kwargs)


def destroy_process_group(group=None) -> None:
    if not is_initialized():
        return
    if group is None:
        global _SELF_GROUP
        _GROUP_CACHE.clear()
        _SELF_GROUP = None
        dist.destroy_process_group()
    else:
        for k, v in list(_GROUP_CACHE.items()):
            if v is group:
                del _GROUP_CACHE[k]
        dist.destroy_process_group(group)


def get_process_group_ranks(group=None) -> List[int]:
    if not is_initialized():
        return [0]
    return dist.get_process_group_ranks(group if group is not None else dist.group.WORLD)


def get_backend(group=None) -> str:
    if not is_initialized():
        return "undefined"
    return dist.get_backend(group)


def group_for_ranks(ranks: Sequence[int], timeout=None, pg_options=None, group_desc=None, tag=None):
    """Return (creating once) the process group whose members are ``ranks`` in this order.

    Returns ``None`` when torch.distributed is not initialised or the group has a
    single member (every collective over it is the identity).  ``tag`` asks for a separate
    group (its own communicator and stream) over the same ranks, e.g. one per traffic direction.
    """
    ranks_key = tuple(int(r) for r in ranks)
    key = ranks_key if tag is None else ranks_key + (str(tag),)
    if not is_initialized() or len(ranks_key) <= 1:
        return None
    grp = _GROUP_CACHE.get(key)
    if grp is not None:
        return grp
    if tag is None and ranks_key == tuple(range(dist.get_world_size())):
        grp = dist.group.WORLD
    else:
        if dist.get_rank() not in ranks_key:
            return None
        kwargs = {}
        if timeout is not None:
            kwargs["timeout"] = timeout
        if pg_options is not None:
            kwargs["pg_options"] = pg_options
        if group_desc is not None:
            kwargs["group_desc"] = group_desc
        grp = dist.new_group(list(ranks_key), use_local_synchronization=True, **kwargs)
    _GROUP_CACHE[key] = grp
    return grp


_SELF_GROUP = None


def self_group():
    """A process group whose only member is this rank.  ``None`` means "the world" to
    ``torch.distributed``, so a mesh axis of size one must not hand out ``None`` to callers that pass
    it on to ``dist.*``; this package's own collectives treat the group like ``None`` (size 1 = no-op)."""
    global _SELF_GROUP
    if _SELF_GROUP is None and is_initialized():
        if dist.get_world_size() == 1:
            _SELF_GROUP = dist.group.WORLD
        else:
            _SELF_GROUP = dist.new_group([dist.get_rank()], use_local_synchronization=True)
    return _SELF_GROUP


def world_collective_groups(specs: Sequence[Tuple[Sequence[int], str]]) -> Dict[Tuple[Tuple[int, ...], str], object]:
    """Create (once) one group per ``(ranks, tag)`` of ``specs``; EVERY rank of the world must call
    this with the same list.  Returns the groups this rank is a member of.

    Unlike :func:`group_for_ranks` this does not rely on member-only creation, whose group names
    depend on how many groups each member has created before (torch/distributed/distributed_c10d.py,
    ``_hash_ranks_to_str``) and therefore break when members have different histories -- as the
    two ends of a pipeline do.
    """
    mine: Dict[Tuple[Tuple[int, ...], str], object] = {}
    if not is_initialized():
        return mine
    me = dist.get_rank()
    for ranks, tag in specs:
        rk = tuple(int(r) for r in ranks)
        key = rk + (str(tag),)
        grp = _GROUP_CACHE.get(key)
        if grp is None:
            grp = dist.new_group(list(rk))
            _GROUP_CACHE[key] = grp
        if me in rk:
            mine[(rk, str(tag))] = grp
    return mine


def generate_groups_from_template(template: Sequence[int], world_size: int) -> List[List[int]]:
    """The partition of ``range(world_size)`` into groups shaped like ``template``.

    A mesh axis gives every rank a group that is an arithmetic progression ``base + i * step``
    (``i < n``); all such groups together tile the world: blocks of ``n * step`` consecutive ranks,
    ``step`` interleaved groups per block.  Given one of them the others follow -- what the reference
    uses so that every process can take part in creating every group
    (hyper_parallel/platform/torch/group_utils.py:47-140).  Raises if ``template`` is not an arithmetic
    progression or does not tile ``world_size``."""
    ranks = sorted(int(r) for r in template)
    n = len(ranks)
    if n == 0 or len(set(ranks)) != n:
        raise ValueError(f"template {list(template)} must hold distinct ranks")
    if n == 1:
        return [[r] for r in range(world_size)]
    step = ranks[1] - ranks[0]
    if any(b - a != step for a, b in zip(ranks, ranks[1:])):
        raise ValueError(f"template {ranks} is not an arithmetic progression")
    block = n * step
    if world_size % block or ranks[-1] >= world_size or (ranks[0] % block) >= step:
        raise ValueError(f"template {ranks} does not tile a world of {world_size} ranks")
    return [[start + off + i * step for i in range(n)]
            for start in range(0, world_size, block) for off in range(step)]


def split_group(parent_pg=None, split_ranks: Optional[Sequence[Sequence[int]]] = None, timeout=None,
                pg_options=None, group_desc=None):
    """Create the sub-group of ``split_ranks`` that contains this rank (``None`` if none does).

    ``split_ranks`` are global ranks; they must be members of ``parent_pg`` when one is given.
    """
    if split_ranks is None:
        raise ValueError("split_ranks must be a list of rank lists")
    if not is_initialized():
        return None
    me = dist.get_rank()
    parent = set(get_process_group_ranks(parent_pg)) if parent_pg is not None else None
    mine = None
    for ranks in split_ranks:
        if parent is not None and not set(ranks) <= parent:
            raise ValueError(f"ranks {list(ranks)} are not all members of the parent group")
        if me in ranks:
            mine = ranks
    if mine is None:
        return None
    return group_for_ranks(mine, timeout=timeout, pg_options=pg_options, group_desc=group_desc)


def group_size(group) -> int:
    if group is None or not is_initialized():
        return 1
    return dist.get_world_size(group)


def group_rank(group) -> int:
    if group is None or not is_initialized():
        return 0
    return dist.get_rank(group)


# ------------------------------------------------------ reduce-op handling --
def _reduce_op(op: str):
    table = {
        "sum": dist.ReduceOp.SUM, "avg": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX,
        "min": dist.ReduceOp.MIN, "prod": dist.ReduceOp.PRODUCT, "all": dist.ReduceOp.MIN,
    }
    if op not in table:
        raise ValueError(f"unsupported reduce op {op!r}")
    return table[op]


def all_reduce_(t: torch.Tensor, op: str, group, async_op: bool = False):
    """In-place all-reduce.  ``avg`` = sum / n, ``all`` = logical-and via integer MIN."""
    n = group_size(group)
    if n == 1:
        return None
    if op == "all" or t.dtype == torch.bool:
        # logical reductions go through integers: all = MIN, any = MAX over {0, 1}
        buf = t.to(torch.int32)
        dist.all_reduce(buf, _reduce_op(op), group=group)
        t.copy_(buf.to(t.dtype))
        return None
    work = dist.all_reduce(t, _reduce_op(op), group=group, async_op=async_op)
    if op == "avg":
        if async_op:
            return _ScaledWork(work, t, 1.0 / n)
        t.div_(n)
    return work


class _ScaledWork:
    """Async handle that applies a scale once the collective has completed."""

    def __init__(self, work, tensor, scale):
        self.work, self.tensor, self.scale = work, tensor, scale

    def wait(self):
        if self.work is not None:
            self.work.wait()
        self.tensor.mul_(self.scale)
        return True


def all_gather_into(out: torch.Tensor, inp: torch.Tensor, group, async_op: bool = False):
    """Gather ``inp`` from every member into ``out`` (concatenated along dim 0)."""
    if group_size(group) == 1:
        out.copy_(inp.reshape(out.shape))
        return None
    return dist.all_gather_into_tensor(out, inp.contiguous(), group=group, async_op=async_op)


def reduce_scatter_into(out: torch.Tensor, inp: torch.Tensor, group, op: str = "sum",
                        async_op: bool = False):
    """Sum-reduce ``inp`` (``n`` equal chunks along dim 0) and keep chunk ``rank`` in ``out``."""
    n = group_size(group)
    if n == 1:
        out.copy_(inp.reshape(out.shape))
        return None
    if dist.get_backend(group) == "gloo":
        # gloo has no reduce_scatter: all-reduce then slice (CPU test path only)
        tmp = inp.contiguous().clone()
        dist.all_reduce(tmp, _reduce_op(op), group=group)
        r = dist.get_rank(group)
        out.copy_(tmp.reshape(n, -1)[r].reshape(out.shape))
        if op == "avg":
            out.div_(n)
        return None
    work = dist.reduce_scatter_tensor(out, inp.contiguous(), _reduce_op(op), group=group,
                                      async_op=async_op)
    if op == "avg":
        if async_op:
            return _ScaledWork(work, out, 1.0 / n)
        out.div_(n)
    return work


def broadcast(t: torch.Tensor, src: int, group=None, async_op: bool = False):
    if group_size(group) == 1 and group is not None:
        return None
    if not is_initialized():
        return None
    return dist.broadcast(t, src=src, group=group, async_op=async_op)


def all_gather_object(obj, group=None) -> list:
    if not is_initialized() or (group is not None and group_size(group) == 1):
        return [obj]
    out = [None] * dist.get_world_size(group)
    dist.all_gather_object(out, obj, group=group)
    return out


# ---------------------------------------------- differentiable collectives --
class _AllGatherConcat(torch.autograd.Function):
    """Concatenate every member's shard along ``dim``; backward reduce-scatters the gradient."""

    @staticmethod
    def forward(ctx, x, dim, group):
        ctx.dim, ctx.group = dim, group
        n = group_size(group)
        xc = x.contiguous()
        out = torch.empty((n,) + tuple(xc.shape), dtype=x.dtype, device=x.device)
        all_gather_into(out.view(n * xc.shape[0], *xc.shape[1:]) if xc.dim() > 0 else out, xc, group)
        # out[r] is rank r's shard: move the rank axis next to `dim` and merge
        if xc.dim() == 0:
            return out
        out = out.movedim(0, dim)  # [..., n, local_dim, ...]
        shape = list(xc.shape)
        shape[dim] *= n
        return out.reshape(shape)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_along(g, ctx.dim, ctx.group), None, None


def _reduce_scatter_along(t: torch.Tensor, dim: int, group, op: str = "sum") -> torch.Tensor:
    n = group_size(group)
    if n == 1:
        return t
    shape = list(t.shape)
    local = shape[dim] // n
    # bring the chunk axis to the front so chunks are contiguous
    chunks = t.reshape(shape[:dim] + [n, local] + shape[dim + 1:]).movedim(dim, 0).contiguous()
    out = torch.empty(chunks.shape[1:], dtype=t.dtype, device=t.device)
    reduce_scatter_into(out, chunks, group, op)
    return out


class _ReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, group, op):
        ctx.dim, ctx.group, ctx.op = dim, group, op
        return _reduce_scatter_along(x, dim, group, op)

    @staticmethod
    def backward(ctx, g):
        out = _AllGatherConcat.apply(g, ctx.dim, ctx.group)
        if ctx.op == "avg":
            out = out / group_size(ctx.group)
        return out, None, None, None


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, group):
        ctx.op, ctx.group = op, group
        out = x.contiguous().clone()
        all_reduce_(out, op, group)
        if op in ("max", "min"):
            ctx.save_for_backward(x, out)
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        all_reduce_(g, "sum", ctx.group)
        if ctx.op == "avg":
            g = g / group_size(ctx.group)
        elif ctx.op in ("max", "min"):
            x, out = ctx.saved_tensors
            g = g * (x == out).to(g.dtype)
        elif ctx.op in ("prod", "all"):
            raise RuntimeError(f"all_reduce({ctx.op}) is not differentiable")
        return g, None, None


class _AllToAll(torch.autograd.Function):
    """Re-shard: split ``x`` along ``split_dim`` into n chunks, exchange, concat along ``concat_dim``."""

    @staticmethod
    def forward(ctx, x, split_dim, concat_dim, group):
        ctx.split_dim, ctx.concat_dim, ctx.group = split_dim, concat_dim, group
        return _all_to_all(x, split_dim, concat_dim, group)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all(g, ctx.concat_dim, ctx.split_dim, ctx.group), None, None, None


def _all_to_all(x: torch.Tensor, split_dim: int, concat_dim: int, group) -> torch.Tensor:
    n = group_size(group)
    if n == 1:
        return x
    shape = list(x.shape)
    local = shape[split_dim] // n
    send = x.reshape(shape[:split_dim] + [n, local] + shape[split_dim + 1:]).movedim(split_dim, 0).contiguous()
    recv = torch.empty_like(send)
    if dist.get_backend(group) == "gloo":
        # gloo has no all-to-all: exchange the chunks with point-to-point messages
        me = dist.get_rank(group)
        ranks = dist.get_process_group_ranks(group)
        reqs = []
        for r in range(n):
            if r == me:
                recv[r].copy_(send[r])
            else:
                reqs.append(dist.isend(send[r].contiguous(), dst=ranks[r], group=group))
                reqs.append(dist.irecv(recv[r], src=ranks[r], group=group))
        for q in reqs:
            q.wait()
    else:
        dist.all_to_all_single(recv, send, group=group)
    # recv[r] = chunk that rank r held for me, shaped like x with split_dim -> local
    recv = recv.movedim(0, concat_dim)  # [..., n, cdim, ...]
    s2 = list(recv.shape)
    merged = s2[:concat_dim] + [s2[concat_dim] * s2[concat_dim + 1]] + s2[concat_dim + 2:]
    return recv.reshape(merged)


def all_gather_concat(x: torch.Tensor, dim: int, group) -> torch.Tensor:
    """Differentiable all-gather + concatenate along ``dim``."""
    if group_size(group) == 1:
        return x
    return _AllGatherConcat.apply(x, dim, group)


def reduce_scatter(x: torch.Tensor, dim: int, group, op: str = "sum") -> torch.Tensor:
    """Differentiable reduce-scatter along ``dim``."""
    if group_size(group) == 1:
        return x
    return _ReduceScatter.apply(x, dim, group, op)


def all_reduce(x: torch.Tensor, op: str, group) -> torch.Tensor:
    """Differentiable (out-of-place) all-reduce."""
    if group_size(group) == 1:
        return x
    return _AllReduce.apply(x, op, group)


def all_to_all(x: torch.Tensor, split_dim: int, concat_dim: int, group) -> torch.Tensor:
    """Differentiable all-to-all that moves the sharding from ``concat_dim`` to ``split_dim``."""
    if group_size(group) == 1:
        return x
    return _AllToAll.apply(x, split_dim, concat_dim, group)
