"""Layout-to-layout redistribution of a DTensor.

Capability of hyper_parallel/core/tensor_redistribution.py:32-324 and
hyper_parallel/core/redistribute_infer.py:196-653 of the reference, with the
Partial -> Shard path implemented as a real reduce-scatter (for any tensor dim).

Planning works on ``dim_axes`` (per tensor dim, the mesh axes sharding it, outer
first) and emits a minimal list of steps:

* ``("all_reduce", axis, op)``            pending reduction, result replicated on ``axis``
* ``("reduce_scatter", axis, dim, op)``   pending reduction whose result is sharded on ``dim``
* ``("all_gather", axis, dim)``           drop the innermost shard axis of ``dim``
* ``("all_to_all", axis, src_dim, dst_dim)`` move a shard axis between tensor dims
* ``("split", axis, dim)``                local chunk, no communication

Reduce-scatters are ordered before all-reduces, and lower mesh axes first.  Plans
are cached per (source layout, target layout); every step is differentiable.
"""
from __future__ import annotations

from typing import Dict, List, Tuple


from ..collectives import cc
from .layout import Layout

Step = tuple


class MeshMismatchError(RuntimeError, ValueError):
    """Redistribution between two different device meshes.  The reference raises ``RuntimeError``
    here (tests/torch/shard/redistribute.py:84-115); earlier callers of this package caught
    ``ValueError``: the class is both."""


def plan_redistribution(src: Layout, dst: Layout) -> List[Step]:
    """Pure planning: the list of steps that turns ``src`` into ``dst`` (same mesh)."""
    if src.mesh != dst.mesh:
        raise MeshMismatchError("redistribute between different device meshes is not supported: "
                                f"{src.mesh} vs {dst.mesh}")
    if len(src.dim_axes) != len(dst.dim_axes):
        raise ValueError("source and target layouts describe tensors of different rank")
    cur = [list(a) for a in src.dim_axes]
    tgt = [list(a) for a in dst.dim_axes]
    steps: List[Step] = []

    # 1. pending reductions ------------------------------------------------
    rs, ar = [], []
    for axis, op in enumerate(src.partial):
        if op is None:
            continue
        if dst.partial[axis] is not None:
            if dst.partial[axis] != op:
                raise ValueError(f"cannot change partial op {op} -> {dst.partial[axis]} on mesh axis {axis}")
            continue  # stays partial
        target_dim = next((d for d, axes in enumerate(tgt) if axis in axes), None)
        if (target_dim is not None and op in ("sum", "avg")
                and tgt[target_dim][:len(cur[target_dim]) + 1] == cur[target_dim] + [axis]):
            rs.append((axis, target_dim, op))
        else:
            ar.append((axis, op))
    for axis, d, op in sorted(rs, key=lambda t: (tgt[t[1]].index(t[0]), t[0])):
        # re-check appendability (an earlier reduce-scatter may have extended the same dim)
        if tgt[d][:len(cur[d]) + 1] == cur[d] + [axis]:
            steps.append(("reduce_scatter", axis, d, op))
            cur[d].append(axis)
        else:
            ar.append((axis, op))
    for axis, op in sorted(ar):
        steps.append(("all_reduce", axis, op))
    for axis, op in enumerate(dst.partial):
        if op is not None and src.partial[axis] is None:
            raise ValueError("redistribute cannot create a Partial placement from a non-partial one")

    # 2. sharding ------------------------------------------------------------
    def common_prefix(a, b):
        n = 0
        while n < len(a) and n < len(b) and a[n] == b[n]:
            n += 1
        return n

    guard = 0
    while cur != tgt:
        guard += 1
        if guard > 64:
            raise RuntimeError(f"redistribution planning did not converge: {src} -> {dst}")
        progressed = False
        # all-to-all: innermost surplus axis of dim i is the next missing axis of dim j
        for i in range(len(cur)):
            if len(cur[i]) > common_prefix(cur[i], tgt[i]):
                a = cur[i][-1]
                for j in range(len(cur)):
                    if j != i and len(cur[j]) < len(tgt[j]) and cur[j] == tgt[j][:len(cur[j])] \
                            and tgt[j][len(cur[j])] == a:
                        steps.append(("all_to_all", a, i, j))
                        cur[i].pop()
                        cur[j].append(a)
                        progressed = True
                        break
            if progressed:
                break
        if progressed:
            continue
        # all-gather: drop an innermost surplus axis
        for i in range(len(cur)):
            if len(cur[i]) > common_prefix(cur[i], tgt[i]):
                a = cur[i].pop()
                steps.append(("all_gather", a, i))
                progressed = True
                break
        if progressed:
            continue
        # split: add the next missing axis
        for j in range(len(cur)):
            if len(cur[j]) < len(tgt[j]) and cur[j] == tgt[j][:len(cur[j])]:
                a = tgt[j][len(cur[j])]
                if any(a in c for c in cur):
                    continue
                steps.append(("split", a, j))
                cur[j].append(a)
                progressed = True
                break
        if not progressed:
            raise RuntimeError(f"cannot plan redistribution {src} -> {dst}")
    return steps


class TensorRedistribution:
    """Executes (and caches) redistribution plans."""

    def __init__(self):
        self._plans: Dict[Tuple[str, str], List[Step]] = {}

    def plan(self, src: Layout, dst: Layout) -> List[Step]:
        key = (src.compact_str, dst.compact_str)
        p = self._plans.get(key)
        if p is None:
            p = plan_redistribution(src, dst)
            self._plans[key] = p
        return p

    def redistribution(self, dtensor, dst: Layout):
        from .dtensor import DTensor
        src = dtensor.layout
        if src == dst:
            return dtensor
        steps = self.plan(src, dst)
        mesh = src.mesh
        x = dtensor.to_local()
        for st in steps:
            kind, axis = st[0], st[1]
            group = mesh.get_group(axis)
            if kind == "all_reduce":
                x = cc.all_reduce(x, st[2], group)
            elif kind == "reduce_scatter":
                x = cc.reduce_scatter(x, st[2], group, st[3])
            elif kind == "all_gather":
                x = cc.all_gather_concat(x, st[2], group)
            elif kind == "all_to_all":
                x = cc.all_to_all(x, st[3], st[2], group)
            elif kind == "split":
                n = mesh.mesh_shape[axis]
                x = x.chunk(n, dim=st[2])[mesh.get_local_rank(axis)]
            else:  # pragma: no cover
                raise RuntimeError(f"unknown redistribution step {st}")
        return DTensor._wrap(x, dst)

    def reduce_partial(self, dtensor, to_layout: Layout):
        return self.redistribution(dtensor, to_layout)


_tensor_redistribution = TensorRedistribution()
