"""Default planners (capability of hyper_parallel/core/checkpoint/standard_planner.py:42-548).

Save: a DTensor contributes one chunk at the offsets of this rank's slice; a plain tensor one
full chunk; anything else is pickled bytes.  Replicated chunks are written by one rank only
(the least loaded, or the minimum rank).  Load: for every destination tensor the planner
intersects its own chunk with every saved chunk and emits one ``ReadItem`` per overlap, which
is what makes *resharding on load* (save on 8 ranks, load on 4) work.
"""
from __future__ import annotations

import io
import pickle
from typing import Any, Dict, List

import torch

from ..dtensor import DTensor
from .metadata import (BytesStorageMetadata, ChunkStorageMetadata, Metadata, MetadataIndex,
                       TensorProperties, TensorStorageMetadata)
from .planner import (LoadItemType, LoadPlan, LoadPlanner, ReadItem, SavePlan, SavePlanner,
                      TensorWriteData, WriteItem, WriteItemType)
from .util import dedup_plans, dtype_to_str, local_chunk_of


def flatten_state_dict(state_dict: Dict[str, Any], prefix: str = "") -> Dict[str, Any]:
    flat: Dict[str, Any] = {}
    for k, v in state_dict.items():
        key = f"{prefix}{k}"
        if isinstance(v, dict):
            flat.update(flatten_state_dict(v, key + "."))
        else:
            flat[key] = v
    return flat


class StandardSavePlanner(SavePlanner):
    def __init__(self, remove_redundancy: bool = True, save_to_minimum_rank: bool = False):
        self.remove_redundancy = remove_redundancy
        self.save_to_minimum_rank = save_to_minimum_rank
        self.state_dict: Dict[str, Any] = {}
        self.is_coordinator = False
        self.rank = 0

    def set_up_planner(self, state_dict, is_coordinator=False, rank: int = 0, **kw):
        self.state_dict = flatten_state_dict(state_dict)
        self.is_coordinator = is_coordinator
        self.rank = rank

    def create_local_plan(self) -> SavePlan:
        items: List[WriteItem] = []
        for fqn, v in self.state_dict.items():
            if isinstance(v, torch.Tensor):
                local, gshape, offsets, sizes = local_chunk_of(v)
                props = TensorProperties(dtype_to_str(local.dtype), bool(getattr(v, "requires_grad", False)))
                items.append(WriteItem(MetadataIndex(fqn, offsets), WriteItemType.TENSOR,
                                       TensorWriteData(ChunkStorageMetadata(offsets, sizes), props, gshape)))
            else:
                items.append(WriteItem(MetadataIndex(fqn), WriteItemType.BYTE_IO))
        return SavePlan(items=items, rank=self.rank)

    def create_global_plan(self, all_plans: List[SavePlan]):
        plans = dedup_plans(all_plans, self.save_to_minimum_rank) if self.remove_redundancy else \
            [SavePlan(items=list(p.items), rank=r) for r, p in enumerate(all_plans)]
        md: Dict[str, Any] = {}
        new_plans = []
        for r, plan in enumerate(plans):
            new_items = []
            for it in plan.items:
                if it.type == WriteItemType.BYTE_IO:
                    md.setdefault(it.index.fqn, BytesStorageMetadata())
                    # keyed without a chunk index, as the reference's reader looks it up
                    new_items.append(WriteItem(MetadataIndex(it.index.fqn, (), None), it.type))
                    continue
                td = it.tensor_data
                entry = md.get(it.index.fqn)
                if entry is None:
                    entry = TensorStorageMetadata(td.properties, td.size, [])
                    md[it.index.fqn] = entry
                elif tuple(entry.size) != tuple(td.size):
                    raise ValueError(f"{it.index.fqn}: ranks disagree on the global shape "
                                     f"({entry.size} vs {td.size})")
                if td.chunk in entry.chunks:       # identical replica kept by several ranks (no dedup)
                    idx = entry.chunks.index(td.chunk)
                else:
                    entry.chunks.append(td.chunk)
                    idx = len(entry.chunks) - 1
                new_items.append(WriteItem(MetadataIndex(it.index.fqn, td.chunk.offsets, idx), it.type, td))
            new_plans.append(SavePlan(items=new_items, rank=r))
        return new_plans, Metadata(state_dict_metadata=md)

    def finish_plan(self, new_plan: SavePlan) -> SavePlan:
        self.plan = new_plan
        return new_plan

    def resolve_data(self, write_item: WriteItem):
        v = self.state_dict[write_item.index.fqn]
        if write_item.type == WriteItemType.BYTE_IO:
            buf = io.BytesIO()
            pickle.dump(v, buf)
            return buf.getvalue()
        local = v.to_local() if isinstance(v, DTensor) else v
        return local.detach()


def _intersect(off_a, size_a, off_b, size_b):
    lo, ln = [], []
    for oa, sa, ob, sb in zip(off_a, size_a, off_b, size_b):
        s, e = max(oa, ob), min(oa + sa, ob + sb)
        if e <= s:
            return None
        lo.append(s)
        ln.append(e - s)
    return tuple(lo), tuple(ln)


class StandardLoadPlanner(LoadPlanner):
    def __init__(self, allow_partial_load: bool = False):
        self.allow_partial_load = allow_partial_load

    def set_up_planner(self, state_dict, metadata=None, is_coordinator=False, **kw):
        self.original = state_dict
        self.state_dict = flatten_state_dict(state_dict)
        self.metadata = metadata
        self.loaded_bytes: Dict[str, Any] = {}

    def create_local_plan(self) -> LoadPlan:
        items: List[ReadItem] = []
        md = self.metadata.state_dict_metadata
        for fqn, v in self.state_dict.items():
            if fqn not in md:
                if self.allow_partial_load:
                    continue
                raise KeyError(f"{fqn} is missing from the checkpoint (allow_partial_load=False)")
            entry = md[fqn]
            if isinstance(entry, BytesStorageMetadata):
                idx = next((k for k in (self.metadata.storage_data or {}) if k.fqn == fqn), MetadataIndex(fqn))
                items.append(ReadItem(LoadItemType.BYTE_IO, MetadataIndex(fqn), (), idx, (), ()))
                continue
            if not isinstance(v, torch.Tensor):
                raise TypeError(f"{fqn}: checkpoint holds a tensor but the state_dict entry is {type(v)}")
            _, gshape, d_off, d_size = local_chunk_of(v)
            if tuple(gshape) != tuple(entry.size):
                raise ValueError(f"{fqn}: global shape {tuple(gshape)} differs from the saved {tuple(entry.size)}")
            covered = 0
            for ci, chunk in enumerate(entry.chunks):
                hit = _intersect(d_off, d_size, chunk.offsets, chunk.sizes)
                if hit is None:
                    continue
                lo, ln = hit
                items.append(ReadItem(
                    LoadItemType.TENSOR, MetadataIndex(fqn, d_off),
                    tuple(a - b for a, b in zip(lo, d_off)),
                    MetadataIndex(fqn, chunk.offsets, ci),
                    tuple(a - b for a, b in zip(lo, chunk.offsets)), ln))
                n = 1
                for x in ln:
                    n *= x
                covered += n
            need = 1
            for x in d_size:
                need *= x
            if covered < need:
                raise ValueError(f"{fqn}: saved chunks cover only {covered} of {need} requested elements")
        return LoadPlan(items=items)

    def create_global_plan(self, all_plans):
        return all_plans

    def finish_plan(self, new_plan):
        return new_plan

    def load_bytes(self, read_item: ReadItem, value: bytes) -> None:
        obj = pickle.loads(value)
        self.loaded_bytes[read_item.dest_index.fqn] = obj
        self._assign(self.original, read_item.dest_index.fqn, obj)

    @staticmethod
    def _assign(tree, fqn, obj):
        if fqn in tree:
            tree[fqn] = obj
            return True
        for k, v in tree.items():
            if isinstance(v, dict) and fqn.startswith(k + "."):
                if StandardLoadPlanner._assign(v, fqn[len(k) + 1:], obj):
                    return True
        return False

    def resolve_tensor(self, read_item: ReadItem):
        v = self.state_dict[read_item.dest_index.fqn]
        local = v.to_local() if isinstance(v, DTensor) else v
        view = local.detach()
        for d, (o, n) in enumerate(zip(read_item.dest_offsets, read_item.lengths)):
            view = view.narrow(d, o, n)
        return view

    def commit_tensor(self, read_item, tensor) -> None:
        pass


def create_read_items_for_chunk_list(fqn: str, checkpoint_md, local_chunks) -> List[ReadItem]:
    """Read items that fill ``local_chunks`` (what this rank needs) from the saved chunks of
    ``checkpoint_md``: one item per overlap, with offsets inside the destination chunk and inside the
    saved chunk (reference standard_planner.py:324-370)."""
    items: List[ReadItem] = []
    for li, lc in enumerate(local_chunks or ()):
        for si, sc in enumerate(checkpoint_md.chunks or ()):
            hit = _intersect(tuple(lc.offsets), tuple(lc.sizes), tuple(sc.offsets), tuple(sc.sizes))
            if hit is None:
                continue
            lo, ln = hit
            items.append(ReadItem(LoadItemType.TENSOR, MetadataIndex(fqn, tuple(lc.offsets), li),
                                  tuple(a - b for a, b in zip(lo, lc.offsets)),
                                  MetadataIndex(fqn, tuple(sc.offsets), si),
                                  tuple(a - b for a, b in zip(lo, sc.offsets)), tuple(ln)))
    return items
