"""File-system storage with the reference's on-disk layout
(hyper_parallel/core/checkpoint/filesystem_storage.py:42-501).

Files inside ``checkpoint_id/``:

* ``_rank{r}_.safetensors`` -- ``torch.save`` of ``{fqn: local tensor}`` written by rank ``r`` (the
  reference's torch build uses ``torch.save`` under this name as well);
* ``{fqn}_rank{r}.bytes``    -- one pickled non-tensor entry;
* ``.metadata``              -- pickled :class:`Metadata`, written by rank 0; or
  ``.rank{r}_metadata`` per rank when collectives are disabled.

Additions: every file is written to a temporary name, flushed, fsync'ed and renamed, so a
crash never leaves a half-written checkpoint that looks valid.
"""
from __future__ import annotations

import os
import pickle
from typing import Dict, List, Optional

import torch

from .metadata import Metadata, MetadataIndex
from .planner import LoadPlan, LoadPlanner, SavePlan, SavePlanner, WriteItemType
from .storage import StorageInfo, StorageReader, StorageWriter, WriteResult, _metadata_file_name
from ._compat import ReferenceCompatUnpickler, reference_module_names


def _atomic_write(path: str, writer) -> None:
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        writer(f)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


def _safe_name(fqn: str) -> str:
    return fqn.replace(os.sep, "_")


class FileSystemWriter(StorageWriter):
    def __init__(self, path: Optional[str] = None):
        self.path = path
        self.rank = 0
        self.is_coordinator = True
        self.use_collectives = True

    def initialize_writer(self, checkpoint_id) -> None:
        if checkpoint_id is not None:
            self.path = str(checkpoint_id)
        if self.path is None:
            raise ValueError("checkpoint_id (a directory) is required")
        os.makedirs(self.path, exist_ok=True)

    def configure_writer(self, is_coordinator: bool, rank: int, use_collectives: bool = True) -> None:
        self.is_coordinator, self.rank, self.use_collectives = is_coordinator, rank, use_collectives

    def optimize_local_plan(self, plan: SavePlan) -> SavePlan:
        return plan

    def optimize_global_plan(self, plans: List[SavePlan]) -> List[SavePlan]:
        return plans

    def execute_write(self, plan: SavePlan, planner: SavePlanner) -> List[WriteResult]:
        results: List[WriteResult] = []
        tensors: Dict[str, torch.Tensor] = {}
        tfile = f"_rank{self.rank}_.safetensors"
        for it in plan.items:
            attached = getattr(it, "bytes_io_data", None) if it.type == WriteItemType.BYTE_IO else None
            if attached is not None:
                data = attached if isinstance(attached, bytes) else pickle.dumps(attached)
            else:
                data = planner.resolve_data(it)
            if it.type == WriteItemType.BYTE_IO:
                rel = f"{_safe_name(it.index.fqn)}_rank{self.rank}.bytes"
                _atomic_write(os.path.join(self.path, rel), lambda f, d=data: f.write(d))
                results.append(WriteResult(it.index, len(data), StorageInfo(rel, 0, len(data))))
            else:
                t = data.cpu() if data.device.type != "cpu" else data
                tensors[it.index.fqn] = t.contiguous()
                results.append(WriteResult(it.index, t.numel() * t.element_size(), StorageInfo(tfile, 0, -1)))
        if tensors:
            _atomic_write(os.path.join(self.path, tfile), lambda f: torch.save(tensors, f))
        return results

    def finalize_checkpoint(self, metadata: Metadata, results: List[List[WriteResult]]) -> None:
        storage = {}
        for per_rank in results:
            for wr in per_rank:
                storage[wr.index] = wr.storage_data
        metadata.storage_data = storage
        name = _metadata_file_name if self.use_collectives else f".rank{self.rank}_metadata"
        if self.use_collectives and not self.is_coordinator:
            return
        with reference_module_names():
            blob = pickle.dumps(metadata)
        _atomic_write(os.path.join(self.path, name), lambda f: f.write(blob))


class FileSystemReader(StorageReader):
    def __init__(self, path: Optional[str] = None):
        self.path = path
        self.metadata: Optional[Metadata] = None

    def initialize_reader(self, checkpoint_id) -> None:
        if checkpoint_id is not None:
            self.path = str(checkpoint_id)
        if self.path is None or not os.path.isdir(self.path):
            raise FileNotFoundError(f"checkpoint directory {self.path!r} does not exist")

    def load_metadata(self, rank: Optional[int] = None) -> Metadata:
        cand = [os.path.join(self.path, _metadata_file_name)]
        if rank is not None:
            cand.append(os.path.join(self.path, f".rank{rank}_metadata"))
        for p in cand:
            if os.path.exists(p):
                with open(p, "rb") as f:
                    md = ReferenceCompatUnpickler(f).load()
                if not isinstance(md, Metadata):
                    raise ValueError(f"{p} does not contain checkpoint metadata")
                return md
        merged = self._merge_rank_metadata()
        if merged is not None:
            return merged
        raise FileNotFoundError(f"no metadata file in {self.path} (looked for {[os.path.basename(c) for c in cand]})")

    def _merge_rank_metadata(self) -> Optional[Metadata]:
        """Union of all ``.rank{r}_metadata`` files: a checkpoint written rank by rank (without
        collectives) then loads on any number of ranks and layout, like a coordinated one."""
        import dataclasses
        import re
        files = sorted(f for f in os.listdir(self.path) if re.fullmatch(r"\.rank\d+_metadata", f))
        if not files:
            return None
        state: Dict[str, object] = {}
        storage: Dict[MetadataIndex, object] = {}
        for fn in files:
            with open(os.path.join(self.path, fn), "rb") as f:
                md = ReferenceCompatUnpickler(f).load()
            for fqn, entry in md.state_dict_metadata.items():
                have = state.get(fqn)
                if have is None or not hasattr(entry, "chunks"):
                    state[fqn] = entry
                else:
                    chunks = list(have.chunks) + [c for c in entry.chunks if c not in have.chunks]
                    state[fqn] = dataclasses.replace(have, chunks=chunks)
            for idx, info in (md.storage_data or {}).items():
                storage.setdefault(idx, info)
        # chunk indices are positions in the merged chunk lists
        fixed: Dict[MetadataIndex, object] = {}
        for idx, info in storage.items():
            entry = state.get(idx.fqn)
            if hasattr(entry, "chunks") and idx.offset is not None:
                pos = next((i for i, c in enumerate(entry.chunks) if tuple(c.offsets) == tuple(idx.offset)), idx.index)
                fixed[MetadataIndex(idx.fqn, idx.offset, pos)] = info
            else:
                fixed[idx] = info
        return Metadata(state_dict_metadata=state, storage_data=fixed)

    def configure_reader(self, metadata: Metadata, is_coordinator: bool, rank: int = 0) -> None:
        self.metadata = metadata

    def optimize_local_plan(self, plan: LoadPlan) -> LoadPlan:
        return plan

    def optimize_global_plan(self, plans):
        return plans

    def execute_read(self, plan: LoadPlan, planner: LoadPlanner) -> None:
        storage = self.metadata.storage_data or {}
        by_file: Dict[str, list] = {}
        for it in plan.items:
            info = storage.get(it.storage_index)
            if info is None:
                # metadata written without chunk index (older layout): match on fqn + offset
                info = next((v for k, v in storage.items()
                             if k.fqn == it.storage_index.fqn and tuple(k.offset) == tuple(it.storage_index.offset)), None)
            if info is None:
                raise KeyError(f"no storage record for {it.storage_index}")
            by_file.setdefault(info.relative_path, []).append(it)
        for rel, items in by_file.items():
            full = os.path.join(self.path, rel)
            if not os.path.exists(full):
                raise FileNotFoundError(f"checkpoint file {full} is missing")
            if rel.endswith(".bytes"):
                with open(full, "rb") as f:
                    blob = f.read()
                for it in items:
                    planner.load_bytes(it, blob)
                continue
            tensors = torch.load(full, map_location="cpu", weights_only=True)
            for it in items:
                src = tensors[it.storage_index.fqn]
                for d, (o, n) in enumerate(zip(it.storage_offsets, it.lengths)):
                    src = src.narrow(d, o, n)
                dst = planner.resolve_tensor(it)
                dst.copy_(src)
                planner.commit_tensor(it, dst)
