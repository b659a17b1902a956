"""Small helpers of the checkpoint package (hyper_parallel/core/checkpoint/util.py)."""
from __future__ import annotations

import os
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..dtensor import DTensor

_DTYPE_NAMES = {str(d): d for d in (torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int8,
                                    torch.uint8, torch.int16, torch.int32, torch.int64, torch.bool,
                                    torch.float8_e4m3fn, torch.float8_e5m2)}


def dtype_to_str(dtype: torch.dtype) -> str:
    return str(dtype)


def str_to_dtype(name: str) -> torch.dtype:
    if name not in _DTYPE_NAMES:
        raise ValueError(f"unknown dtype string {name!r}")
    return _DTYPE_NAMES[name]


def has_valid_filename(path) -> bool:
    """The reference's rule (core/checkpoint/util.py:49-70 there): a file name with a stem and a suffix,
    each containing at least one letter."""
    p = Path(path)
    return bool(p.name and p.stem and len(p.suffix) > 1 and any(c.isalpha() for c in p.stem)
                and any(c.isalpha() for c in p.suffix[1:]))


def check_file_name(path, suffixes: Optional[Sequence[str]] = None) -> str:
    """Validate a single-file checkpoint path (a ``str`` or ``Path``) and return it as an absolute string;
    the parent directory is created when missing.  ``suffixes`` restricts the extension when given."""
    if isinstance(path, Path):
        path = str(path)
    if not isinstance(path, str) or not path:
        raise ValueError("checkpoint file path must be a non-empty string or Path")
    if "\x00" in path:
        raise ValueError("checkpoint file path contains a NUL byte")
    if not has_valid_filename(path):
        raise ValueError(f"Saver file_path should contains valid filename but get: {path}")
    if suffixes is not None and not path.endswith(tuple(suffixes)):
        raise ValueError(f"checkpoint file must end with one of {tuple(suffixes)}, got {path!r}")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    return os.path.abspath(path)


def local_chunk_of(value) -> Tuple[torch.Tensor, Tuple[int, ...], Tuple[int, ...], Tuple[int, ...]]:
    """``(local tensor, global shape, chunk offsets, chunk sizes)`` of a state-dict tensor.

    Handles DTensors (offsets from the layout's slice area) and HSDP-sharded parameters (an
    additional dim-0 chunk of the TP-local tensor).
    """
    hp = getattr(value, "_hsdp_param", None)
    if isinstance(value, DTensor):
        local = value.to_local()
        lay = value.layout
        tp_local_shape = hp.full_shape if (hp is not None and hp.sharded and hp.is_sharded_now) else tuple(local.shape)
        gshape = tuple(lay.get_global_shape(tp_local_shape))
        area = lay.slice_area(gshape)
        offsets = [b for b, _ in area]
        sizes = [e - b for b, e in area]
    else:
        local = value
        if hp is not None and hp.sharded and hp.is_sharded_now:
            gshape = tuple(hp.full_shape)
        else:
            gshape = tuple(local.shape)
        offsets = [0] * len(gshape)
        sizes = list(gshape)
    if hp is not None and hp.sharded and hp.is_sharded_now:
        step = sizes[0] // hp.shard_size
        offsets[0] += hp.sharded_group_info.index * step
        sizes[0] = step
    return local, gshape, tuple(offsets), tuple(sizes)


def dedup_plans(plans, save_to_minimum_rank: bool = False):
    """Keep each (fqn, offsets) chunk on exactly one rank: the minimum rank, or the least loaded one."""
    owners: Dict[tuple, List[int]] = {}
    for r, plan in enumerate(plans):
        for it in plan.items:
            key = (it.index.fqn, it.index.offset)
            owners.setdefault(key, []).append(r)
    load = [0] * len(plans)
    keep: Dict[tuple, int] = {}
    for key in sorted(owners, key=lambda k: (len(owners[k]), k[0], k[1])):
        ranks = owners[key]
        r = min(ranks) if save_to_minimum_rank else min(ranks, key=lambda x: (load[x], x))
        keep[key] = r
        load[r] += 1
    out = []
    for r, plan in enumerate(plans):
        items = [it for it in plan.items if keep[(it.index.fqn, it.index.offset)] == r]
        out.append(type(plan)(items=items, storage_data=plan.storage_data, planner_data=plan.planner_data, rank=r))
    return out


# ---- helpers for planners written against the reference (its core/checkpoint/util.py:31-235) ----------
def check_path(path) -> None:
    """Create the folder ``path`` names -- its parent when ``path`` has a suffix -- unless it exists."""
    p = Path(path)
    if p.exists():
        return
    (p.parent if p.suffix else p).mkdir(parents=True, exist_ok=True)


def narrow_tensor_by_index(tensor, offsets: tuple, lengths: tuple):
    """``tensor[off : off + len]`` per dimension (the whole tensor when either tuple is empty)."""
    if not offsets or not lengths:
        return tensor
    return tensor[tuple(slice(int(o), int(o) + int(n)) for o, n in zip(offsets, lengths))]


def chunk_to_area(chunk) -> Tuple[Tuple[int, int], ...]:
    """``((start, end), ...)`` of a ``ChunkStorageMetadata``."""
    return tuple((int(o), int(o) + int(n)) for o, n in zip(chunk.offsets, chunk.sizes))


def create_chunk_list_for_tensor(obj) -> list:
    """The chunks of the global tensor that this rank holds: one for a DTensor (its slice area), the
    whole tensor for a plain one."""
    from .metadata import ChunkStorageMetadata
    _, _, offsets, sizes = local_chunk_of(obj)
    return [ChunkStorageMetadata(offsets=tuple(offsets), sizes=tuple(sizes))]


def remove_redundant_plans(all_plans, save_to_minimum_rank: bool = False):
    """Keep every duplicated entry in one plan only (the least loaded plan, or the minimum rank)."""
    return dedup_plans(all_plans, save_to_minimum_rank)
