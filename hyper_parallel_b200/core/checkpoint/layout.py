"""Layout json I/O (hyper_parallel/core/checkpoint/layout.py:26-131): per-rank ``*.layout`` files.

Formats are the reference's, so that files written by either package read in the other:
``get_current_layout`` returns ``{"<rank>": {parameter name: layout.to_dict() + {"type": dtype string,
"full_shape": global shape}}}``, ``get_global_layout`` the union over all ranks, ``combine_layout`` the
union over the ``*.layout`` files of a folder (a rank id may appear once only).  Parameters are named
by their qualified name in the module (the reference reads a ``name`` attribute that torch parameters
do not have).
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict

from ...collectives import cc
from ..dtensor import DTensor


def _jsonable(v):
    if isinstance(v, (tuple, list)):
        return [_jsonable(i) for i in v]
    return v


def get_current_layout(cell) -> Dict[str, Dict[str, dict]]:
    """``{"<this rank>": {parameter fqn: layout + dtype + global shape}}`` of the DTensor parameters."""
    params: Dict[str, dict] = {}
    for name, p in cell.named_parameters():
        if isinstance(p, DTensor):
            d = {k: _jsonable(v) for k, v in p.layout.to_dict().items()}
            d["type"] = str(p.dtype)
            d["full_shape"] = [int(s) for s in p.shape]
            params[name] = d
    return {str(cc.get_rank()): params}


def get_global_layout(cell) -> Dict[str, Dict[str, dict]]:
    """The layouts of every rank, keyed by rank id (a collective: every rank must call it)."""
    local = get_current_layout(cell)
    if not cc.is_initialized():
        return local
    out: Dict[str, Dict[str, dict]] = {}
    for part in cc.all_gather_object(local):
        out.update(part)
    return out


def save_layout(layout_dict: dict, path: str) -> None:
    path = str(path)              # any name is accepted; ``combine_layout`` reads the ``*.layout`` files of a folder
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(layout_dict, f, ensure_ascii=False)
    os.replace(tmp, path)


def load_layout(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def combine_layout(directory: str) -> Dict[str, dict]:
    """Union of every ``*.layout`` file of ``directory``, keyed by rank id; a rank id found in two files
    raises ``ValueError``."""
    out: Dict[str, dict] = {}
    for p in sorted(glob.glob(os.path.join(str(directory), "*.layout"))):
        for rank_id, params in load_layout(p).items():
            if rank_id in out:
                raise ValueError(f"rank id {rank_id} appears in more than one layout file ({p})")
            out[rank_id] = params
    return out
