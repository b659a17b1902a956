"""Layout json I/O (hyper_parallel/core/checkpoint/layout.py:26-131): per-rank ``*.layout`` files."""
from __future__ import annotations

import glob
import json
import os
from typing import Dict

from ...collectives import cc
from ..dtensor import DTensor


def get_current_layout(cell) -> Dict[str, dict]:
    """``{parameter fqn: layout.to_dict()}`` of this rank's DTensor parameters."""
    out = {}
    for name, p in cell.named_parameters():
        if isinstance(p, DTensor):
            d = p.layout.to_dict()
            out[name] = {k: (list(v) if isinstance(v, tuple) else v) for k, v in d.items()}
    return out


def get_global_layout(cell) -> Dict[int, Dict[str, dict]]:
    """``{rank: get_current_layout(cell)}`` gathered from every rank."""
    local = get_current_layout(cell)
    if not cc.is_initialized():
        return {0: local}
    return dict(enumerate(cc.all_gather_object(local)))


def save_layout(layout_dict: dict, path: str) -> None:
    if not path.endswith(".layout"):
        raise ValueError("layout files must end with .layout")
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    with open(tmp, "w", encoding="utf-8") as f:
        json.dump(layout_dict, f, indent=1)
    os.replace(tmp, path)


def load_layout(path: str) -> dict:
    with open(path, "r", encoding="utf-8") as f:
        return json.load(f)


def combine_layout(directory: str) -> Dict[str, dict]:
    """Merge every ``*.layout`` file of ``directory`` into ``{file stem: layout dict}``."""
    out = {}
    for p in sorted(glob.glob(os.path.join(directory, "*.layout"))):
        out[os.path.splitext(os.path.basename(p))[0]] = load_layout(p)
    return out
