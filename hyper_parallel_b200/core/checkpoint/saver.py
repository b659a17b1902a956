"""Single-file helper (hyper_parallel/core/checkpoint/saver.py:25-40)."""
import os

import torch

from .util import check_file_name


def save_checkpoint(obj, file_path: str) -> None:
    """Atomically ``torch.save`` ``obj`` to ``file_path`` (validated name)."""
    path = check_file_name(file_path)
    tmp = path + ".tmp"
    with open(tmp, "wb") as f:
        torch.save(obj, f)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)
