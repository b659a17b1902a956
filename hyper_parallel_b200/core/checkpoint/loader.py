"""Single-file helper (hyper_parallel/core/checkpoint/loader.py:25-40)."""
import os

import torch

from .util import check_file_name


def load_checkpoint(file_path: str, map_location="cpu", weights_only: bool = False):
    path = check_file_name(file_path)
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    return torch.load(path, map_location=map_location, weights_only=weights_only)
