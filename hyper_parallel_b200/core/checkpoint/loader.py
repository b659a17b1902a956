"""Single-file helper (hyper_parallel/core/checkpoint/loader.py:25-40)."""
import os

import torch

from .util import has_valid_filename


def load_checkpoint(file_path: str, map_location="cpu", weights_only: bool = False):
    path = os.path.abspath(str(file_path))
    if not has_valid_filename(path):
        raise ValueError(f"Loader file_path should contains valid filename but get: {file_path}")
    if not os.path.exists(path):
        raise FileNotFoundError(path)
    return torch.load(path, map_location=map_location, weights_only=weights_only)
