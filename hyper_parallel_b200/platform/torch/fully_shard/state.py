"""Names of hyper_parallel/platform/torch/fully_shard/state.py that outside code imports."""
from typing import Optional

import torch

from ....core.fully_shard.state import FSDPState as TorchHSDPStateV2  # noqa: F401


def _to_dtype_if_needed(tensor: torch.Tensor, dtype: Optional[torch.dtype]) -> torch.Tensor:
    """``tensor`` itself when ``dtype`` is None or already its dtype, else a cast copy."""
    return tensor if dtype is None or tensor.dtype == dtype else tensor.to(dtype)
