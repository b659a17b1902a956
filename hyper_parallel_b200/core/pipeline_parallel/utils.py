"""Micro-batch splitting helpers (hyper_parallel/core/pipeline_parallel/utils.py:18-47 and
hyper_parallel/platform/torch/pipeline_parallel/_utils.py:20-103 of the reference)."""
from __future__ import annotations

from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch

from ..dtensor import DTensor


class BatchDimSpec:
    """Which dimension of an argument is the batch dimension (split into micro-batches)."""

    __slots__ = ("batch_dim",)

    def __init__(self, batch_dim: int):
        if not isinstance(batch_dim, int) or isinstance(batch_dim, bool):
            raise TypeError(f"batch_dim must be int, but got type {type(batch_dim)}.")
        self.batch_dim = batch_dim

    def __repr__(self):
        return f"BatchDimSpec({self.batch_dim})"

    @staticmethod
    def from_tuple(batch_dims):
        if not isinstance(batch_dims, tuple):
            raise TypeError(f"batch_dims must be tuple, but got type {type(batch_dims)}.")
        return tuple(BatchDimSpec(d) for d in batch_dims)

    @staticmethod
    def from_dict(batch_dims):
        if not isinstance(batch_dims, dict):
            raise TypeError(f"batch_dims must be dict, but got type {type(batch_dims)}.")
        return {k: BatchDimSpec(d) for k, d in batch_dims.items()}


def _split_one(value, n: int, spec: Optional[BatchDimSpec]):
    if not isinstance(value, torch.Tensor) or spec is None:
        return [value] * n
    dim = spec.batch_dim
    if isinstance(value, DTensor):
        local = value.to_local()
        if local.shape[dim] % n:
            raise ValueError(f"local batch dim of size {local.shape[dim]} is not divisible by {n} micro-batches")
        return [DTensor._wrap(c, value.layout) for c in local.chunk(n, dim=dim)]
    if value.shape[dim] % n:
        raise ValueError(f"batch dim of size {value.shape[dim]} is not divisible by {n} micro-batches")
    return list(value.chunk(n, dim=dim))


class MicroBatch:
    """Splits ``args`` / ``kwargs`` into ``micro_batch_num`` micro-batches along their batch dims."""

    def __init__(self, micro_batch_num: int, args_batch_dim=None, kwargs_batch_dim=None):
        if not isinstance(micro_batch_num, int) or micro_batch_num < 1:
            raise ValueError(f"micro_batch_num must be a positive int, got {micro_batch_num}")
        self.n = micro_batch_num
        self.args_batch_dim = args_batch_dim
        self.kwargs_batch_dim = kwargs_batch_dim

    def __call__(self, args: Sequence, kwargs: Dict[str, Any]) -> Tuple[List[tuple], List[dict]]:
        n = self.n
        specs = self.args_batch_dim
        if specs is None:
            specs = tuple(BatchDimSpec(0) for _ in args)
        if len(specs) != len(args):
            raise ValueError(f"args_batch_dim has {len(specs)} entries for {len(args)} arguments")
        cols = [_split_one(a, n, s) for a, s in zip(args, specs)]
        kspecs = self.kwargs_batch_dim or {k: BatchDimSpec(0) for k in kwargs}
        kcols = {k: _split_one(v, n, kspecs.get(k)) for k, v in kwargs.items()}
        micro_args = [tuple(c[i] for c in cols) for i in range(n)]
        micro_kwargs = [{k: c[i] for k, c in kcols.items()} for i in range(n)]
        return micro_args, micro_kwargs
