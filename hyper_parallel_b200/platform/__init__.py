"""The single (torch) platform object.

The reference selects a MindSpore or torch backend at import time
(hyper_parallel/platform/platform.py:63-90); here torch is the only backend, and
``get_platform()`` returns a small facade over :mod:`hyper_parallel_b200.collectives.cc`
for code that was written against the reference's ``platform`` object.
"""
from __future__ import annotations

import torch

from ..collectives import cc


class TorchPlatform:
    Tensor = torch.Tensor
    Module = torch.nn.Module
    Parameter = torch.nn.Parameter

    @property
    def DTensorBase(self):
        from ..core.dtensor import DTensor
        return DTensor

    # rank / world ---------------------------------------------------------
    get_rank = staticmethod(cc.get_rank)
    get_world_size = staticmethod(cc.get_world_size)
    init_process_group = staticmethod(cc.init_process_group)
    destroy_process_group = staticmethod(cc.destroy_process_group)
    get_process_group_ranks = staticmethod(cc.get_process_group_ranks)
    get_backend = staticmethod(cc.get_backend)
    split_group = staticmethod(cc.split_group)

    @staticmethod
    def create_group(rank_list, group_name=None):
        return cc.group_for_ranks(rank_list, group_desc=group_name)

    # differentiable collectives ------------------------------------------
    differentiable_all_gather_concat = staticmethod(
        lambda data, group, concat_size=None, concat_dim=0: cc.all_gather_concat(data, concat_dim, group))
    differentiable_all_reduce = staticmethod(lambda data, op, group: cc.all_reduce(data, op, group))
    differentiable_reduce_scatter = staticmethod(
        lambda data, dev_num, axis, op, group: cc.reduce_scatter(data, axis, group, op))
    differentiable_all_to_all = staticmethod(
        lambda data, split_dim, concat_dim, group: cc.all_to_all(data, split_dim, concat_dim, group))

    # raw collectives --------------------------------------------------------
    all_gather_into_tensor = staticmethod(cc.all_gather_into)
    reduce_scatter_tensor = staticmethod(cc.reduce_scatter_into)
    all_reduce = staticmethod(cc.all_reduce_)
    broadcast = staticmethod(cc.broadcast)
    all_gather_object = staticmethod(cc.all_gather_object)

    @staticmethod
    def device():
        if torch.cuda.is_available():
            return torch.device("cuda", torch.cuda.current_device())
        return torch.device("cpu")

    @staticmethod
    def get_op_name(func):
        from ..core.shard._op_dispatch import get_op_name
        return get_op_name(func)


_PLATFORM = TorchPlatform()


def get_platform() -> TorchPlatform:
    return _PLATFORM
