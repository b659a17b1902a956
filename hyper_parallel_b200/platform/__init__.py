"""The single (_torch) platform object.

The reference selects a MindSpore or _torch backend at import time
(hyper_parallel/platform/platform.py:63-90); here _torch is the only backend, and
``get_platform()`` returns a small facade over :mod:`hyper_parallel_b200.collectives.cc`
for code that was written against the reference's ``platform`` object.
"""
from __future__ import annotations

import torch as _torch      # not ``torch``: the sub-package ``platform.torch`` takes that name in this namespace

from ..collectives import cc


class TorchPlatform:
    Tensor = _torch.Tensor
    Module = _torch.nn.Module
    Parameter = _torch.nn.Parameter

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
        if _torch.cuda.is_available():
            return _torch.device("cuda", _torch.cuda.current_device())
        return _torch.device("cpu")

    # tensors -----------------------------------------------------------------------
    ones = staticmethod(lambda size, dtype=None: _torch.ones(size, dtype=dtype))
    zeros = staticmethod(lambda size, dtype=None: _torch.zeros(size, dtype=dtype))
    full = staticmethod(lambda size, fill_value, dtype=None: _torch.full(size, fill_value, dtype=dtype))
    empty = staticmethod(lambda size, dtype=None: _torch.empty(size, dtype=dtype))
    full_like = staticmethod(lambda tensor, fill_value, dtype=None: _torch.full_like(tensor, fill_value, dtype=dtype))
    empty_like = staticmethod(lambda tensor, *, dtype=None, device=None, pin_memory=False:
                              _torch.empty_like(tensor, dtype=dtype, device=device, pin_memory=pin_memory))
    new_tensor = staticmethod(lambda shape, dtype, device: _torch.empty(size=shape, dtype=dtype, device=device))
    new_zero_parameter = staticmethod(lambda shape, dtype, requires_grad, device: _torch.nn.Parameter(
        _torch.zeros(shape, dtype=dtype, device=device), requires_grad=requires_grad))
    chunk = staticmethod(lambda data, split_dim, split_size, index: _torch.chunk(data, split_size, dim=split_dim)[index])
    tensor_to_numpy = staticmethod(lambda tensor: tensor.detach().cpu().numpy())
    no_grad = staticmethod(_torch.no_grad)
    manual_seed = staticmethod(_torch.manual_seed)

    @staticmethod
    def tensor_type_cast(input_data, cast_type):
        """Cast to a dtype given by name (``"float32"``, ``"bfloat16"``, ...) or as a ``torch.dtype``."""
        dtype = getattr(_torch, cast_type, None) if isinstance(cast_type, str) else cast_type
        if not isinstance(dtype, _torch.dtype):
            raise ValueError(f"unknown dtype {cast_type!r}")
        return input_data.to(dtype)

    @staticmethod
    def cast_fp_tensor(dtype, x):
        """``x`` cast to ``dtype`` when it is a floating-point tensor of another dtype, else ``x``."""
        if isinstance(x, _torch.Tensor) and x.is_floating_point() and dtype is not None and x.dtype != dtype:
            return x.to(dtype)
        return x

    @staticmethod
    def set_tensor_requires_grad(input_tensor):
        if input_tensor.is_leaf:
            input_tensor.requires_grad_()
        return input_tensor

    @staticmethod
    def tree_map(fn, tree):
        return _torch.utils._pytree.tree_map(fn, tree)

    @classmethod
    def apply_to_tensors(cls, fn, container):
        """``fn`` applied to every tensor inside nested lists / tuples / dicts; the rest is kept."""
        return cls.tree_map(lambda x: fn(x) if isinstance(x, _torch.Tensor) else x, container)

    # devices, streams, generators ---------------------------------------------------------
    @staticmethod
    def get_device_handle():
        """``torch.cuda`` (the module that owns devices, streams, events and generators)."""
        return _torch.cuda

    device_count = staticmethod(lambda device_handle=None: (device_handle or _torch.cuda).device_count())
    device_type = staticmethod(lambda: "cuda")
    new_stream = staticmethod(lambda: _torch.cuda.Stream())
    new_event = staticmethod(lambda: _torch.cuda.Event())
    get_current_stream = staticmethod(lambda: _torch.cuda.current_stream())
    get_stream_context = staticmethod(lambda: _torch.cuda.stream)

    @staticmethod
    def get_rng_state(device=None, device_handle=None):
        if device_handle is None:
            return _torch.get_rng_state()
        return device_handle.get_rng_state() if device is None else device_handle.get_rng_state(device)

    @staticmethod
    def set_rng_state(state, device=None, device_handle=None):
        if device_handle is None:
            return _torch.set_rng_state(state)
        return device_handle.set_rng_state(state) if device is None else device_handle.set_rng_state(state, device)

    # point-to-point and object collectives -------------------------------------------------------
    @staticmethod
    def get_global_rank(group, group_rank):
        return _torch.distributed.get_global_rank(group, group_rank)

    isend = staticmethod(lambda tensor, dst=None, group=None, tag=0: _torch.distributed.isend(tensor, dst, group, tag))
    irecv = staticmethod(lambda tensor, src=None, group=None, tag=0: _torch.distributed.irecv(tensor, src, group, tag))
    send_object_list = staticmethod(lambda obj_list, dst=None, group=None:
                                    _torch.distributed.send_object_list(obj_list, dst, group))
    recv_object_list = staticmethod(lambda obj_list, src=None, group=None:
                                    _torch.distributed.recv_object_list(obj_list, src, group))

    # modules and parameters -------------------------------------------------------------------
    get_cells_and_names = staticmethod(lambda cell: cell.named_modules())
    parameters_dict = staticmethod(lambda cell: cell.named_parameters())
    update_param_data = staticmethod(lambda param, data: setattr(param, "data", data))
    get_param_type_size = staticmethod(lambda param: param.element_size())
    register_forward_pre_hook = staticmethod(lambda cell, hook, **kw: cell.register_forward_pre_hook(hook, **kw))
    register_full_backward_hook = staticmethod(lambda cell, hook, **kw: cell.register_full_backward_hook(hook, **kw))
    register_full_backward_pre_hook = staticmethod(
        lambda cell, hook, **kw: cell.register_full_backward_pre_hook(hook, **kw))

    @staticmethod
    def get_param_local_shape(param):
        return param.local_shape if hasattr(param, "to_local") else param.shape

    @staticmethod
    def get_param_local_data(param):
        return param.to_local() if hasattr(param, "to_local") else param

    @staticmethod
    def search_parameter_by_name(cell, param_name: str):
        """``(owning module, name inside it, parameter)`` of a qualified parameter name, or ``None``."""
        owner, _, leaf = param_name.rpartition(".")
        try:
            mod = cell.get_submodule(owner) if owner else cell
        except AttributeError:
            return None
        p = mod._parameters.get(leaf)
        return None if p is None else (mod, leaf, p)

    @staticmethod
    def update_parameter_by_name(cell, result: tuple, new_param) -> bool:
        """Put ``new_param`` where ``search_parameter_by_name`` found the old one."""
        if not result:
            return False
        mod, leaf, _ = result
        mod._parameters[leaf] = new_param
        return True

    @staticmethod
    def set_layout_into_parameter(param, layout):
        """A parameter holding this rank's slice of ``param`` under ``layout`` (a DTensor parameter)."""
        from ..core.dtensor import DTensor, distribute_tensor
        if isinstance(param, DTensor):
            return param
        return _torch.nn.Parameter(distribute_tensor(param.detach(), layout), requires_grad=param.requires_grad)

    # checkpoints, activation checkpointing, pipelines, gradient handles ------------------------------------
    save_checkpoint = staticmethod(lambda cell, file_path: _torch.save(obj=cell, f=file_path))
    load_checkpoint = staticmethod(lambda file_path: _torch.load(f=file_path, weights_only=False))

    @property
    def checkpoint(self):
        return _torch.utils.checkpoint.checkpoint

    @property
    def noop_context_fn(self):
        return _torch.utils.checkpoint.noop_context_fn

    @staticmethod
    def ckpt_wrapper(module, checkpoint_fn=None, **kw):
        from ..core.activation_checkpoint import checkpoint_wrapper
        return checkpoint_wrapper(module, checkpoint_fn=checkpoint_fn, **kw)

    @staticmethod
    def create_selective_checkpoint_contexts(policy_fn_or_list, allow_cache_entry_mutation=False):
        from ..core.activation_checkpoint import create_selective_checkpoint_contexts
        return create_selective_checkpoint_contexts(policy_fn_or_list, allow_cache_entry_mutation)

    @staticmethod
    def async_save_on_cpu(policy_fn=None):
        from ..core.activation_checkpoint import AsyncSaveOnCpu
        return AsyncSaveOnCpu(policy_fn)

    @staticmethod
    def micro_batch(micro_batch_num, args_batch_dim=None, kwargs_batch_dim=None):
        from ..core.pipeline_parallel.utils import MicroBatch
        return MicroBatch(micro_batch_num, args_batch_dim, kwargs_batch_dim)

    @staticmethod
    def init_parameters(module, stage_index=0, **kw):
        from ..core.parameter_init import init_parameters
        return init_parameters(module, **kw)

    @staticmethod
    def wait_grad_handle():
        """Wait for the gradient reductions of ``hsdp`` and ``fully_shard`` that are still in flight."""
        from ..core.fully_shard import hsdp_sync_stream as fs_sync
        from ..core.hsdp import hsdp_sync_stream
        hsdp_sync_stream()
        fs_sync()

    @staticmethod
    def get_op_name(func):
        from ..core.shard._op_dispatch import get_op_name
        return get_op_name(func)


_PLATFORM = TorchPlatform()


def get_platform() -> TorchPlatform:
    return _PLATFORM
