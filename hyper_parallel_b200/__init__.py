"""hyper_parallel_b200: a Blackwell-native hybrid-parallel training framework for PyTorch.

Public surface (the names of hyper_parallel/__init__.py:16-34 of the reference plus the
spellings its README uses).
"""
__version__ = "0.1.0"

from .platform import get_platform
from .collectives.cc import (destroy_process_group, get_backend, get_process_group_ranks,
                             init_process_group, split_group)
from .core.placement_types import Partial, Placement, Replicate, Shard
from .core.device_mesh import DeviceMesh, init_device_mesh
from .core.layout import Layout
from .core.dtensor import (DTensor, SkipDTensorDispatch, distribute_tensor, empty, full, ones, zeros)
from .core.shard import (ShardingPlan, custom_shard, parallelize_value_and_grad, shard, shard_module)
from .core.shard.ops.parallel_ops import DistributedOp
from .core.hsdp import HSDPCell, hsdp, hsdp_sync_stream, teardown_hsdp
from .core.parameter_init import init_parameters
from .core.pipeline_parallel import (BatchDimSpec, MetaStep, MetaStepType, PipelineStage, Schedule1F1B,
                                     ScheduleGPipe, ScheduleInterleaved1F1B, SharedParameterInfo,
                                     validate_pipeline_execution)

from .core import function_override as _function_override

_function_override.install()

__all__ = [
    "get_platform", "hsdp", "hsdp_sync_stream", "teardown_hsdp", "HSDPCell", "Layout", "DTensor", "DeviceMesh",
    "init_device_mesh", "init_parameters", "shard_module", "shard", "custom_shard",
    "parallelize_value_and_grad", "SkipDTensorDispatch", "ShardingPlan", "DistributedOp",
    "Shard", "Replicate", "Partial", "Placement", "distribute_tensor", "ones", "zeros", "empty", "full",
    "init_process_group", "destroy_process_group", "get_process_group_ranks", "get_backend",
    "split_group",
    "MetaStep", "MetaStepType", "BatchDimSpec", "PipelineStage", "SharedParameterInfo",
    "ScheduleInterleaved1F1B", "Schedule1F1B", "ScheduleGPipe", "validate_pipeline_execution",
]
