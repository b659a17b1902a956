"""The names of hyper_parallel/platform/torch/fully_shard/utils.py:8-93 of the reference."""
from ....core.fully_shard.utils import (CPUOffloadPolicy, DataParallelMeshInfo, DDPMeshInfo, FSDPMeshInfo,  # noqa: F401
                                        HSDPMeshInfo, MixedPrecisionPolicy, OffloadPolicy)
