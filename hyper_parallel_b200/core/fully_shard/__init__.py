from .api import HSDPModule, fully_shard, get_model_state_dict  # noqa: F401
from .utils import (CPUOffloadPolicy, DDPMeshInfo, FSDPMeshInfo, HSDPMeshInfo, MixedPrecisionPolicy,  # noqa: F401
                    OffloadPolicy, StateDictOptions)
