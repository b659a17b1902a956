from .api import HSDPModule, fully_shard, get_model_state_dict, hsdp_sync_stream  # noqa: F401
from .utils import (CPUOffloadPolicy, DDPMeshInfo, FSDPMeshInfo, HSDPMeshInfo, MixedPrecisionPolicy,  # noqa: F401
                    OffloadPolicy, StateDictOptions)
