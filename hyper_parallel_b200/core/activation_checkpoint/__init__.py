from .activation_checkpoint import (CheckpointPolicy, CheckpointWrapper, checkpoint, checkpoint_wrapper,  # noqa: F401
                                    create_selective_checkpoint_contexts)
from .activation_swap import ActivationPolicy, AsyncSaveOnCpu, SwapWrapper, swap_wrapper  # noqa: F401
from .swap import Storage, SwapGroup, SwapManager, SwapState, SwapTensor  # noqa: F401
