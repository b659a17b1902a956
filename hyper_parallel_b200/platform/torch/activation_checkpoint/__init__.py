"""The names of hyper_parallel/platform/torch/activation_checkpoint/__init__.py of the reference."""
from ....core.activation_checkpoint.activation_swap import (ActivationPolicy, AsyncSaveOnCpu, SwapWrapper,  # noqa: F401
                                                            swap_wrapper)
