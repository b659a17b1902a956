"""``get_platform`` / ``get_torch_platform`` under the module path the reference uses
(hyper_parallel/platform/platform.py:63-110).  Torch is the only backend here, so both return the
same object."""
from . import TorchPlatform, get_platform  # noqa: F401


def get_torch_platform() -> TorchPlatform:
    return get_platform()
