"""sm_100a kernels and their autograd wrappers."""
from . import native  # noqa: F401
from .functional import *  # noqa: F401,F403
from . import attention, moe  # noqa: F401,E402
