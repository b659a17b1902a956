"""Registry access under the module name the reference uses."""
from .parallel_ops import (get_distributed_op, register_distributed_op,  # noqa: F401
                           registered_ops)
