"""Process groups and collective primitives."""
from .cc import (destroy_process_group, get_backend, get_process_group_ranks,  # noqa: F401
                 init_process_group, split_group)
