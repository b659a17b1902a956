from .api import HSDPCell, hsdp, hsdp_sync_stream  # noqa: F401
from .hsdp_scheduler import teardown_hsdp  # noqa: F401

from .state_dict import get_sharded_state_dict, restore_optimizer_step  # noqa: F401,E402
