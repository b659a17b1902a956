from .api import parallelize_value_and_grad, shard, shard_module, shard_parameter  # noqa: F401
from .local_func import custom_shard  # noqa: F401
from .sharding_plan import ShardingPlan  # noqa: F401
