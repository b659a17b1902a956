"""``fully_shard`` policies and mesh descriptions under the reference's module path."""
from . import utils  # noqa: F401
