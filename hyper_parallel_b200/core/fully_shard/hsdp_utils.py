"""State names of a ``fully_shard`` parameter, under the reference's module path
(hyper_parallel/core/fully_shard/hsdp_utils.py:76-83)."""
import enum


class ShardedState(enum.Enum):
    """``FSDPParam.sharded_state``: the module holds the DTensor shard (``SHARDED``), or the gathered
    full tensor (``UNSHARDED``).  ``SHARDED_POST_FORWARD`` (a differently sharded copy kept between
    forward and backward) is named for completeness; this implementation always reshards to the
    original shard."""
    SHARDED = enum.auto()
    SHARDED_POST_FORWARD = enum.auto()
    UNSHARDED = enum.auto()


class FSDPSchedulerState(enum.Enum):
    """Where a wrapped module is within one step: its pre-forward hook has run, its post-forward
    hook has run, its pre-backward hook has run, its post-backward hook has run."""
    PRE_FORWARD = enum.auto()
    FORWARD = enum.auto()
    PRE_BACKWARD = enum.auto()
    BACKWARD = enum.auto()


from ..hsdp.hsdp_utils import GroupInfo, OptimizerLevel  # noqa: E402,F401  (shared with ``hsdp``)
