"""``ShardingPlan``: declarative description of how a module is sharded
(hyper_parallel/core/shard/sharding_plan.py:20-52 of the reference)."""
from dataclasses import dataclass
from typing import Any, Dict, List, Optional


@dataclass
class ShardingPlan:
    """
    Attributes:
        plan: ``{parameter fqn: spec}``; a spec is a tuple of axis aliases (one entry per tensor
            dim, ``"None"`` = unsharded, nested tuple = several axes) or of placements (one per
            mesh dim), or a ready ``Layout``.
        input_plan: ``{"input" | "<submodule>.input": spec | [spec per positional arg] | {kwarg: spec}}``.
        output_plan: ``{"output" | "<submodule>.output": spec | [spec per output]}``.
        return_local_tensor: names of submodules whose outputs are converted to local tensors.
    """
    plan: Optional[Dict[str, Any]] = None
    input_plan: Optional[Dict[str, Any]] = None
    output_plan: Optional[Dict[str, Any]] = None
    return_local_tensor: Optional[List[str]] = None
