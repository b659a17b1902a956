"""Base class and registry of distributed-op layout rules.

Contract (same as hyper_parallel/core/shard/ops/parallel_ops.py:21-84 and
parallel_ops_register.py:18-40 of the reference, so that user-written rules port
unchanged): a rule derives :class:`DistributedOp`, is instantiated with the op
name it serves (which registers it), and implements

``infer_layout(layouts, extra_args)``
    ``layouts`` has one entry per positional argument and then per keyword
    argument: the :class:`Layout` of a DTensor argument, ``None`` otherwise.
    ``extra_args`` lists the non-DTensor arguments in order.  Returns the output
    ``Layout`` (or a tuple of layouts, ``None`` entries for non-tensor outputs).

``get_expand_impl(func, output_layout, layouts, extra_args)`` (optional)
    returns a callable to run on the *local* tensors instead of ``func``.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

from ...layout import Layout

_DISTRIBUTED_OPS: Dict[str, "DistributedOp"] = {}


def register_distributed_op(op_name: str, op: "DistributedOp") -> None:
    _DISTRIBUTED_OPS[op_name] = op


def get_distributed_op(op_name: str) -> Optional["DistributedOp"]:
    return _DISTRIBUTED_OPS.get(op_name)


def registered_ops() -> List[str]:
    return sorted(_DISTRIBUTED_OPS)


class DistributedOp:
    """Layout rule of one operator name."""

    _allow_partial_inputs = False

    def __init__(self, op_name: str):
        self.op_name = op_name
        register_distributed_op(op_name, self)

    # -- helpers -------------------------------------------------------------
    def _check_partial_inputs(self, layouts: Sequence[Optional[Layout]]) -> None:
        if self._allow_partial_inputs:
            return
        for i, lay in enumerate(layouts):
            if lay is not None and lay.is_partial():
                raise ValueError(
                    f"For {self.op_name}, input {i} with {lay} has Partial status which is not allowed. "
                    "Should be without Partial status for this operation.")

    @staticmethod
    def first_layout(layouts: Sequence[Optional[Layout]]) -> Layout:
        for lay in layouts:
            if lay is not None:
                return lay
        raise ValueError("operator received no distributed tensor")

    # -- contract ------------------------------------------------------------
    def infer_layout(self, layouts, extra_args):
        """Default: the output is laid out like the first distributed input."""
        self._check_partial_inputs(layouts)
        return self.first_layout(layouts)

    def get_expand_impl(self, func, output_layout, layouts, extra_args):
        return None
