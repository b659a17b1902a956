"""Per-mesh-dimension placement tags: ``Shard(dim)``, ``Replicate()``, ``Partial(op)``.

Same vocabulary as hyper_parallel/core/placement_types.py:19-135 of the reference:
one placement per *mesh* dimension says how the tensor relates to that axis.
"""
from __future__ import annotations

_REDUCE_OPS = ("sum", "max", "min", "avg", "prod", "all")


class Placement:
    """Base class of all placements."""

    __slots__ = ()

    def is_shard(self, dim=None) -> bool:
        return False

    def is_replicate(self) -> bool:
        return False

    def is_partial(self, reduce_op=None) -> bool:
        return False


class Shard(Placement):
    """The tensor dimension ``dim`` is split evenly along this mesh axis."""

    __slots__ = ("dim",)

    def __init__(self, dim: int):
        if not isinstance(dim, int) or isinstance(dim, bool):
            raise TypeError(f"Shard dim must be an int, got {type(dim).__name__}")
        object.__setattr__(self, "dim", dim)

    def __setattr__(self, key, value):
        raise AttributeError("Shard is immutable")

    def __reduce__(self):
        # immutable slots: pickling (placements travel between pipeline stages) goes through __init__
        return (Shard, (self.dim,))

    def is_shard(self, dim=None) -> bool:
        return dim is None or dim == self.dim

    def __eq__(self, other):
        return isinstance(other, Shard) and other.dim == self.dim

    def __hash__(self):
        return hash(("S", self.dim))

    def __repr__(self):
        return f"Shard(dim={self.dim})"

    __str__ = lambda self: f"S({self.dim})"  # noqa: E731


class Replicate(Placement):
    """Every rank along this mesh axis holds the same data."""

    __slots__ = ()

    def is_replicate(self) -> bool:
        return True

    def __eq__(self, other):
        return isinstance(other, Replicate)

    def __hash__(self):
        return hash("R")

    def __repr__(self):
        return "Replicate()"

    __str__ = lambda self: "R"  # noqa: E731


class Partial(Placement):
    """Ranks along this mesh axis hold partial values pending a reduction ``reduce_op``."""

    __slots__ = ("reduce_op",)

    def __init__(self, reduce_op: str = "sum"):
        if reduce_op not in _REDUCE_OPS:
            raise ValueError(f"reduce_op must be one of {_REDUCE_OPS}, got {reduce_op!r}")
        object.__setattr__(self, "reduce_op", reduce_op)

    def __setattr__(self, key, value):
        raise AttributeError("Partial is immutable")

    def __reduce__(self):
        return (Partial, (self.reduce_op,))

    def is_partial(self, reduce_op=None) -> bool:
        return reduce_op is None or reduce_op == self.reduce_op

    def __eq__(self, other):
        return isinstance(other, Partial) and other.reduce_op == self.reduce_op

    def __hash__(self):
        return hash(("P", self.reduce_op))

    def __repr__(self):
        return f"Partial({self.reduce_op})"

    __str__ = lambda self: f"P({self.reduce_op})"  # noqa: E731
