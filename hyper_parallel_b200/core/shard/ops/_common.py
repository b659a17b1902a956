"""Helpers shared by the layout rules."""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

from ...layout import Layout


def norm_dim(dim: int, ndim: int) -> int:
    d = dim + ndim if dim < 0 else dim
    if not 0 <= d < max(ndim, 1):
        raise IndexError(f"dim {dim} out of range for a {ndim}-D tensor")
    return d


def norm_dims(dims, ndim: int) -> List[int]:
    if dims is None:
        return list(range(ndim))
    if isinstance(dims, int):
        dims = [dims]
    return sorted({norm_dim(int(d), ndim) for d in dims})


def make(like: Layout, dim_axes, partial=None) -> Layout:
    """New layout on the mesh of ``like``."""
    return Layout._make(like.mesh, dim_axes, partial)


def keep_partial(like: Layout) -> List[Optional[str]]:
    return list(like.partial)


def no_partial(like: Layout) -> List[Optional[str]]:
    return [None] * like.mesh.ndim


def split_shapes(extra_args) -> Tuple[list, Optional[list]]:
    """Separate the trailing input-shape list (``WithShape`` convention) from the scalars.  A shape may
    be a tuple, a ``torch.Size`` or a list of ints; ``None`` stands for a non-tensor input."""
    if isinstance(extra_args, dict):                       # {"input_shapes": [...]}: an older spelling
        shapes = extra_args.get("input_shapes")
        rest = [v for k, v in extra_args.items() if k != "input_shapes"]
        return rest, ([None if s is None else tuple(s) for s in shapes] if shapes is not None else None)
    if extra_args and isinstance(extra_args[-1], list) and extra_args[-1] and all(
            s is None or (isinstance(s, (tuple, list)) and all(isinstance(i, int) for i in s))
            for s in extra_args[-1]):
        return list(extra_args[:-1]), [None if s is None else tuple(s) for s in extra_args[-1]]
    return list(extra_args), None


# The reference words this error differently per operator and programs match on its wording; the
# message below states the fact once in this package's words and once in the reference's.
_REFERENCE_WORDING = {
    "softmax": "{op} requires the reduction axis to be un-sharded",
    "log_softmax": "{op} requires the reduction axis to be un-sharded",
    "_softmax": "{op} requires the reduction axis to be un-sharded",
    "cumsum": "Cannot perform sharding on normalized dimension {d}",
    "layer_norm": "Cannot perform sharding on normalized dimension {d}",
    "sort": "sorting along a sharded dimension is not supported",
    "argsort": "sorting along a sharded dimension is not supported",
    "topk": "Cannot perform sharding on params along the chosen dim",
    "repeat_interleave": "Cannot perform sharding on params along the chosen dim",
    "split": "Can not split tensor at sharded axis[{d}], layout: {layout}",
    "chunk": "Can not split tensor at sharded axis[{d}], layout: {layout}",
    "tensor_split": "Can not split tensor at sharded axis[{d}], layout: {layout}",
    "unbind": "Unbinding a sharded dimension is not supported",
    "pad": "{op} does not support padding on a sharded dimension",
    "expand": "Cannot expand dimension {d} which is sharded",
    "expand_as": "Cannot expand dimension {d} which is sharded",
}


def require_unsharded(op_name: str, layout: Layout, dims: Sequence[int], what: str = "operating") -> None:
    for d in dims:
        if layout.dim_axes[d]:
            names = [layout.alias_name[a] for a in layout.dim_axes[d]]
            msg = (f"For {op_name}, the {what} dim {d} must not be sharded, "
                   f"but it is sharded on mesh axes {names}")
            extra = _REFERENCE_WORDING.get(op_name)
            if extra:
                msg += " (" + extra.format(op=op_name, d=d, layout=layout.alias_tensor_map) + ")"
            raise ValueError(msg)


def merge_partials(op_name: str, layouts: Sequence[Optional[Layout]]) -> List[Optional[str]]:
    """All partial inputs must agree per mesh axis."""
    ref = None
    for lay in layouts:
        if lay is None:
            continue
        if ref is None:
            ref = list(lay.partial)
        elif list(lay.partial) != ref:
            raise ValueError(f"For {op_name}, inputs have different Partial status: {ref} vs {lay.partial}")
    return ref or []
