"""Distributed-op dispatcher: every ``torch`` call on a DTensor lands here.

Behaviour follows hyper_parallel/core/shard/_op_dispatch.py:91-675 of the reference:

* rules are declared in YAML files (``core/shard/ops/yaml`` or the directory named
  by ``HYPER_PARALLEL_OPS_YAML_DIR``); each entry names a rule class and the
  module or file that defines it; ``__default__`` supplies per-file defaults;
  ``HYPER_PARALLEL_OPS_PYTHON_PATH`` (``:``-separated) is searched for rule files
  -- this is how custom distributed ops are registered;
* the op name is ``func.__name__`` (or the core name of an ``OpOverload``);
* names on the pass-through list, and everything inside ``SkipDTensorDispatch``,
  run on the local tensors and return plain results;
* an op with no rule raises ``RuntimeError``;
* otherwise: collect input layouts -> (cached) ``infer_layout`` -> optional
  replacement callable -> run on local tensors -> wrap outputs in DTensors.

``infer_layout_suffix`` selects what the rule receives in ``extra_args``:
``""`` the non-DTensor args; ``"WithShape"`` the same plus, appended, the list of
input global shapes; ``"WithTupleExpand"`` expands a leading list/tuple of
tensors into individual inputs (``cat``-like ops).  ``"Reshape"`` and ``"Slice"``
are the reference's two special forms (``_op_dispatch.py:372-417`` and ``:543-593``
there): the rule of ``op(x, shape)`` receives ``[shape, global input shape]`` and
returns ``(layout, local shape)``, the rule of ``op(x, begin, end)`` receives
``[begin, end, global input shape]`` and returns ``(layout, local begin, local end)``;
the op then runs as ``impl(local x, local shape)`` / ``impl(local x, begin, end)``.
Rules written for the reference and registered with these suffixes work unchanged.
This package's own reshape / slice rules set ``_with_shape_convention`` and are
called in the ``"WithShape"`` form instead, which also serves ``view(*sizes)``,
``flatten``, ``unflatten``, ``narrow``, ``select`` and ``__getitem__``.

The cache key is a tuple of the input layouts' interned strings and the reprs of
the scalar arguments, so a steady-state call costs one dict lookup.
"""
from __future__ import annotations

import importlib
import os
import sys
from typing import Any, Dict, List, Optional, Tuple

import torch
import yaml

from ..dtensor import DTensor, _dispatch_enabled
from ..layout import Layout
from .ops.parallel_ops import get_distributed_op

_PASSTHROUGH = {
    "requires_grad_", "item", "__get__", "__set__", "register_hook", "is_complex", "__bool__",
    "__len__", "__format__", "dim", "__repr__", "__str__", "tolist", "numpy", "is_floating_point",
    "data_ptr", "element_size", "is_contiguous", "stride", "storage_offset", "untyped_storage",
    "_is_view", "is_shared", "get_device", "record_stream", "is_pinned", "__hash__", "__index__",
    "__int__", "__float__", "is_inference", "_version", "nelement", "retain_grad", "is_same_size",
    "__deepcopy__", "__reduce_ex__", "__setstate__", "is_meta", "is_cpu", "is_cuda",
    "has_names", "is_signed", "is_nonzero", "result_type", "can_cast", "set_", "__dlpack__",
    "share_memory_", "pin_memory", "_foreach_add_", "_foreach_mul_", "_foreach_addcmul_",
    "_foreach_addcdiv_", "_foreach_sqrt", "_foreach_div_", "_foreach_lerp_", "_foreach_neg",
    "_foreach_add", "_foreach_mul", "_foreach_div", "_foreach_sub_", "_foreach_zero_",
    "_foreach_norm", "_foreach_copy_", "_foreach_pow", "_foreach_maximum_", "_foreach_sub",
    "_foreach_reciprocal_", "_foreach_neg_", "_foreach_sqrt_", "_fused_adamw_", "_fused_adam_",
    "_fused_sgd_", "is_grads_batched", "_has_compatible_shallow_copy_type",
}


# Where the reference keeps a rule class in a file of another name (or under another class name), so
# that a YAML entry written against the reference's catalogue -- an own op mapped onto a stock rule --
# resolves here too.  Keys: the reference's ``distributed_op_file`` / ``distributed_op_class``.
_AXIS_OPS_FILES = ("parallel_activation_with_axis", "parallel_concat", "parallel_cumsum", "parallel_gather",
                   "parallel_isin", "parallel_masked_scatter", "parallel_multinomial", "parallel_new_ones",
                   "parallel_one_hot_ext", "parallel_pad", "parallel_repeat_interleave", "parallel_scatter",
                   "parallel_scatter_update", "parallel_sort", "parallel_split", "parallel_topk", "parallel_unbind")
_FILE_ALIASES = {**{f: "parallel_axis_ops" for f in _AXIS_OPS_FILES},
                 "parallel_argmax_with_value_ops": "parallel_reduce",
                 "parallel_tuple_elementwise": "parallel_elementwise",
                 "parallel_npu_flash_attention_score": "parallel_flash_attention_score",
                 "parallel_ms_flash_attention_score": "parallel_flash_attention_score",
                 "parallel_slice_ext": "parallel_slice"}
_CLASS_ALIASES = {"GatherNdDistributedOp": "GatherDistributedOp", "ScatterUpdateDistributedOp": "ScatterDistributedOp",
                  "SliceExtDistributedOp": "SliceDistributedOp", "SplitTensorDistributedOp": "SplitDistributedOp",
                  "SplitTensorViewDistributedOp": "SplitDistributedOp", "SplitWithSizeDistributedOp": "SplitDistributedOp",
                  "SplitWithSizeViewDistributedOp": "SplitDistributedOp"}


def _plain(a):
    """torch.Size / nested lists as plain tuples (hashable, printable the same on every rank)."""
    return tuple(_plain(i) for i in a) if isinstance(a, (list, tuple)) else a


def get_op_name(func) -> str:
    name = getattr(func, "__name__", None)
    if name is not None:
        return name
    if isinstance(func, torch._ops.OpOverload):
        return func.name().split("::")[-1].split(".")[0]
    if isinstance(func, torch._ops.OpOverloadPacket):
        return str(func).split(".")[-1]
    text = str(func)
    if "built-in function" in text or "built-in method" in text:
        return text.split()[2].strip(">")
    if "function" in text:
        return text.split()[1]
    return "unknown_op"


def _unwrap(obj):
    if isinstance(obj, DTensor):
        return obj._local_tensor
    if isinstance(obj, (list, tuple)):
        if any(isinstance(o, (DTensor, list, tuple)) for o in obj):
            return type(obj)(_unwrap(o) for o in obj)
        return obj
    if isinstance(obj, dict):
        return {k: _unwrap(v) for k, v in obj.items()}
    return obj


def _key_of(arg) -> Any:
    if isinstance(arg, torch.Tensor):
        return "T"
    if isinstance(arg, (int, float, bool, str, type(None), torch.dtype, torch.device)):
        return arg
    if isinstance(arg, (list, tuple)):
        return tuple(_key_of(a) for a in arg)
    if isinstance(arg, slice):
        return ("slice", arg.start, arg.stop, arg.step)
    if arg is Ellipsis:
        return "..."
    return repr(arg)


class OpDispatcher:
    """Holds the YAML-declared rules and dispatches DTensor calls through them."""

    def __init__(self):
        self._env_yaml_dir = os.environ.get("HYPER_PARALLEL_OPS_YAML_DIR")
        self._env_python_path = os.environ.get("HYPER_PARALLEL_OPS_PYTHON_PATH")
        self.whitelist = set(_PASSTHROUGH)
        self._suffix: Dict[str, str] = {}
        self._cache: Dict[tuple, tuple] = {}
        self._extend_sys_path(self._env_python_path)
        here = os.path.dirname(os.path.realpath(__file__))
        self.layout_infer_ops: Dict[str, dict] = {}
        self.layout_infer_ops.update(self._load_yaml_dir(os.path.join(here, "ops", "yaml")))
        if self._env_yaml_dir:
            ydir = self._env_yaml_dir
            if not os.path.isabs(ydir):
                ydir = os.path.normpath(os.path.join(here, "..", ydir))
            self.layout_infer_ops.update(self._load_yaml_dir(ydir))
        for op_name, cfg in self.layout_infer_ops.items():
            self._register(op_name, cfg)

    # ------------------------------------------------------------ loading --
    @staticmethod
    def _extend_sys_path(paths: Optional[str]) -> None:
        for p in (paths or "").split(":"):
            if p and os.path.isdir(p) and p not in sys.path:
                sys.path.insert(0, p)

    @staticmethod
    def _load_yaml_dir(ydir: str) -> Dict[str, dict]:
        merged: Dict[str, dict] = {}
        if not os.path.isdir(ydir):
            return merged
        for fn in sorted(os.listdir(ydir)):
            if not fn.endswith((".yaml", ".yml")):
                continue
            with open(os.path.join(ydir, fn), "r", encoding="utf-8") as f:
                data = yaml.safe_load(f) or {}
            default = data.pop("__default__", {}) or {}
            for op_name, cfg in data.items():
                entry = dict(default)
                entry.update(cfg or {})
                merged[op_name] = entry
        return merged

    def _register(self, op_name: str, cfg: dict) -> None:
        cls_name = cfg["distributed_op_class"]
        if "distributed_op_module" in cfg:
            module = importlib.import_module(cfg["distributed_op_module"])
        else:
            mod_file = cfg["distributed_op_file"]
            try:
                module = importlib.import_module(f"{__package__}.ops.{mod_file}")
            except ImportError:
                try:
                    if not self._env_python_path:
                        raise
                    module = importlib.import_module(mod_file)
                except ImportError:
                    if mod_file not in _FILE_ALIASES:
                        raise
                    module = importlib.import_module(f"{__package__}.ops.{_FILE_ALIASES[mod_file]}")
        if not hasattr(module, cls_name) and cls_name in _CLASS_ALIASES:
            cls_name = _CLASS_ALIASES[cls_name]
        getattr(module, cls_name)(op_name)
        self._suffix[op_name] = cfg.get("infer_layout_suffix", "") or ""

    def register_op(self, op_name: str, rule_cls, suffix: str = "") -> None:
        """Programmatic registration (same effect as a YAML entry)."""
        rule_cls(op_name)
        self._suffix[op_name] = suffix
        self._cache = {k: v for k, v in self._cache.items() if k[0] != op_name}

    # ----------------------------------------------------------- dispatch --
    def dispatch(self, func, args: tuple, kwargs: dict):
        name = get_op_name(func)
        if not _dispatch_enabled() or name in self.whitelist:
            return func(*_unwrap(args), **_unwrap(kwargs))
        rule = get_distributed_op(name)
        if rule is None:
            raise RuntimeError(f"Operator {name} does not have a distributed layout rule; register one "
                               "through a YAML entry (HYPER_PARALLEL_OPS_YAML_DIR) or wrap the call in "
                               "custom_shard / SkipDTensorDispatch")
        suffix = self._suffix.get(name, "")
        if suffix == "WithTupleExpand" and args and isinstance(args[0], (list, tuple)):
            return self._dispatch_tuple_expand(func, name, rule, args, kwargs)

        if suffix in ("Reshape", "Slice") and not getattr(rule, "_with_shape_convention", False):
            return self._dispatch_reference_form(func, name, rule, suffix, args, kwargs)
        with_shape = suffix in ("WithShape", "Reshape", "Slice")
        layouts: List[Optional[Layout]] = []
        extra: List[Any] = []
        shapes: List[Any] = []
        key_parts: List[Any] = [name]
        local_args = []
        for a in args:
            if isinstance(a, DTensor):
                lay = a._layout
                layouts.append(lay)
                key_parts.append(lay.compact_str)
                local_args.append(a._local_tensor)
                if with_shape:
                    shp = tuple(lay.get_global_shape(a._local_tensor.shape))
                    shapes.append(shp)
                    key_parts.append(shp)
            else:
                layouts.append(None)
                if a is not None:
                    extra.append(a)
                key_parts.append(_key_of(a))
                local_args.append(_unwrap(a))
                if with_shape:
                    shapes.append(tuple(a.shape) if isinstance(a, torch.Tensor) else None)
        local_kwargs = {}
        for k, v in kwargs.items():
            if isinstance(v, DTensor):
                lay = v._layout
                layouts.append(lay)
                key_parts.append((k, lay.compact_str))
                local_kwargs[k] = v._local_tensor
                if with_shape:
                    shp = tuple(lay.get_global_shape(v._local_tensor.shape))
                    shapes.append(shp)
                    key_parts.append(shp)
            else:
                layouts.append(None)
                if v is not None:
                    extra.append(v)
                key_parts.append((k, _key_of(v)))
                local_kwargs[k] = _unwrap(v)
                if with_shape:
                    shapes.append(tuple(v.shape) if isinstance(v, torch.Tensor) else None)
        if with_shape:
            extra.append(shapes)
        key = tuple(key_parts)
        try:
            plan = self._cache.get(key)
        except TypeError:  # unhashable scalar argument
            key, plan = None, None
        if plan is None:
            out_layout = rule.infer_layout(layouts, extra)
            impl = rule.get_expand_impl(func, out_layout, layouts, extra) or func
            plan = (out_layout, impl)
            if key is not None:
                self._cache[key] = plan
        out_layout, impl = plan
        result = impl(*local_args, **local_kwargs)
        return self._wrap_outputs(result, out_layout)

    def _dispatch_reference_form(self, func, name, rule, suffix, args, kwargs):
        """``Reshape``: ``op(x, shape)``; ``Slice``: ``op(x, begin, end)`` -- the argument lists and
        return tuples of the reference (see the module docstring)."""
        n_extra = 1 if suffix == "Reshape" else 2
        if kwargs or len(args) != 1 + n_extra or not isinstance(args[0], DTensor):
            raise TypeError(f"{name}: the {suffix!r} calling convention takes (DTensor, "
                            + ("shape)" if suffix == "Reshape" else "begin, end)") + " positionally")
        x = args[0]
        lay = x._layout
        global_shape = tuple(lay.get_global_shape(x._local_tensor.shape))
        extra = [_plain(a) for a in args[1:]] + [global_shape]
        key = (name, suffix, lay.compact_str) + tuple(_key_of(e) for e in extra)
        try:
            plan = self._cache.get(key)
        except TypeError:
            key, plan = None, None
        if plan is None:
            inferred = rule.infer_layout([lay], extra)
            if not isinstance(inferred, (tuple, list)) or len(inferred) != 1 + n_extra:
                raise TypeError(f"{name}: a {suffix!r} rule must return (layout, "
                                + ("local_shape)" if suffix == "Reshape" else "begin, end)"))
            impl = rule.get_expand_impl(func, inferred, [lay], extra) or func
            plan = (inferred, impl)
            if key is not None:
                self._cache[key] = plan
        inferred, impl = plan
        result = impl(x._local_tensor, *inferred[1:])
        return DTensor(result, inferred[0]) if isinstance(result, torch.Tensor) else result

    def _dispatch_tuple_expand(self, func, name, rule, args, kwargs):
        seq = args[0]
        layouts = [t._layout if isinstance(t, DTensor) else None for t in seq]
        rest = list(args[1:])
        extra = [a for a in rest if a is not None] + [v for v in kwargs.values() if v is not None]
        key = (name, tuple(l.compact_str if l is not None else "T" for l in layouts),
               tuple(_key_of(a) for a in rest), tuple((k, _key_of(v)) for k, v in kwargs.items()),
               tuple(tuple(t.shape) for t in seq))
        plan = self._cache.get(key)
        if plan is None:
            shapes = [tuple(t.shape) for t in seq]
            out_layout = rule.infer_layout(layouts, extra + [shapes])
            impl = rule.get_expand_impl(func, out_layout, layouts, extra + [shapes]) or func
            plan = (out_layout, impl)
            self._cache[key] = plan
        out_layout, impl = plan
        result = impl(type(seq)(_unwrap(t) for t in seq), *_unwrap(tuple(rest)), **_unwrap(kwargs))
        return self._wrap_outputs(result, out_layout)

    @staticmethod
    def _wrap_outputs(result, out_layout):
        if out_layout is None:
            return result
        if isinstance(result, (tuple, list)):
            if not isinstance(out_layout, (tuple, list)):
                out_layout = [out_layout] * len(result)
            if len(out_layout) != len(result):
                raise RuntimeError(f"Output tuple size ({len(result)}) does not match layout tuple "
                                   f"size ({len(out_layout)})")
            wrapped = [DTensor._wrap(r, l) if (l is not None and isinstance(r, torch.Tensor)) else r
                       for r, l in zip(result, out_layout)]
            if hasattr(result, "_fields"):  # namedtuple (torch.return_types.*) -> plain tuple
                return tuple(wrapped)
            return type(result)(wrapped)
        if isinstance(out_layout, (tuple, list)):
            out_layout = out_layout[0]
        if not isinstance(result, torch.Tensor):
            return result
        return DTensor._wrap(result, out_layout)

    def clear_cache(self) -> None:
        self._cache.clear()


_OP_DISPATCHER = OpDispatcher()


def enable_dtensor_dispatch():
    from .. import dtensor as _d
    _d._DISPATCH_ENABLED = True


def disable_dtensor_dispatch():
    from .. import dtensor as _d
    _d._DISPATCH_ENABLED = False
