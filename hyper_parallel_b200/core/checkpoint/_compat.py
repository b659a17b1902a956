"""Pickle compatibility with checkpoints written by the reference's torch build.

``.metadata`` is a pickle of dataclasses; a pickle names classes by module path.  Metadata
written here names the reference's module paths (``hyper_parallel.core.checkpoint...``) so the
reference can read it, and the reader accepts both spellings.
"""
from __future__ import annotations

import contextlib
import pickle
import sys
import types

_REF_PREFIX = "hyper_parallel.core.checkpoint."
_OUR_PREFIX = __name__.rsplit(".", 1)[0] + "."
_CLASSES = {"metadata": ["MetadataIndex", "ChunkStorageMetadata", "TensorProperties", "BytesStorageMetadata",
                         "TensorStorageMetadata", "Metadata"],
            "storage": ["StorageInfo"]}


class ReferenceCompatUnpickler(pickle.Unpickler):
    def find_class(self, module, name):
        if module.startswith(_REF_PREFIX):
            sub = module[len(_REF_PREFIX):]
            if sub == "filesystem_storage" and name == "StorageInfo":
                sub = "storage"
            module = _OUR_PREFIX + sub
        return super().find_class(module, name)


@contextlib.contextmanager
def reference_module_names():
    """While active, the metadata classes pickle under the reference's module paths."""
    import importlib
    installed, renamed = [], []
    try:
        for sub, names in _CLASSES.items():
            ours = importlib.import_module(_OUR_PREFIX + sub)
            ref_name = _REF_PREFIX + sub
            if ref_name not in sys.modules:
                # also provide the parent packages so that pickle's import succeeds
                parts = ref_name.split(".")
                for i in range(1, len(parts)):
                    pkg = ".".join(parts[:i])
                    if pkg not in sys.modules:
                        sys.modules[pkg] = types.ModuleType(pkg)
                        installed.append(pkg)
                shim = types.ModuleType(ref_name)
                for n in names:
                    setattr(shim, n, getattr(ours, n))
                sys.modules[ref_name] = shim
                installed.append(ref_name)
            else:
                continue   # the real reference is importable: keep our own names
            for n in names:
                cls = getattr(ours, n)
                renamed.append((cls, cls.__module__))
                cls.__module__ = ref_name
        yield
    finally:
        for cls, mod in renamed:
            cls.__module__ = mod
        for name in installed:
            sys.modules.pop(name, None)
