"""Run test functions written for ``hyper_parallel`` against this package on CPU ranks.

A migration aid: the torch tests of the reference project (``tests/torch/**``) are plain functions that
initialise ``torch.distributed`` on NPUs and assert on DTensors.  This module rewrites such a file on
the fly -- package name, ``"npu"`` device strings and ``.npu()`` calls, the HCCL backend name, the
``torch_npu`` import -- and runs one of its functions, or all of them, on ``gloo`` ranks:

    python -m hyper_parallel_b200.utils.reference_compat --root <checkout of the reference> \\
        tests/torch/shard/submesh.py [test_function] [--world 8]

Helper modules the tests import (``tests.torch.utils``, ``tests.torch.common_net``,
``tests.torch.shard.utils``, ``tests.torch.hsdp.hsdp_test_common``) are rewritten the same way, with
``init_dist`` replaced by a gloo initialisation.  Nothing of the reference is imported as a package:
only the named files are read.  Exit status 0 when every function passed.

Known differences that make a reference test fail here on purpose: ``distribute_tensor`` refuses
dimensions that do not divide evenly (the reference slices with a floored size), a placement list
longer than the mesh may only be padded with ``Replicate()``, and ``squeeze`` of a dim whose size is
not 1 is the identity as in torch (the reference raises).
"""
from __future__ import annotations

import argparse
import importlib
import os
import re
import socket
import sys
import tempfile
import traceback
from typing import List

_HELPERS = ("tests/torch/common_net.py", "tests/torch/hsdp/hsdp_test_common.py", "tests/torch/shard/utils.py",
            "tests/torch/shard/base_shard.py")
_INIT_DIST = ("import torch.distributed as dist\n\n\ndef init_dist():\n    if not dist.is_initialized():\n"
              "        dist.init_process_group('gloo')\n    return dist.get_rank(), 0\n\n\n"
              "def torchrun_case(*args, **kwargs):\n    raise RuntimeError('launcher files are not run; name the worker file')\n")
_MARK_UTILS = "def arg_mark(*args, **kwargs):\n    return lambda fn: fn\n"


def rewrite(source: str, package: str = "hyper_parallel_b200") -> str:
    """The text of a reference test file with this package's name and CPU devices."""
    s = re.sub(r"\bhyper_parallel\b(?!_b200)", package, source)
    if "torch_npu.npu_fusion_attention" in s:
        # the fused-attention operator of the NPU extension has a same-named counterpart here
        s = s.replace("torch_npu.npu_fusion_attention", "_hpb_fa.npu_fusion_attention")
        s = re.sub(r"^(\s*)import torch_npu.*$", rf"\1from {package}.ops import flash_attention_score as _hpb_fa", s,
                   count=1, flags=re.M)
    s = re.sub(r"^\s*import torch_npu.*$", "", s, flags=re.M)
    s = s.replace(".npu()", ".cpu()").replace('"npu"', '"cpu"').replace("'npu'", "'cpu'")
    s = s.replace("torch.npu.get_rng_state()", "torch.get_rng_state()")
    s = re.sub(r"torch\.npu\.current_device\(\)", "0", s)
    s = s.replace("npu:", "cpu:")
    s = re.sub(r"torch\.npu\.\w+\([^)]*\)", "None", s)
    return s.replace('"hccl"', '"gloo"')


def list_test_functions(path: str) -> List[str]:
    with open(path, encoding="utf-8") as f:
        return re.findall(r"^def (test_\w+)\(", f.read(), flags=re.M)


def _generate(root: str, rel: str, out_root: str) -> str:
    out = os.path.join(out_root, rel)
    os.makedirs(os.path.dirname(out), exist_ok=True)
    with open(os.path.join(root, rel), encoding="utf-8") as f:
        text = rewrite(f.read())
    with open(out, "w", encoding="utf-8") as f:
        f.write(text)
    return out


def prepare(root: str, rel: str, out_root: str) -> str:
    """Write the rewritten test file and its helper modules under ``out_root``; returns the file's path."""
    for helper in _HELPERS:
        if os.path.exists(os.path.join(root, helper)):
            _generate(root, helper, out_root)
    parts = rel.split("/")[:-1]
    for i in range(1, len(parts) + 1):
        d = os.path.join(out_root, *parts[:i])
        os.makedirs(d, exist_ok=True)
        open(os.path.join(d, "__init__.py"), "a").close()
    for d in ("tests", "tests/torch", "tests/torch/hsdp", "tests/torch/shard"):
        os.makedirs(os.path.join(out_root, d), exist_ok=True)
        open(os.path.join(out_root, d, "__init__.py"), "a").close()
    with open(os.path.join(out_root, "tests/torch/utils.py"), "w", encoding="utf-8") as f:
        f.write(_INIT_DIST)
    os.makedirs(os.path.join(out_root, "tests/common"), exist_ok=True)
    open(os.path.join(out_root, "tests/common/__init__.py"), "a").close()
    with open(os.path.join(out_root, "tests/common/mark_utils.py"), "w", encoding="utf-8") as f:
        f.write(_MARK_UTILS)
    # siblings of the test file, for its relative imports
    folder = os.path.dirname(rel)
    for name in sorted(os.listdir(os.path.join(root, folder))):
        if name.endswith(".py") and name != "__init__.py":
            _generate(root, os.path.join(folder, name), out_root)
    return _generate(root, rel, out_root)


def _worker(rank: int, world: int, port: int, out_root: str, path: str, fn: str, errq) -> None:
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    sys.path.insert(0, out_root)
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        real_init = dist.init_process_group
        # helpers of the tests initialise the default group themselves, unconditionally
        dist.init_process_group = lambda *a, **k: None if dist.is_initialized() else real_init(*a, **k)
        # imported under its package path so that relative imports of sibling files resolve
        name = os.path.relpath(path, out_root)[:-3].replace(os.sep, ".")
        module = importlib.import_module(name)
        getattr(module, fn)()
        if dist.is_initialized():           # some tests destroy the process group themselves
            dist.barrier()
    except Exception:  # noqa: BLE001  (reported to the parent, then re-raised for the exit code)
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_function(out_root: str, path: str, fn: str, world: int, timeout: float = 600.0):
    """Run ``fn`` of the rewritten file on ``world`` gloo ranks; returns ``(passed, first traceback)``."""
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out_root, path, fn, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    for p in procs:
        if p.is_alive():
            p.kill()
    first = None
    while not errq.empty():
        rank, tb = errq.get()
        first = first or f"rank {rank}:\n{tb}"
    ok = all(p.exitcode == 0 for p in procs)
    return ok, (first if not ok else None)


def run_unittest_file(out_root: str, path: str) -> int:
    """Files made of ``unittest.TestCase`` classes (pure-Python unit tests, no ranks): run them in this
    process; returns the number of failures and errors."""
    import importlib
    import unittest
    sys.path.insert(0, out_root)
    module = importlib.import_module(os.path.relpath(path, out_root)[:-3].replace(os.sep, "."))
    suite = unittest.defaultTestLoader.loadTestsFromModule(module)
    result = unittest.TextTestRunner(verbosity=1).run(suite)
    return len(result.failures) + len(result.errors)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--root", required=True, help="checkout of the reference project (the folder holding tests/)")
    ap.add_argument("file", help="test file relative to --root, e.g. tests/torch/shard/submesh.py")
    ap.add_argument("function", nargs="?", help="one test function (default: every test_* of the file)")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--timeout", type=float, default=600.0)
    ns = ap.parse_args(argv)
    failed = 0
    with tempfile.TemporaryDirectory(prefix="hpb_compat_") as out_root:
        path = prepare(ns.root, ns.file, out_root)
        functions = [ns.function] if ns.function else list_test_functions(os.path.join(ns.root, ns.file))
        if not functions:                                   # unittest classes only
            return 1 if run_unittest_file(out_root, path) else 0
        for fn in functions:
            ok, tb = run_function(out_root, path, fn, ns.world, ns.timeout)
            print(("PASS " if ok else "FAIL ") + f"{ns.file}::{fn}", flush=True)
            if not ok:
                failed += 1
                print("    " + "\n    ".join((tb or "no traceback (timeout or a crash)").strip().splitlines()[-6:]), flush=True)
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
