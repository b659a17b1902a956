"""In-tree build of the sm_100a CUDA library ``libhpb200.so``.

The kernels are plain CUDA translation units with ``extern "C"`` launchers (no
torch headers), so a full rebuild takes seconds.  ``nvcc`` cross-compiles for
sm_100a without a GPU.  The shared object is written next to this file so that it
ships with the source tree; Python binds to it with ``ctypes``
(:mod:`hyper_parallel_b200.ops.native`).
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
BUILD_DIR = HERE / "build"
LIB_PATH = HERE / "libhpb200.so"
# debug flavour: every kernel compiled with -DHPB_DEBUG_BOUNDS (index checks that record status
# code 7 and skip the access); selected at run time with HPB_DEBUG_BOUNDS=1
DEBUG_BUILD_DIR = HERE / "build_dbg"
DEBUG_LIB_PATH = HERE / "libhpb200_dbg.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")
    return cand


def _digest(paths) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def sources():
    return sorted(CSRC.glob("*.cu"))


def lib_path(debug_bounds: bool = False) -> Path:
    return DEBUG_LIB_PATH if debug_bounds else LIB_PATH


def is_current(debug_bounds: bool = False) -> bool:
    stamp = (DEBUG_BUILD_DIR if debug_bounds else BUILD_DIR) / "stamp"
    if not lib_path(debug_bounds).exists() or not stamp.exists():
        return False
    return stamp.read_text().strip() == _digest(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) +
                                                list(CSRC.glob("*.h")))


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libhpb200.so`` (``debug_bounds``: the
    ``-DHPB_DEBUG_BOUNDS`` flavour ``libhpb200_dbg.so``)."""
    if not force and is_current(debug_bounds):
        return lib_path(debug_bounds)
    BUILD_DIR = DEBUG_BUILD_DIR if debug_bounds else globals()["BUILD_DIR"]
    LIB_PATH = lib_path(debug_bounds)
    extra = ["-DHPB_DEBUG_BOUNDS"] if debug_bounds else []
    BUILD_DIR.mkdir(exist_ok=True)
    nvcc = _nvcc()
    srcs = sources()
    log_lines = []

    def compile_one(src: Path) -> Path:
        obj = BUILD_DIR / (src.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log_lines.append(f"$ {' '.join(cmd)}\n{r.stdout}{r.stderr}")
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = [nvcc, "-shared", "-o", str(LIB_PATH), *map(str, objs), "-cudart", "static"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    (BUILD_DIR / "ptxas.log").write_text("\n".join(log_lines))
    (BUILD_DIR / "stamp").write_text(
        _digest(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))))
    if verbose:
        print("\n".join(log_lines))
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_bounds="--debug-bounds" in sys.argv)
    print(path)
