"""ctypes binding to ``libhpb200.so`` (the hand-written sm_100a kernels).

Every launcher is an ``extern "C"`` function taking raw device pointers and a
CUDA stream; this module turns ``torch.Tensor`` arguments into those.  On a
machine with a GPU the library MUST be present: a missing or unloadable library
raises instead of silently falling back to eager PyTorch.
"""
from __future__ import annotations

import ctypes
import os
import threading
from typing import Optional

import torch

from . import build as _build

_lock = threading.Lock()
_lib: Optional[ctypes.CDLL] = None
_status = {}  # device index -> int32[2] tensor written by kernels on bounded-wait expiry
_sm_count = {}

c_void_p, c_int, c_int64, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

_SIGNATURES = {
    "hpb_gemm_bf16": [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64, c_int,
                      c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "hpb_gemm2_bf16": [c_void_p, c_int, c_int64, c_void_p, c_int, c_int64, c_void_p, c_int64, c_int,
                       c_int, c_int, c_int, c_int, c_void_p, c_int, c_void_p],
    "hpb_rmsnorm_fwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int,
                        c_float, c_void_p],
    "hpb_rmsnorm_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_void_p, c_int, c_int, c_int64, c_int, c_void_p],
    "hpb_swiglu_fwd": [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p],
    "hpb_swiglu_bwd": [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p],
    "hpb_rope": [c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int64, c_float, c_int, c_int,
                 c_void_p],
    "hpb_rope_table": [c_void_p, c_int, c_int, c_float, c_void_p],
    "hpb_rope_vec": [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int64, c_int, c_int, c_void_p],
    "hpb_rope_vec_strided": [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int64, c_int64, c_int, c_int,
                             c_void_p],
    "hpb_embedding_fwd": [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p],
    "hpb_embedding_bwd": [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p],
    "hpb_cross_entropy": [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int64, c_float, c_void_p],
    "hpb_adamw": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_float, c_float,
                  c_float, c_float, c_float, c_int, c_float, c_int, c_void_p],
}


def available() -> bool:
    """True when the compiled library exists on disk (it may still need a GPU to run)."""
    return _build.LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    """Load (once) and return the native library; raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            # HPB_DEBUG_BOUNDS=1: the flavour whose kernels check their indices (status code 7)
            debug = os.environ.get("HPB_DEBUG_BOUNDS", "0") == "1"
            path = _build.lib_path(debug)
            if debug and not path.exists():
                _build.build(debug_bounds=True)
            if not path.exists():
                if os.environ.get("HPB_BUILD_ON_IMPORT", "0") == "1":
                    _build.build()
                else:
                    raise RuntimeError(
                        f"{path} is missing: run `python -m hyper_parallel_b200.ops.build` "
                        "(the CUDA kernels are required on a GPU machine)")
            handle = ctypes.CDLL(str(path), mode=ctypes.RTLD_GLOBAL)
            for name, argtypes in _SIGNATURES.items():
                if hasattr(handle, name):
                    fn = getattr(handle, name)
                    fn.argtypes = argtypes
                    fn.restype = c_int
            _lib = handle
    return _lib


def bind(name: str, argtypes, restype=c_int):
    """Declare the signature of an additional exported symbol and return it."""
    fn = getattr(lib(), name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def use_native(t: torch.Tensor) -> bool:
    """Kernels run for CUDA tensors; CPU tensors take the PyTorch reference path."""
    return t.is_cuda


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def stream(device=None):
    return torch.cuda.current_stream(device).cuda_stream


_sm_reserve = 0


def reserve_sms(n: int) -> None:
    """Leave ``n`` SMs (an even number: the GEMMs run CTA pairs) out of the grids of the persistent
    kernels.  A persistent kernel strides its tiles over ``gridDim`` CTAs, one per SM; when another
    kernel holds an SM for a long time -- an NCCL receive posted ahead that spins until its peer
    sends, inside a pipeline stage -- the CTA meant for that SM starts only when another CTA has
    finished, and the kernel takes up to twice as long.  Reserving the SMs that such kernels take
    costs n / 148 of the peak and removes the tail.  ``HPB_RESERVE_SMS`` sets the initial value."""
    global _sm_reserve
    _sm_reserve = max(0, int(n)) // 2 * 2


def sm_count(device) -> int:
    """SMs that a persistent kernel may fill on ``device`` (all of them minus ``reserve_sms``)."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    n = _sm_count.get(idx)
    if n is None:
        n = torch.cuda.get_device_properties(idx).multi_processor_count
        _sm_count[idx] = n
    return max(n - _sm_reserve, 2)


reserve_sms(int(os.environ.get("HPB_RESERVE_SMS", "0")))


def status_word(device) -> torch.Tensor:
    """Per-device int32[2] that kernels write when a bounded wait expires."""
    idx = torch.device(device).index
    if idx is None:
        idx = torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(2, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


_STATUS_TEXT = {
    1: "timeout waiting for a TMA stage (full barrier)",
    2: "timeout waiting for a free smem stage (empty barrier)",
    3: "timeout waiting for an accumulator (tmem full)",
    4: "timeout waiting for accumulator drain (tmem empty)",
    5: "timeout waiting for a peer flag",
    6: "bad argument seen on device",
    7: "index out of bounds caught by a debug-build check (the access was skipped)",
}


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel recorded a bounded-wait expiry."""
    for idx, t in list(_status.items()):
        if device is not None and torch.device(device).index not in (None, idx):
            continue
        code, detail = t.tolist()
        if code != 0:
            t.zero_()
            raise RuntimeError(
                f"hyper_parallel_b200 kernel error on cuda:{idx}: "
                f"{_STATUS_TEXT.get(code, code)} (detail={detail})")


launch_count = 0   # number of native launcher calls made by this process


def check(rc: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
