"""Symmetric memory over NVLink / NVSwitch: one buffer per rank, mapped into every peer.

The reference has no counterpart (its communication is ``torch.distributed`` only,
hyper_parallel/platform/torch/platform.py:176-424); this is the layer the fused compute+collective
kernels are built on.

``SymmetricMemory(group, nbytes)`` allocates ``nbytes`` on every rank of ``group`` plus a
signal pad, exchanges CUDA IPC handles through the process group and maps all peers.  It
exposes ``ptrs`` / ``pad_ptrs`` (ctypes arrays of N device pointers, own rank included),
``tensor(dtype, numel, offset)`` views of the local buffer, and ``barrier()``.  Epochs of the
signal pads only grow, so flags never need clearing.

Ranks are processes of one node (one process per GPU).  With a single rank no IPC is needed
and the object degenerates to a plain local buffer.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..collectives import cc
from ..ops import native

_PAD_BYTES = 4096          # 64 slots x 16 ranks x 4 B
DEFAULT_WAIT_NS = 2_000_000_000


class _Holder:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


def _bind():
    lib = native.lib()
    vp, ci = ctypes.c_void_p, ctypes.c_int
    lib.hpb_symm_alloc.argtypes = [ctypes.POINTER(vp), ctypes.c_size_t]
    lib.hpb_symm_alloc.restype = ci
    lib.hpb_symm_free.argtypes = [vp]
    lib.hpb_symm_export.argtypes = [vp, vp]
    lib.hpb_symm_import.argtypes = [vp, ctypes.POINTER(vp)]
    lib.hpb_symm_unmap.argtypes = [vp]
    lib.hpb_symm_barrier.argtypes = [ctypes.POINTER(vp), ci, ci, ci, ctypes.c_uint, ctypes.c_ulonglong,
                                     ci, vp, vp]
    lib.hpb_symm_barrier.restype = ci
    return lib


class SymmetricMemory:
    def __init__(self, group, nbytes: int, device: Optional[torch.device] = None):
        self.lib = _bind()
        self.group = group
        self.world = cc.group_size(group)
        self.rank = cc.group_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        total = self.nbytes + _PAD_BYTES
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            native.check(self.lib.hpb_symm_alloc(ctypes.byref(base), total), "hpb_symm_alloc")
        self._base = base.value
        self._holder = _Holder(self._base, total)
        self._bytes = torch.as_tensor(self._holder, device=self.device)
        self._mapped: List[int] = []
        peer_bases = [self._base] * self.world
        if self.world > 1:
            hbytes = self.lib.hpb_symm_handle_bytes()
            buf = ctypes.create_string_buffer(hbytes)
            native.check(self.lib.hpb_symm_export(self._base, buf), "hpb_symm_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(buf.raw), group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                out = ctypes.c_void_p()
                hb = ctypes.create_string_buffer(h, len(h))
                with torch.cuda.device(self.device):
                    native.check(self.lib.hpb_symm_import(hb, ctypes.byref(out)), "hpb_symm_import")
                peer_bases[r] = out.value
                self._mapped.append(out.value)
        arr = ctypes.c_void_p * max(self.world, 1)
        self.ptrs = arr(*peer_bases)
        self.pad_ptrs = arr(*[b + self.nbytes for b in peer_bases])
        self.peer_bases = peer_bases
        self._epoch = 0
        self.done_counter = torch.zeros(4, dtype=torch.int32, device=self.device)
        if self.world > 1:
            dist.barrier(group=group)

    # ------------------------------------------------------------------ views --
    def tensor(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        """A view of the LOCAL buffer."""
        nb = numel * torch.empty((), dtype=dtype).element_size()
        if byte_offset % 16 or byte_offset + nb > self.nbytes:
            raise ValueError(f"view [{byte_offset}, {byte_offset + nb}) outside the buffer or unaligned")
        return self._bytes[byte_offset:byte_offset + nb].view(dtype)

    def ptr_table(self, byte_offset: int = 0):
        """ctypes array of the N peers' device pointers at ``byte_offset``."""
        arr = ctypes.c_void_p * max(self.world, 1)
        return arr(*[b + byte_offset for b in self.peer_bases])

    def next_epoch(self) -> int:
        self._epoch += 1
        return self._epoch

    # ---------------------------------------------------------------- barrier --
    def barrier(self, slot: int = 63, limit_ns: int = DEFAULT_WAIT_NS, signal: bool = True,
                epoch: Optional[int] = None) -> None:
        """Device-side barrier over the group on the current stream (bounded wait)."""
        ep = self.next_epoch() if epoch is None else epoch
        st = native.status_word(self.device)
        native.check(self.lib.hpb_symm_barrier(self.pad_ptrs, self.rank, self.world, slot, ep, limit_ns,
                                               int(signal), st.data_ptr(), native.stream(self.device)),
                     "hpb_symm_barrier")

    def close(self) -> None:
        for p in self._mapped:
            self.lib.hpb_symm_unmap(p)
        self._mapped = []
        if self._base:
            self._bytes = None
            self.lib.hpb_symm_free(self._base)
            self._base = 0
