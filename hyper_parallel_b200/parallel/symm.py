"""Symmetric memory over NVLink / NVSwitch: one buffer per rank, mapped into every peer.

The reference has no counterpart (its communication is ``torch.distributed`` only,
hyper_parallel/platform/torch/platform.py:176-424); this is the layer the fused compute+collective
kernels are built on.

``SymmetricMemory(group, nbytes)`` allocates ``nbytes`` on every rank of ``group`` plus a
signal pad and maps all peers.  It exposes ``ptrs`` / ``pad_ptrs`` (ctypes arrays of N device
pointers, own rank included), ``tensor(dtype, numel, offset)`` views of the local buffer, and
``barrier()``.  Epochs of the signal pads only grow, so flags never need clearing.

Two transports:

* ``vmm`` (default): CUDA virtual-memory-management allocations shared through POSIX file
  descriptors (the descriptors travel over Unix-domain datagram sockets between the ranks of one
  node).  With ``multicast=True`` on a machine whose NVSwitch supports it, the ranks' buffers are
  also bound to one NVLink multicast object and ``mc_base`` is the address of its mapping:
  ``multimem.ld_reduce`` there returns the sum over all ranks, reduced inside the switch.
  ``HPB_NVLS=0`` switches multicast off.
* ``ipc`` (``HPB_SYMM=ipc``, and the fallback when the VMM path is unavailable): ``cudaMalloc`` +
  CUDA IPC handles exchanged through the process group; no multicast.

Ranks are processes of one node (one process per GPU).  With a single rank nothing is shared
and the object degenerates to a plain local buffer.
"""
from __future__ import annotations

import array
import ctypes
import os
import socket
import uuid
from typing import List, Optional

import torch
import torch.distributed as dist

from ..collectives import cc
from ..ops import native

_PAD_BYTES = 4096          # 64 slots x 16 ranks x 4 B
_CANARY_BYTES = 256        # guard words in front of the data region and behind the signal pad
_CANARY = 0x5A
DEFAULT_WAIT_NS = 2_000_000_000

# signal-pad slots with a fixed meaning (every kernel family uses its own slots of its own region)
SLOT_SHARD_VERSION = 4     # "my parameter shard has reached version v" (HSDP buffers)
SLOT_BARRIER = 63


class _Holder:
    """Exposes a raw device allocation to torch through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 2, "strides": None}


_bound = False


def _bind():
    global _bound
    lib = native.lib()
    if _bound:
        return lib
    vp, ci, sz, ull = ctypes.c_void_p, ctypes.c_int, ctypes.c_size_t, ctypes.c_ulonglong
    pvp, pull, pci = ctypes.POINTER(vp), ctypes.POINTER(ull), ctypes.POINTER(ci)
    lib.hpb_symm_alloc.argtypes = [pvp, sz]
    lib.hpb_symm_alloc.restype = ci
    lib.hpb_symm_free.argtypes = [vp]
    lib.hpb_symm_export.argtypes = [vp, vp]
    lib.hpb_symm_import.argtypes = [vp, pvp]
    lib.hpb_symm_unmap.argtypes = [vp]
    lib.hpb_symm_barrier.argtypes = [pvp, ci, ci, ci, ctypes.c_uint, ull, ci, vp, vp]
    lib.hpb_symm_barrier.restype = ci
    lib.hpb_symm_signal.argtypes = [pvp, ci, ci, ci, ctypes.c_uint, vp]
    lib.hpb_symm_signal.restype = ci
    lib.hpb_vmm_supported.argtypes = [pci, pci]
    lib.hpb_vmm_granularity.argtypes = [ci, ci, ctypes.POINTER(sz)]
    lib.hpb_vmm_alloc.argtypes = [sz, sz, pvp, pull, pci]
    lib.hpb_vmm_import.argtypes = [ci, sz, sz, pvp, pull]
    lib.hpb_vmm_unmap.argtypes = [vp, sz, ull]
    lib.hpb_mc_create.argtypes = [ci, sz, pull, pci]
    lib.hpb_mc_import.argtypes = [ci, pull]
    lib.hpb_mc_add_device.argtypes = [ull]
    lib.hpb_mc_bind_map.argtypes = [ull, ull, sz, sz, pvp]
    lib.hpb_mc_unbind.argtypes = [ull, vp, sz]
    for name in ("hpb_vmm_supported", "hpb_vmm_granularity", "hpb_vmm_alloc", "hpb_vmm_import", "hpb_vmm_unmap",
                 "hpb_mc_create", "hpb_mc_import", "hpb_mc_add_device", "hpb_mc_bind_map", "hpb_mc_unbind",
                 "hpb_symm_free", "hpb_symm_export", "hpb_symm_import", "hpb_symm_unmap"):
        getattr(lib, name).restype = ci
    _bound = True
    return lib


def nvls_enabled() -> bool:
    return os.environ.get("HPB_NVLS", "1") != "0"


_NOTES: List[str] = []        # why a VMM / multicast set-up step fell back (first few, for diagnostics)


def _note(msg: str) -> None:
    if len(_NOTES) < 16:
        _NOTES.append(msg)
    if os.environ.get("HPB_SYMM_DEBUG", "0") == "1":
        print(f"[hpb symm] {msg}", flush=True)


def _all_agree(group, ok: bool) -> bool:
    """True only when every rank of the group reports success (keeps the ranks on one code path)."""
    flags = [None] * cc.group_size(group)
    dist.all_gather_object(flags, bool(ok), group=group)
    return all(flags)


class _FdExchange:
    """Pass file descriptors between the ranks of one node over abstract Unix datagram sockets."""

    def __init__(self, group):
        self.group = group
        self.world = cc.group_size(group)
        self.rank = cc.group_rank(group)
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_DGRAM)
        self.name = f"\0hpb-symm-{uuid.uuid4().hex}"
        self.sock.bind(self.name)
        self.sock.settimeout(60.0)
        names = [None] * self.world
        dist.all_gather_object(names, self.name, group=group)      # every socket is bound after this
        self.names = names

    def _send(self, fd: int, dst: int) -> None:
        # sendmsg with an explicit address: the socket is unconnected (socket.send_fds drops the address)
        self.sock.sendmsg([self.rank.to_bytes(4, "little")],
                          [(socket.SOL_SOCKET, socket.SCM_RIGHTS, array.array("i", [fd]))], 0, self.names[dst])

    def all_to_all(self, fd: int) -> List[int]:
        """Every rank sends ``fd`` to every peer; returns the received descriptors by source rank."""
        for r in range(self.world):
            if r != self.rank:
                self._send(fd, r)
        out = [-1] * self.world
        for _ in range(self.world - 1):
            msg, fds, _flags, _addr = socket.recv_fds(self.sock, 16, 1)
            out[int.from_bytes(msg[:4], "little")] = fds[0]
        return out

    def broadcast(self, fd: Optional[int], src: int = 0) -> int:
        """Rank ``src`` sends ``fd`` to everybody else; the others return their copy."""
        if self.rank == src:
            for r in range(self.world):
                if r != src:
                    self._send(fd, r)
            return fd
        _msg, fds, _flags, _addr = socket.recv_fds(self.sock, 16, 1)
        return fds[0]

    def close(self) -> None:
        self.sock.close()


class SymmetricMemory:
    def __init__(self, group, nbytes: int, device: Optional[torch.device] = None, multicast: bool = False):
        self.lib = _bind()
        self.group = group
        self.world = cc.group_size(group)
        self.rank = cc.group_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        self._mapped: List[int] = []          # ipc: peer mappings
        self._vmm_maps: List[tuple] = []      # vmm: (ptr, bytes, handle) of every mapping, own first
        self._mc = None                       # (mc handle, mc ptr)
        self.mc_base: Optional[int] = None    # multicast address of the buffers (None: no multicast)
        self.transport = "ipc"
        # [canary | data (nbytes) | signal pad | canary]; every pointer handed out is relative to the data
        total = _CANARY_BYTES + self.nbytes + _PAD_BYTES + _CANARY_BYTES
        want_vmm = os.environ.get("HPB_SYMM", "vmm") != "ipc" and self.world > 1
        peer_bases = None
        if want_vmm:
            peer_bases = self._init_vmm(total, multicast and nvls_enabled())
        if peer_bases is None:
            peer_bases = self._init_ipc(total)
        self._holder = _Holder(self._base, self._total)
        raw = torch.as_tensor(self._holder, device=self.device)
        self._guards = (raw[:_CANARY_BYTES], raw[_CANARY_BYTES + self.nbytes + _PAD_BYTES:
                                                 2 * _CANARY_BYTES + self.nbytes + _PAD_BYTES])
        for g in self._guards:
            g.fill_(_CANARY)
        self._bytes = raw[_CANARY_BYTES:_CANARY_BYTES + self.nbytes + _PAD_BYTES]
        peer_bases = [b + _CANARY_BYTES for b in peer_bases]
        if self.mc_base is not None:
            self.mc_base += _CANARY_BYTES
        arr = ctypes.c_void_p * max(self.world, 1)
        self.ptrs = arr(*peer_bases)
        self.pad_ptrs = arr(*[b + self.nbytes for b in peer_bases])
        self.peer_bases = peer_bases
        self._epoch = 0
        self.done_counter = torch.zeros(4, dtype=torch.int32, device=self.device)
        if self.world > 1:
            dist.barrier(group=group)

    # ------------------------------------------------------------ transports --
    def _init_ipc(self, total: int) -> List[int]:
        base = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            native.check(self.lib.hpb_symm_alloc(ctypes.byref(base), total), "hpb_symm_alloc")
        self._base, self._total = base.value, total
        peer_bases = [self._base] * self.world
        if self.world > 1:
            hbytes = self.lib.hpb_symm_handle_bytes()
            buf = ctypes.create_string_buffer(hbytes)
            native.check(self.lib.hpb_symm_export(self._base, buf), "hpb_symm_export")
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(buf.raw), group=self.group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                out = ctypes.c_void_p()
                hb = ctypes.create_string_buffer(h, len(h))
                with torch.cuda.device(self.device):
                    native.check(self.lib.hpb_symm_import(hb, ctypes.byref(out)), "hpb_symm_import")
                peer_bases[r] = out.value
                self._mapped.append(out.value)
        self.transport = "ipc"
        return peer_bases

    def _init_vmm(self, total: int, multicast: bool) -> Optional[List[int]]:
        """VMM allocation shared through file descriptors (+ multicast).  Returns ``None`` when any
        rank cannot do it; nothing stays allocated in that case."""
        lib = self.lib
        ok = True
        gran = ctypes.c_size_t(0)
        with torch.cuda.device(self.device):
            vmm, mc = ctypes.c_int(0), ctypes.c_int(0)
            rc = lib.hpb_vmm_supported(ctypes.byref(vmm), ctypes.byref(mc))
            ok = rc == 0 and vmm.value == 1
            if not ok:
                _note(f"vmm_supported rc={rc} vmm={vmm.value} multicast={mc.value}")
            use_mc = multicast and mc.value == 1
            flags = [None] * self.world
            dist.all_gather_object(flags, (ok, use_mc), group=self.group)
            if not all(f[0] for f in flags):
                return None
            use_mc = all(f[1] for f in flags)
            rc = lib.hpb_vmm_granularity(self.world, int(use_mc), ctypes.byref(gran))
            ok = rc == 0
            if not ok:
                _note(f"vmm_granularity rc={rc}")
            if not _all_agree(self.group, ok):
                return None
            g = gran.value
            size = (total + g - 1) // g * g
            ptr, handle, fd = ctypes.c_void_p(), ctypes.c_ulonglong(0), ctypes.c_int(-1)
            rc = lib.hpb_vmm_alloc(size, g, ctypes.byref(ptr), ctypes.byref(handle), ctypes.byref(fd))
            if rc == 0:
                self._vmm_maps.append((ptr.value, size, handle.value))
            else:
                _note(f"vmm_alloc({size}, gran {g}) rc={rc}")
            if not _all_agree(self.group, rc == 0):
                self._release_vmm()
                return None
            ex = _FdExchange(self.group)
            peer_bases = [ptr.value] * self.world
            try:
                fds = ex.all_to_all(fd.value)
                rc = 0
                for r, pfd in enumerate(fds):
                    if r == self.rank:
                        continue
                    p, h = ctypes.c_void_p(), ctypes.c_ulonglong(0)
                    rc = rc or lib.hpb_vmm_import(pfd, size, g, ctypes.byref(p), ctypes.byref(h))
                    os.close(pfd)
                    if rc == 0:
                        self._vmm_maps.append((p.value, size, h.value))
                        peer_bases[r] = p.value
            except OSError as e:
                _note(f"fd exchange failed: {e!r}")
                rc = -1
            if rc != 0:
                _note(f"vmm_import rc={rc}")
            if not _all_agree(self.group, rc == 0):
                os.close(fd.value)
                ex.close()
                self._release_vmm()
                return None
            os.close(fd.value)
            if use_mc:
                self._init_multicast(ex, size, g, handle.value)
            ex.close()
        self._base, self._total = ptr.value, size
        self.transport = "vmm"
        return peer_bases

    def _init_multicast(self, ex: _FdExchange, size: int, gran: int, mem_handle: int) -> None:
        """Bind every rank's allocation to one multicast object (NVLS).  On failure the object keeps
        working without ``mc_base``."""
        lib = self.lib
        mc, fd = ctypes.c_ulonglong(0), ctypes.c_int(-1)
        rc = 0
        if self.rank == 0:
            rc = lib.hpb_mc_create(self.world, size, ctypes.byref(mc), ctypes.byref(fd))
        if rc != 0:
            _note(f"mc_create rc={rc}")
        ok0 = [rc == 0]
        dist.broadcast_object_list(ok0, src=dist.get_global_rank(self.group, 0) if self.group is not None else 0,
                                   group=self.group)
        if not ok0[0]:
            return
        try:
            got = ex.broadcast(fd.value if self.rank == 0 else None, 0)
            if self.rank != 0:
                rc = lib.hpb_mc_import(got, ctypes.byref(mc))
            os.close(got)
        except OSError as e:
            _note(f"multicast fd exchange failed: {e!r}")
            rc = -1
        if rc == 0:
            rc = lib.hpb_mc_add_device(mc.value)
        if rc != 0:
            _note(f"mc_import / mc_add_device rc={rc}")
        if not _all_agree(self.group, rc == 0):     # also the barrier "every device was added"
            return
        mc_ptr = ctypes.c_void_p()
        rc = lib.hpb_mc_bind_map(mc.value, mem_handle, size, gran, ctypes.byref(mc_ptr))
        if rc == 0:
            self._mc = (mc.value, mc_ptr.value, size)
        else:
            _note(f"mc_bind_map rc={rc}")
        if _all_agree(self.group, rc == 0):
            self.mc_base = mc_ptr.value
        elif self._mc is not None:
            lib.hpb_mc_unbind(*self._mc[:2], size)
            self._mc = None

    def _release_vmm(self) -> None:
        if self._mc is not None:
            self.lib.hpb_mc_unbind(self._mc[0], self._mc[1], self._mc[2])
            self._mc = None
            self.mc_base = None
        for p, size, h in reversed(self._vmm_maps):
            self.lib.hpb_vmm_unmap(p, size, h)
        self._vmm_maps = []

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
    def barrier(self, slot: int = SLOT_BARRIER, limit_ns: int = DEFAULT_WAIT_NS, signal: bool = True,
                epoch: Optional[int] = None) -> None:
        """Device-side barrier over the group on the current stream (bounded wait)."""
        ep = self.next_epoch() if epoch is None else epoch
        st = native.status_word(self.device)
        native.check(self.lib.hpb_symm_barrier(self.pad_ptrs, self.rank, self.world, slot, ep, limit_ns,
                                               int(signal), st.data_ptr(), native.stream(self.device)),
                     "hpb_symm_barrier")

    def signal(self, slot: int, value: int) -> None:
        """Publish ``value`` on ``slot`` of every peer's pad (current stream, no wait)."""
        if not getattr(self, "_base", 0):
            raise RuntimeError("symmetric memory region is closed")
        native.check(self.lib.hpb_symm_signal(self.pad_ptrs, self.rank, self.world, slot, value,
                                              native.stream(self.device)), "hpb_symm_signal")

    def check_canaries(self) -> None:
        """Raise if anything wrote in front of the data region or behind the signal pad of the LOCAL
        buffer (a peer's or an own kernel running past the end of a symmetric region).  Synchronises."""
        for name, g in zip(("front", "back"), self._guards):
            bad = (g != _CANARY).nonzero()
            if bad.numel():
                raise RuntimeError(f"symmetric memory guard ({name}) overwritten at byte {int(bad[0])} of "
                                   f"{_CANARY_BYTES} on rank {self.rank}")

    def reset_counters(self) -> None:
        """Zero the last-CTA counters (after a kernel reported a bounded-wait expiry they may be off)."""
        self.done_counter.zero_()

    def close(self) -> None:
        """Unmap the peers and free the local buffer.  Collective: every rank of the group calls it.
        The device is synchronised and the group meets before anything is unmapped, so no peer kernel
        can still be reading this rank's buffer, and all ranks unmap before any of them frees."""
        if not getattr(self, "_base", 0):
            return
        with torch.cuda.device(self.device):
            torch.cuda.synchronize(self.device)
            if self.world > 1 and dist.is_initialized():
                dist.barrier(group=self.group)
            self._bytes = None
            self._guards = ()
            if self.transport == "vmm":
                own = self._vmm_maps[0]
                if self._mc is not None:
                    self.lib.hpb_mc_unbind(self._mc[0], self._mc[1], self._mc[2])
                    self._mc, self.mc_base = None, None
                for p, size, h in reversed(self._vmm_maps[1:]):
                    self.lib.hpb_vmm_unmap(p, size, h)
                self._vmm_maps = [own]
                if self.world > 1 and dist.is_initialized():
                    dist.barrier(group=self.group)
                self.lib.hpb_vmm_unmap(*own)
                self._vmm_maps = []
            else:
                for p in self._mapped:
                    self.lib.hpb_symm_unmap(p)
                self._mapped = []
                if self.world > 1 and dist.is_initialized():
                    dist.barrier(group=self.group)
                self.lib.hpb_symm_free(self._base)
            self._base = 0
