"""Symmetric device memory through the CUDA virtual-memory-management API (``csrc/sm100/symm_vmm.cu``): this framework's
own allocator for the buffers that peers read and write, selected with ``HG_SYMM_ALLOC=vmm``
(``parallel/fused_zero.py::SymmetricBuffer``; the default is ``torch.distributed._symmetric_memory``).

Per buffer, collectively over a single-node process group: every rank creates an exportable physical allocation, the
file descriptors travel between the ranks' processes over abstract-namespace Unix sockets (``SCM_RIGHTS``), every rank
imports its peers' allocations and maps all of them into its own address space.  What comes out is a list of device
pointers, one per rank, all valid on this GPU.
"""
from __future__ import annotations

import array
import ctypes
import os
import socket
from typing import List

import torch
import torch.distributed as dist

from ..ops import _lib

_SEQ = 0


def _bind(lib):
    if getattr(lib, "_vmm_bound", False):
        return
    c_ull, c_ll, c_int, c_void_p = ctypes.c_ulonglong, ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p
    lib.hg_vmm_padded_size.argtypes, lib.hg_vmm_padded_size.restype = [c_ll, c_int], c_ll
    lib.hg_vmm_create.argtypes, lib.hg_vmm_create.restype = [c_ll, c_int, ctypes.POINTER(c_ull), ctypes.POINTER(c_int)], c_int
    lib.hg_vmm_import.argtypes, lib.hg_vmm_import.restype = [c_int, ctypes.POINTER(c_ull)], c_int
    lib.hg_vmm_map.argtypes, lib.hg_vmm_map.restype = [ctypes.POINTER(c_ull), c_int, c_ll, c_int, ctypes.POINTER(c_void_p)], c_int
    lib.hg_vmm_unmap_release.argtypes, lib.hg_vmm_unmap_release.restype = [c_void_p, c_ll, c_ull], c_int
    lib._vmm_bound = True


class _DevicePointer:
    """Lets ``torch.as_tensor`` wrap a raw device pointer (no copy, no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _exchange_fds(fd: int, pg, tag: str) -> List[int]:
    """Every rank of ``pg`` sends its descriptor to every other rank; returns the received descriptors by group rank
    (``-1`` at this rank's own index).  Abstract-namespace sockets named after the job, the group and ``tag``."""
    t, me = dist.get_world_size(pg), dist.get_rank(pg)
    ranks = dist.get_process_group_ranks(pg)
    job = "%s_%s" % (os.environ.get("MASTER_PORT", "0"), "_".join(map(str, ranks)))
    name = lambda r: "\0hg_vmm_%s_%s_%d" % (job, tag, r)  # noqa: E731
    srv = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
    srv.settimeout(60.0)                         # a peer that failed before connecting ends the wait with an error
    srv.bind(name(me))
    srv.listen(t)
    dist.barrier(group=pg)                       # every listener exists before anybody connects
    for r in range(t):
        if r == me:
            continue
        c = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        c.connect(name(r))
        socket.send_fds(c, [me.to_bytes(4, "little")], [fd])
        c.close()
    got = [-1] * t
    for _ in range(t - 1):
        conn, _addr = srv.accept()
        msg, fds, _flags, _a = socket.recv_fds(conn, 4, 1)
        conn.close()
        got[int.from_bytes(msg, "little")] = fds[0]
    srv.close()
    return got


class VmmSymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``pg``, each rank's block mapped into every rank."""

    def __init__(self, nbytes: int, device: torch.device, pg):
        global _SEQ
        lib = _lib.load()
        _bind(lib)
        _SEQ += 1
        dev = device.index if device.index is not None else torch.cuda.current_device()
        t, me = dist.get_world_size(pg), dist.get_rank(pg)
        self.padded = int(lib.hg_vmm_padded_size(nbytes, dev))
        if self.padded <= 0:
            raise RuntimeError("hg_vmm_padded_size failed (%d)" % self.padded)
        h, fd = ctypes.c_ulonglong(0), ctypes.c_int(-1)
        _lib.check(lib.hg_vmm_create(self.padded, dev, ctypes.byref(h), ctypes.byref(fd)), "hg_vmm_create")
        fds = [-1] * t
        handles = (ctypes.c_ulonglong * t)()
        try:
            fds = _exchange_fds(fd.value, pg, "b%d" % _SEQ)
            for r in range(t):
                if r == me:
                    handles[r] = h.value
                else:
                    hr = ctypes.c_ulonglong(0)
                    _lib.check(lib.hg_vmm_import(fds[r], ctypes.byref(hr)), "hg_vmm_import")
                    handles[r] = hr.value
        finally:        # the descriptors are only needed for the import: none outlives this block, error or not
            for r, other in enumerate(fds):
                if r != me and other >= 0:
                    os.close(other)
            os.close(fd.value)
        ptrs = (ctypes.c_void_p * t)()
        _lib.check(lib.hg_vmm_map(handles, t, self.padded, dev, ptrs), "hg_vmm_map")
        self.ptrs = [int(p) for p in ptrs]
        self._handles = [int(x) for x in handles]
        self.nbytes = nbytes
        self.raw = torch.as_tensor(_DevicePointer(self.ptrs[me], nbytes), device=device)
        self.raw.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=pg)                   # every rank's block is mapped and zeroed before anyone uses a peer's

    def view(self, dtype: torch.dtype) -> torch.Tensor:
        return self.raw.view(dtype)

    def close(self):
        """Unmap every rank's block and drop the references.  The caller makes sure (a barrier after the last kernel)
        that no rank still touches the memory; buffers that live as long as the process are simply never closed."""
        lib = _lib.load()
        self.raw = None
        for p, h in zip(self.ptrs, self._handles):
            lib.hg_vmm_unmap_release(ctypes.c_void_p(p), self.padded, ctypes.c_ulonglong(h))
        self.ptrs, self._handles = [], []


def allocator() -> str:
    """``"torch"`` (default) or ``"vmm"``: which allocator backs the peer-visible buffers (``HG_SYMM_ALLOC``)."""
    kind = os.environ.get("HG_SYMM_ALLOC", "torch")
    if kind not in ("torch", "vmm"):
        raise ValueError("HG_SYMM_ALLOC must be 'torch' or 'vmm', got %r" % kind)
    return kind


def allocate(nbytes: int, device: torch.device, pg):
    """Collective over ``pg``: ``nbytes`` of zeroed peer-visible memory per rank.  Returns ``(local uint8 tensor,
    [device pointer of every rank's block], owner)``; ``owner`` keeps the mapping alive."""
    if allocator() == "vmm":
        owner = VmmSymmetricBuffer(nbytes, device, pg)
        return owner.raw, list(owner.ptrs), owner
    import torch.distributed._symmetric_memory as symm

    buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
    buf.zero_()
    owner = symm.rendezvous(buf, pg)
    return buf, [int(p) for p in owner.buffer_ptrs], owner
