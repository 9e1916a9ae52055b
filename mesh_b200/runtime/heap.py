"""Symmetric heap over NVLink peer mappings (Python side).

Each rank owns one equally sized device allocation; every rank maps every other rank's allocation
(CUDA VMM handles passed as file descriptors, or legacy IPC handles), so a kernel can store straight
into a peer's buffer at the same offset — the NVLink form of the reference's shared region and
compiler-fixed landing addresses (rdma/mesh.h:173-228; design/collective-goals.md:30-41).  The first
``signal_bytes`` of the heap are the signal pad: monotonically increasing 32-bit counters, never
reset, that play the role of the reference's phase/count/supplied words (rdma/mesh-flow.c:9-15).

Allocation is a deterministic bump allocator, so every rank that issues the same sequence of
``alloc`` calls gets the same offsets without exchanging anything.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint64, c_void_p
from dataclasses import dataclass

import torch

from .. import _native
from .rendezvous import Rendezvous


class _VmmBlock(ctypes.Structure):
    _fields_ = [("handle", c_uint64), ("ptr", c_uint64), ("size", c_uint64), ("fd", c_int), ("device", c_int)]


class _DevMem:
    """Minimal ``__cuda_array_interface__`` holder so torch can view raw device memory."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}
        self._owner = owner


@dataclass
class SymmBuffer:
    """A region of the symmetric heap: same offset on every rank."""
    heap: "SymmetricHeap"
    offset: int
    nbytes: int
    shape: tuple
    dtype: torch.dtype

    @property
    def local(self) -> torch.Tensor:
        return self.heap.view(self.offset, self.shape, self.dtype)

    def ptr(self, rank: int | None = None) -> int:
        r = self.heap.rank if rank is None else rank
        return self.heap.peer_ptrs[r] + self.offset

    @property
    def mc_ptr(self) -> int:
        return self.heap.mc_ptr + self.offset if self.heap.mc_ptr else 0

    def ptrs(self) -> list[int]:
        return [self.heap.peer_ptrs[r] + self.offset for r in range(self.heap.world)]


class HeapGroup:
    """A subset of a heap's ranks seen as a heap of its own: ``rank`` and ``world`` are positions within the
    group, and buffers resolve peer pointers through the group's member list, so a communicator, a fused layer or a
    model built on it talks to the members only (a tensor-, context- or expert-parallel axis of a larger job; the
    reference's submeshes, mesh/api.py:40-120).

    Allocation moves the parent's bump pointer.  The heap stays symmetric as long as every rank of the job makes the
    same sequence of allocations, each through its own group of an axis (groups of one axis have equal sizes)."""

    def __init__(self, heap: "SymmetricHeap", ranks):
        ranks = [int(r) for r in ranks]
        if heap.rank not in ranks:
            raise ValueError(f"rank {heap.rank} is not a member of group {ranks}")
        if len(set(ranks)) != len(ranks) or any(not 0 <= r < heap.world for r in ranks):
            raise ValueError(f"bad group {ranks} for a heap of {heap.world} ranks")
        self.parent, self.ranks = heap, ranks
        self.rank, self.world = ranks.index(heap.rank), len(ranks)
        self.device = heap.device
        self.peer_ptrs = [heap.peer_ptrs[r] for r in ranks]
        self.mc_ptr = 0                      # the multicast mapping spans all ranks of the parent

    def _wrap(self, b: "SymmBuffer") -> "SymmBuffer":
        return SymmBuffer(self, b.offset, b.nbytes, b.shape, b.dtype)

    def alloc(self, shape, dtype=torch.bfloat16, align: int = 1024) -> "SymmBuffer":
        return self._wrap(self.parent.alloc(shape, dtype, align))

    def alloc_signals(self, count: int) -> "SymmBuffer":
        return self._wrap(self.parent.alloc_signals(count))

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        return self.parent.view(offset, shape, dtype)

    def mark(self):
        return self.parent.mark()

    def release(self, mark) -> None:
        self.parent.release(mark)

    def group(self, ranks) -> "HeapGroup":
        """Sub-group given by positions within this group."""
        return HeapGroup(self.parent, [self.ranks[r] for r in ranks])

    def close(self) -> None:               # the parent owns the memory
        pass


class SymmetricHeap:
    def __init__(self, rdv: Rendezvous, nbytes: int, device: int, *, signal_bytes: int = 1 << 20,
                 multicast: bool = False, mode: str = "auto"):
        self.rdv = rdv
        self.rank, self.world = rdv.rank, rdv.world
        self.device = device
        self.signal_bytes = signal_bytes
        self.mc_ptr = 0
        self._mc_handle = 0
        self._blocks: list[_VmmBlock] = []
        self._ipc_opened: list[int] = []
        self.epoch = rdv.epoch
        L = _native.lib()
        torch.cuda.set_device(device)
        gran = c_uint64(0)
        rc = L.mesh_vmm_granularity(c_int(device), c_int(int(multicast)), c_int(self.world), ctypes.byref(gran))
        if rc != 0:
            if mode == "vmm":
                _native.check(rc, "mesh_vmm_granularity")
            mode = "ipc"
            gran.value = 2 << 20
        g = max(int(gran.value), 2 << 20)
        self.nbytes = (nbytes + signal_bytes + g - 1) // g * g
        self.mode = "vmm" if mode in ("auto", "vmm") else "ipc"
        if self.mode == "vmm":
            try:
                self._init_vmm(L, multicast)
            except Exception:
                if mode == "vmm":
                    raise
                self._teardown_vmm(L)
                self.mode = "ipc"
        # every rank must agree on the mode: fall back together
        modes = rdv.exchange("heap-mode", self.mode)
        if any(m != modes[0] for m in modes):
            if self.mode == "vmm":
                self._teardown_vmm(L)
            self.mode = "ipc"
        if self.mode == "ipc":
            self._init_ipc(L)
        self._holder = _DevMem(self.peer_ptrs[self.rank], self.nbytes, self)
        self._bytes = torch.as_tensor(self._holder, device=torch.device("cuda", device))
        self._bytes.zero_()
        torch.cuda.synchronize(device)
        rdv.barrier("heap-ready")
        self._bump = signal_bytes
        self._sig_bump = 0

    # ------------------------------------------------------------------ bring-up
    def _init_vmm(self, L, multicast: bool) -> None:
        mine = _VmmBlock()
        _native.check(L.mesh_vmm_alloc(c_uint64(self.nbytes), c_int(self.device), ctypes.byref(mine)), "mesh_vmm_alloc")
        self._blocks = [mine]
        fds = self.rdv.exchange_fds("heap", mine.fd)
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = int(mine.ptr)
        import os
        for r, fd in enumerate(fds):
            if r == self.rank:
                continue
            blk = _VmmBlock()
            _native.check(L.mesh_vmm_import(c_int(fd), c_uint64(self.nbytes), c_int(self.device), ctypes.byref(blk)),
                          f"mesh_vmm_import(rank {r})")
            os.close(fd)
            self._blocks.append(blk)
            self.peer_ptrs[r] = int(blk.ptr)
        if multicast and self.world > 1 and L.mesh_mc_supported(c_int(self.device)):
            self._init_multicast(L, mine)

    def _init_multicast(self, L, mine: _VmmBlock) -> None:
        import os
        h = c_uint64(0)
        fd = c_int(-1)
        if self.rank == 0:
            _native.check(L.mesh_mc_create(c_uint64(self.nbytes), c_int(self.world), ctypes.byref(h), ctypes.byref(fd)),
                          "mesh_mc_create")
        fds = self.rdv.exchange_fds("mc", fd.value if self.rank == 0 else os.open("/dev/null", os.O_RDONLY))
        if self.rank != 0:
            _native.check(L.mesh_mc_import(c_int(fds[0]), ctypes.byref(h)), "mesh_mc_import")
        for r, f in enumerate(fds):
            if not (r == 0 and self.rank == 0):
                try:
                    os.close(f)
                except OSError:
                    pass
        _native.check(L.mesh_mc_add_device(h, c_int(self.device)), "mesh_mc_add_device")
        self.rdv.barrier("mc-added")
        p = c_uint64(0)
        _native.check(L.mesh_mc_bind_map(h, c_uint64(mine.handle), c_uint64(self.nbytes), c_int(self.device),
                                         ctypes.byref(p)), "mesh_mc_bind_map")
        self._mc_handle, self.mc_ptr = int(h.value), int(p.value)
        self.rdv.barrier("mc-bound")

    def _teardown_vmm(self, L) -> None:
        for blk in self._blocks:
            L.mesh_vmm_free(ctypes.byref(blk))
        self._blocks = []

    def _init_ipc(self, L) -> None:
        ptr = c_uint64(0)
        handle = (ctypes.c_ubyte * 64)()
        _native.check(L.mesh_ipc_alloc(c_uint64(self.nbytes), c_int(self.device), ctypes.byref(ptr), handle),
                      "mesh_ipc_alloc")
        handles = self.rdv.exchange("ipc", bytes(handle))
        self.peer_ptrs = [0] * self.world
        self.peer_ptrs[self.rank] = int(ptr.value)
        for r, hb in enumerate(handles):
            if r == self.rank:
                continue
            p = c_uint64(0)
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(hb)
            _native.check(L.mesh_ipc_open(buf, c_int(self.device), ctypes.byref(p)), f"mesh_ipc_open(rank {r})")
            self.peer_ptrs[r] = int(p.value)
            self._ipc_opened.append(int(p.value))

    # ------------------------------------------------------------------ allocation
    def alloc(self, shape, dtype=torch.bfloat16, align: int = 1024) -> SymmBuffer:
        shape = tuple(int(s) for s in (shape if isinstance(shape, (tuple, list)) else (shape,)))
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        off = (self._bump + align - 1) // align * align
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {nbytes} at {off}, size {self.nbytes}")
        self._bump = off + nbytes
        return SymmBuffer(self, off, nbytes, shape, dtype)

    def alloc_signals(self, count: int) -> SymmBuffer:
        """``count`` 32-bit counters in the signal pad (zero at creation, then only ever increased)."""
        off = (self._sig_bump + 127) // 128 * 128
        if off + 4 * count > self.signal_bytes:
            raise MemoryError("signal pad exhausted")
        self._sig_bump = off + 4 * count
        return SymmBuffer(self, off, 4 * count, (count,), torch.int32)

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        nbytes = n * torch.empty((), dtype=dtype).element_size()
        return self._bytes[offset:offset + nbytes].view(dtype).view(*shape)

    def group(self, ranks) -> HeapGroup:
        """The ranks ``ranks`` (which must include this one) as a heap of their own."""
        return HeapGroup(self, ranks)

    def mark(self) -> tuple[int, int]:
        return self._bump, self._sig_bump

    def release(self, mark: tuple[int, int]) -> None:
        """Give back everything allocated since ``mark`` (stack discipline, same on every rank; collective).

        Signal words are counters that only grow, and their next owner starts expecting from zero: so the returned
        signal range is cleared here, after every rank's work on it has drained and before any rank can hand it out
        again (barrier on both sides).  Without that, a communicator built on released words would find the old
        totals and pass its first waits before its peers had published anything."""
        bump, sig = mark
        if sig < self._sig_bump:
            torch.cuda.synchronize(self.device)
            self.rdv.barrier("heap-release-drained")            # nobody still signals into the range
            self._bytes[sig:self._sig_bump].zero_()
            torch.cuda.synchronize(self.device)
            self.rdv.barrier("heap-release-cleared")            # cleared everywhere before anyone reuses it
        self._bump, self._sig_bump = bump, sig

    # ------------------------------------------------------------------ teardown
    def close(self) -> None:
        """Bounded, ordered teardown: drain, barrier, unmap peers, then free (never frees memory a
        peer may still be writing: all ranks pass the barrier first)."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        L = _native.lib()
        torch.cuda.synchronize(self.device)
        try:
            self.rdv.barrier("heap-close")
        except Exception:
            pass
        self._bytes = None
        if self.mode == "vmm":
            if self._mc_handle:
                L.mesh_mc_unmap(c_uint64(self._mc_handle), c_uint64(self.mc_ptr), c_uint64(self.nbytes), c_int(self.device))
            self._teardown_vmm(L)
        else:
            for p in self._ipc_opened:
                L.mesh_ipc_close(c_uint64(p))
            L.mesh_ipc_free(c_uint64(self.peer_ptrs[self.rank]))
