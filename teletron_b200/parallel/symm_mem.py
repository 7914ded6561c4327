"""Symmetric heap: identically laid out device buffers on every rank of a group, mapped into each
other's address space, for kernels that move data over NVLink themselves.

Each rank ``cudaMalloc``s one slab, exports a CUDA IPC handle, exchanges handles through the group
(``all_gather_object``) and opens its peers' slabs; kernels then receive a table of peer base pointers.
The first 4 KiB of every slab hold 64-bit flag words used by the device-side barrier
(``tt_comm_barrier``): rank ``r`` writes its epoch into slot ``r`` of every peer and waits, with a bound,
for all slots of its own array.  No NVLS multicast object is ever created, so a rank that leaves only
makes its peers' next barrier time out (``CommTimeoutError``) instead of faulting their GPUs.

The reference has no equivalent: every collective there is an NCCL call
(``teletron/core/parallel_state.py:279-515``).
"""

from __future__ import annotations

import ctypes
import weakref
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops._lib import call

FLAG_BYTES = 4096
DEFAULT_TIMEOUT_CYCLES = 20_000_000_000      # ~10 s of GPU clock


class _RawBuffer:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _as_tensor(ptr: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_RawBuffer(ptr, nbytes), device=device)


ALLOCATED_BYTES = 0      # bytes of symmetric heaps this process holds (outside the PyTorch caching allocator)
LIVE_HEAPS: "weakref.WeakSet[SymmetricHeap]" = weakref.WeakSet()     # read by the per-step status check


def set_barrier_timeout_seconds(seconds: float) -> None:
    """Budget of every device-side barrier created from now on (GPU clock taken as 2 GHz)."""
    global DEFAULT_TIMEOUT_CYCLES
    DEFAULT_TIMEOUT_CYCLES = max(1, int(seconds * 2e9))


class SymmetricHeap:
    """One slab per rank; ``alloc`` hands out identically placed regions (bump allocator, 1 KiB aligned)."""

    def __init__(self, group, nbytes: int, device: Optional[torch.device] = None):
        self.group = group
        self.world = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = int(nbytes) + FLAG_BYTES
        p = ctypes.c_void_p()
        call("tt_symm_alloc", ctypes.c_size_t(self.nbytes), ctypes.byref(p))
        self.local_ptr = p.value
        global ALLOCATED_BYTES
        ALLOCATED_BYTES += self.nbytes
        self.peer_ptrs: List[int] = [0] * self.world
        self.peer_ptrs[self.rank] = self.local_ptr
        self._opened: List[int] = []
        if self.world > 1:
            h = ctypes.create_string_buffer(64)
            call("tt_ipc_get_handle", ctypes.c_void_p(self.local_ptr), h)
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(h.raw), group=group)
            for r, hb in enumerate(handles):
                if r == self.rank:
                    continue
                q = ctypes.c_void_p()
                call("tt_ipc_open", ctypes.create_string_buffer(hb, 64), ctypes.byref(q))
                self.peer_ptrs[r] = q.value
                self._opened.append(q.value)
        self._bump = FLAG_BYTES
        self._epoch = 0
        self._status = torch.zeros(4, dtype=torch.int32, device=self.device)
        self._views: Dict[Tuple[int, int], torch.Tensor] = {}
        self.timeout_cycles = DEFAULT_TIMEOUT_CYCLES
        LIVE_HEAPS.add(self)

    # ------------------------------------------------------------------ allocation
    def alloc(self, nbytes: int) -> int:
        """Reserve ``nbytes`` at the same offset on every rank; returns the offset.  Collective by
        convention: all ranks must make the same sequence of calls."""
        off = self._bump
        self._bump = (off + int(nbytes) + 1023) // 1024 * 1024
        if self._bump > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {self._bump} of {self.nbytes} bytes")
        return off

    def reset(self) -> None:
        self._bump = FLAG_BYTES

    def tensor(self, offset: int, shape: Sequence[int], dtype: torch.dtype, rank: Optional[int] = None) -> torch.Tensor:
        """A tensor over this rank's (or peer ``rank``'s) region starting at ``offset``."""
        r = self.rank if rank is None else rank
        numel = 1
        for s in shape:
            numel *= int(s)
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        if offset + nbytes > self.nbytes:
            raise ValueError("region exceeds the symmetric slab")
        return _as_tensor(self.peer_ptrs[r] + offset, nbytes, self.device).view(dtype).view(*shape)

    def ptr_table(self, offset: int = 0):
        """ctypes array of every rank's pointer to ``offset`` (what the kernels take)."""
        return (ctypes.c_void_p * self.world)(*[p + offset for p in self.peer_ptrs])

    # ------------------------------------------------------------------ synchronisation
    def barrier(self, timeout_cycles: Optional[int] = None) -> None:
        """Device-side barrier on the current stream: everything this rank wrote before is visible to its
        peers after they pass it, and vice versa."""
        self._epoch += 1
        if self.world == 1:
            return
        call("tt_comm_barrier", self.ptr_table(0), ctypes.c_int(self.rank), ctypes.c_int(self.world),
             ctypes.c_ulonglong(self._epoch), ctypes.c_longlong(timeout_cycles or self.timeout_cycles),
             _lib.ptr(self._status), _lib.stream())

    def check(self) -> None:
        """Synchronise and raise :class:`CommTimeoutError` if a barrier on this heap ran out."""
        code = int(self._status[0].item())
        if code:
            self._status.zero_()
            raise _lib.CommTimeoutError(f"symmetric-heap barrier timed out on rank {self.rank} (status {code})")

    def close(self, collective: bool = False) -> None:
        """Unmap the peers' slabs and free this rank's.  ``collective=True`` (every rank of the group calls it at the same
        point of the program): wait for this GPU's work, meet the peers so that none of their kernels still touches this
        slab, unmap, meet again so that nobody frees a slab that is still mapped elsewhere, then free."""
        LIVE_HEAPS.discard(self)
        if collective and self.world > 1 and self.local_ptr:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
            for p in self._opened:
                try:
                    call("tt_ipc_close", ctypes.c_void_p(p))
                except Exception:
                    pass
            self._opened = []
            dist.barrier(group=self.group)
        for p in self._opened:
            try:
                call("tt_ipc_close", ctypes.c_void_p(p))
            except Exception:
                pass
        self._opened = []
        if self.local_ptr:
            call("tt_symm_free", ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0
            global ALLOCATED_BYTES
            ALLOCATED_BYTES -= self.nbytes


_HEAPS: Dict[int, SymmetricHeap] = {}


def get_heap(group, nbytes: int) -> SymmetricHeap:
    """Per-group heap, created on first use (collective) and grown never: size it for the largest use."""
    key = id(group)
    h = _HEAPS.get(key)
    if h is None or h.nbytes < nbytes + FLAG_BYTES:
        if h is not None:
            h.close(collective=True)
        h = _HEAPS[key] = SymmetricHeap(group, nbytes)
    return h
