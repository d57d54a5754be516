"""Symmetric (peer-mapped) device buffers for the in-kernel NVLink paths.

``SymmetricBuffer`` allocates the same-sized buffer on every rank of a group, exchanges the
handles and exposes each peer's base address (``peer_ptrs``), the NVLS multicast address when the
fabric offers one (``multicast_ptr``) and a stream-ordered cross-rank ``barrier``.  Allocation and
rendezvous go through ``torch.distributed._symmetric_memory`` (CUDA VMM export/import under the
hood); all data movement on the hot path is done by this package's own kernels with plain peer
loads / stores (or ``multimem`` through the multicast address).

``LocalPeers`` is the single-process stand-in used by CPU tests and by single-GPU emulation: the
"ranks" are views of one buffer, so the same kernels run over all ranks' data in one process (ranks
that wait on each other are never emulated as separate launches on one GPU).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, group=None, device=None):
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        device = device or torch.device("cuda", torch.cuda.current_device())
        self.local = symm_mem.empty(numel, dtype=dtype, device=device)
        self.handle = symm_mem.rendezvous(self.local, self.group)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.signal_ptrs = [int(p) for p in self.handle.signal_pad_ptrs]
        try:
            self.multicast_ptr = int(self.handle.multicast_ptr)
        except Exception:  # fabric without multicast support
            self.multicast_ptr = 0
        self._arr = (ctypes.c_ulonglong * self.world)(*self.peer_ptrs)

    def ptr_array(self):
        """ctypes array of the peers' base addresses (host memory, passed by pointer to launchers)."""
        return self._arr

    def offset_ptr_array(self, byte_offset: int):
        return (ctypes.c_ulonglong * self.world)(*[p + byte_offset for p in self.peer_ptrs])

    def barrier(self, channel: int = 0) -> None:
        """Cross-rank barrier ordered on the current stream (device-side signal exchange with a
        bounded wait inside torch's implementation)."""
        self.handle.barrier(channel=channel)

    def peer_tensor(self, rank: int, shape, dtype) -> torch.Tensor:
        return self.handle.get_buffer(rank, shape, dtype)


class LocalPeers:
    """``world`` equal buffers inside one process; same accessors as ``SymmetricBuffer``."""

    def __init__(self, numel: int, dtype: torch.dtype, world: int, device="cpu"):
        self.world = world
        self.rank = 0
        self.buffers = [torch.zeros(numel, dtype=dtype, device=device) for _ in range(world)]
        self.local = self.buffers[0]
        self.peer_ptrs = [b.data_ptr() for b in self.buffers]
        self.multicast_ptr = 0

    def view_as_rank(self, rank: int) -> "LocalPeers":
        v = object.__new__(LocalPeers)
        v.__dict__.update(self.__dict__)
        v.rank = rank
        v.local = self.buffers[rank]
        return v

    def ptr_array(self):
        return (ctypes.c_ulonglong * self.world)(*self.peer_ptrs)

    def offset_ptr_array(self, byte_offset: int):
        return (ctypes.c_ulonglong * self.world)(*[p + byte_offset for p in self.peer_ptrs])

    def barrier(self, channel: int = 0) -> None:
        return None

    def peer_tensor(self, rank: int, shape, dtype) -> torch.Tensor:
        return self.buffers[rank].view(dtype)[: int(torch.Size(shape).numel())].view(shape)
