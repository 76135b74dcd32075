"""Symmetric memory: buffers that every rank of a group allocates identically and maps from every peer, so a
kernel can load from / store to any rank's copy over NVLink.  Allocation and handle exchange use
``torch.distributed._symmetric_memory`` (CUDA VMM + fabric/IPC handles under the hood); everything that
*touches* the memory is our own kernels in ``csrc/comm.cu``.

``SymmetricBuffer.peer_ptrs`` is a ctypes ``long long[W + 1]``: the W device addresses (index = rank) and the buffer's
multicast address (0 if none).
``EpochBarrier`` is the flag barrier those kernels are bracketed with: a monotonically increasing epoch per
barrier object (flags are never reset, so there is no ABA window), bounded polling on the device, status word
on expiry.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _backend as B

SPIN_LIMIT = 20_000_000  # × ≥64 ns per poll: gives up after a couple of seconds


def _group(group):
    return dist.group.WORLD if group is None else group


class SymmetricBuffer:
    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm
        self.group = _group(group)
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.tensor = symm.empty(numel, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.tensor, self.group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != self.world:
            raise RuntimeError("symmetric memory rendezvous returned an unexpected number of peers")
        if ptrs[self.rank] != self.tensor.data_ptr():
            raise RuntimeError("symmetric memory: this rank's mapped address is not the tensor's address")
        self.ptr_list = ptrs
        # NVSwitch multicast address of the buffer (one access reaches every rank's copy; 0 when the allocation has no multicast
        # binding).  It rides behind the W peer addresses: kernels that take a `use_mc` flag read it from slot W.
        self.multicast_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        self.peer_ptrs = (ctypes.c_longlong * (self.world + 1))(*ptrs, self.multicast_ptr)
        self.tensor.zero_()


class EpochBarrier:
    def __init__(self, device: torch.device, group=None):
        self.pad = SymmetricBuffer(64, torch.int32, device, group)
        self.epoch = 0
        self.device = device
        # every rank's pad must be zeroed before anyone signals into it
        torch.cuda.synchronize(device)
        dist.barrier(group=self.pad.group)

    def __call__(self) -> None:
        self.epoch += 1
        lib = B.load_library()
        st = B.status_buffer(self.device)
        B.check(lib.cmb_comm_barrier(self.pad.peer_ptrs, self.pad.rank, self.pad.world, self.epoch,
                                     ctypes.c_longlong(SPIN_LIMIT), B.ptr(st), B.stream_ptr()), "comm_barrier")
