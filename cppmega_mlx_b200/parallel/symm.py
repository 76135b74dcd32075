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


class SymmetricAllReduce:
    """In-place sum over the group of up to ``numel`` elements (fp32 or bf16) through one symmetric buffer: copy in, barrier, one
    kernel in which every rank reduces its slice and publishes it to all (``csrc/comm.cu`` ``allreduce_kernel``), barrier, copy
    out.  ``multimem=True`` uses the in-switch reduction and the multicast store when the buffer has a multicast binding; the
    default is plain peer loads / stores in a fixed rank order (bitwise reproducible, and safe if a rank dies mid-step).
    Meant for the small, latency-bound reductions of a step (norm-weight gradients, loss statistics): three short launches on the
    caller's stream, no NCCL kernel."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None, *, multimem: bool = False):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("SymmetricAllReduce supports float32 and bfloat16")
        per_vec = 16 // torch.empty((), dtype=dtype).element_size()
        self.capacity = (numel + per_vec - 1) // per_vec * per_vec
        self.dtype, self.device = dtype, device
        self.buf = SymmetricBuffer(self.capacity, dtype, device, group)
        self.barrier = EpochBarrier(device, group)
        self.use_mc = int(bool(multimem) and self.buf.multicast_ptr != 0)

    def __call__(self, t: torch.Tensor) -> torch.Tensor:
        n = t.numel()
        if n > self.capacity or t.dtype != self.dtype:
            raise ValueError(f"tensor of {n} {t.dtype} elements does not fit this reducer ({self.capacity} {self.dtype})")
        per_vec = 16 // t.element_size()
        padded = (n + per_vec - 1) // per_vec * per_vec
        view = self.buf.tensor[:padded]
        view[:n].copy_(t.reshape(-1))
        if padded > n:
            view[n:].zero_()
        lib = B.load_library()
        self.barrier()                                      # every rank's input is in its buffer
        B.check(lib.cmb_symm_allreduce(self.buf.peer_ptrs, self.buf.rank, self.buf.world, ctypes.c_longlong(padded * t.element_size()),
                                       1 if t.dtype == torch.bfloat16 else 0, self.use_mc, B.stream_ptr()), "symm_allreduce")
        self.barrier()                                      # every slice has been published to this rank
        t.copy_(view[:n].view_as(t))
        return t
