"""Symmetric (peer-mapped) device buffers for the fused compute+collective kernels.

With more than one rank the buffers come from ``torch.distributed._symmetric_memory`` (CUDA VMM
allocations exchanged by handle and mapped at every peer of the NVLink domain); the kernels
that use them are this package's own and address peers with plain 16-byte loads and stores.
With one rank, or on CPU, an ordinary tensor stands in and the peer list has one entry, so the
same code path (and the same kernels) run at every world size.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class SymmBuffer:
    """A tensor that exists at the same size on every rank, with every rank's base address."""

    def __init__(self, numel: int, dtype: torch.dtype, device: torch.device, group=None, zero: bool = True):
        self.world = dist.get_world_size(group) if (dist.is_initialized() and device.type == "cuda") else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.handle = None
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            self.tensor = symm_mem.empty(numel, dtype=dtype, device=device)
            if zero:
                self.tensor.zero_()
            torch.cuda.synchronize(device)
            g = group if group is not None else dist.group.WORLD
            self.handle = symm_mem.rendezvous(self.tensor, group=g)
            self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
            dist.barrier(group)
        else:
            self.tensor = torch.zeros(numel, dtype=dtype, device=device) if zero else \
                torch.empty(numel, dtype=dtype, device=device)
            self.ptrs = [self.tensor.data_ptr()]
        if device.type == "cuda":
            self.ptrs_dev = torch.tensor(self.ptrs, dtype=torch.int64, device=device)
        else:
            self.ptrs_dev = torch.tensor(self.ptrs, dtype=torch.int64)

    @property
    def multicast_ptr(self) -> int:
        """NVLS multicast address of the buffer (0 when the fabric or the driver has none)."""
        if self.handle is None:
            return 0
        if self.ptrs[self.rank] != self.tensor.data_ptr():
            return 0        # the tensor does not start at the allocation base: offsets would not line up
        try:
            return int(self.handle.multicast_ptr or 0)
        except (AttributeError, RuntimeError):
            return 0

    def peer_tensor(self, rank: int, shape, dtype=None) -> torch.Tensor:
        """A view of ``rank``'s buffer (for tests and NCCL-free debugging; not used on hot paths)."""
        if self.handle is None:
            assert rank == 0
            return self.tensor.view(shape)
        return self.handle.get_buffer(rank, shape, dtype or self.tensor.dtype)
