"""Host model of the fused reduce-scatter + optimizer + parameter-push protocol (no GPU).

CPU processes stand in for ranks and a block of POSIX shared memory stands in for the peer-mapped
symmetric buffers: every rank can read every rank's gradient bucket, write every rank's parameter
buffer and flag pad. The step below is the same sequence the device kernel runs
(csrc/comm/rs_optim.cu): publish "my gradients are final" to every pad, wait - bounded - for every
peer's flag, pull and sum the owned slice in rank order, update, push the slice to every rank,
publish "my slice has landed", wait - bounded - for every peer's done flag. Flags carry the epoch,
so nothing is ever cleared. It exists to test the protocol logic, its timeouts and the
skipped-signal fault on CPU ranks; it moves fp32 and does plain SGD.
"""
from __future__ import annotations

import time
from multiprocessing import shared_memory

import numpy as np

OK, ERR_READY_TIMEOUT, ERR_DONE_TIMEOUT = 0, 0x100, 0x200


class HostPeerMemory:
    """[world] gradient buckets, [world] parameter buffers and [world] flag pads (ready[world],
    done[world]) in one shared-memory segment."""

    def __init__(self, name: str, world: int, n: int, create: bool):
        self.world, self.n = world, n
        floats = 2 * world * n
        size = floats * 4 + world * 2 * world * 4
        self.shm = shared_memory.SharedMemory(name=name, create=create, size=size)
        buf = self.shm.buf
        self.grads = np.ndarray((world, n), dtype=np.float32, buffer=buf, offset=0)
        self.params = np.ndarray((world, n), dtype=np.float32, buffer=buf, offset=world * n * 4)
        self.flags = np.ndarray((world, 2, world), dtype=np.int32, buffer=buf, offset=floats * 4)
        if create:
            self.grads[:] = 0
            self.params[:] = 0
            self.flags[:] = 0

    def close(self, unlink: bool = False) -> None:
        self.grads = self.params = self.flags = None
        self.shm.close()
        if unlink:
            self.shm.unlink()


def wait_flags(flags_row: np.ndarray, epoch: int, timeout_s: float) -> int:
    """Bounded wait until every entry of this rank's flag row has reached ``epoch``. Returns -1 on
    success, else the index of the first peer that did not signal in time."""
    deadline = time.monotonic() + timeout_s
    while True:
        behind = np.nonzero(flags_row < epoch)[0]
        if behind.size == 0:
            return -1
        if time.monotonic() > deadline:
            return int(behind[0])
        time.sleep(0.0005)


def fused_step(mem: HostPeerMemory, rank: int, epoch: int, lr: float, timeout_s: float = 2.0,
               skip_ready_signal: bool = False) -> int:
    """One bucket step of one rank. Returns OK or an error code | peer index (never blocks for
    longer than two timeouts)."""
    W, n = mem.world, mem.n
    shard = n // W
    lo, hi = rank * shard, (rank + 1) * shard
    if not skip_ready_signal:                      # fault injection: a rank that never says "ready"
        for r in range(W):
            mem.flags[r, 0, rank] = epoch
    late = wait_flags(mem.flags[rank, 0], epoch, timeout_s)
    if late >= 0:
        return ERR_READY_TIMEOUT | late
    acc = np.zeros(shard, dtype=np.float32)
    for r in range(W):                             # fixed rank order: deterministic sum
        acc += mem.grads[r, lo:hi]
    new = mem.params[rank, lo:hi] - lr * (acc / W)
    for rr in range(W):                            # local copy first, then the peers in rotation
        mem.params[(rank + rr) % W, lo:hi] = new
    for r in range(W):
        mem.flags[r, 1, rank] = epoch
    late = wait_flags(mem.flags[rank, 1], epoch, timeout_s)
    if late >= 0:
        return ERR_DONE_TIMEOUT | late
    return OK
