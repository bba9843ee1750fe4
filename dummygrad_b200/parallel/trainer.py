"""The user-facing training loop object.

``Trainer.step(ids, targets)`` takes one rank's share of a global batch as pinned host tensors,
copies it to the device, runs forward/backward over micro-batches (gradient accumulation), lets
the data-parallel engine overlap the fused reduce-scatter + optimizer + all-gather kernels with
backward, and returns the loss as a Python float (one device-to-host read).
``Trainer.step_device`` is the same step on tensors that are already on the device and returns
the loss without synchronising.
"""
from __future__ import annotations

import torch

from ..ops import kernels as K
from .dp import DataParallel


class Trainer:
    def __init__(self, model, *, micro_batch: int, lr: float = 3e-4, beta1: float = 0.9, beta2: float = 0.95,
                 eps: float = 1e-8, weight_decay: float = 0.0, optimizer: str = "adamw", comm: str = "fused",
                 bucket_mb: float = 64.0, group=None, max_comm_ctas: int = 32, wait_seconds: float = 20.0):
        self.model = model
        self.micro_batch = micro_batch
        self.dp = DataParallel(model, lr=lr, beta1=beta1, beta2=beta2, eps=eps, weight_decay=weight_decay,
                               optimizer=optimizer, comm=comm, bucket_mb=bucket_mb, group=group,
                               max_comm_ctas=max_comm_ctas, wait_seconds=wait_seconds)
        self.device = self.dp.device
        self._ids_dev = None
        self._tgt_dev = None

    # ------------------------------------------------------------------ steps
    def step_device(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """ids [B_local, S] int64 and targets [B_local * S] int64 on the device. Returns the mean
        loss over the local batch as a one-element fp32 device tensor."""
        B, S = ids.shape
        mb = min(self.micro_batch, B)
        assert B % mb == 0, "local batch must be a multiple of the micro-batch"
        n_micro = B // mb
        self.dp.begin_step(accum_steps=n_micro)
        total = None
        for i in range(n_micro):
            self.dp.set_sync(i == n_micro - 1)
            loss = self.model.loss(ids[i * mb:(i + 1) * mb], targets[i * mb * S:(i + 1) * mb * S])
            loss.backward()
            l = loss.data.reshape(1)
            total = l if total is None else K.ew("ADD", total, l)
        self.dp.finish_step()
        if n_micro > 1:
            total = K.ew("MUL_S", total, s0=1.0 / n_micro)
        return total

    def step(self, ids_host: torch.Tensor, targets_host: torch.Tensor) -> float:
        """One optimizer step from pinned host inputs; returns the loss as a float."""
        if self.device.type == "cuda":
            if self._ids_dev is None or self._ids_dev.shape != ids_host.shape:
                self._ids_dev = torch.empty(ids_host.shape, dtype=torch.int64, device=self.device)
                self._tgt_dev = torch.empty(targets_host.shape, dtype=torch.int64, device=self.device)
            self._ids_dev.copy_(ids_host, non_blocking=True)
            self._tgt_dev.copy_(targets_host, non_blocking=True)
            loss = self.step_device(self._ids_dev, self._tgt_dev)
        else:
            loss = self.step_device(ids_host, targets_host)
        return float(loss.item())

    def check(self) -> None:
        """Raise if a bounded device-side wait expired during the previous steps."""
        code = self.dp.check_status() | (K.gemm_status() if self.device.type == "cuda" else 0)
        if code:
            raise RuntimeError(f"device-side wait timed out (status 0x{code:x}); a peer did not signal in time")
