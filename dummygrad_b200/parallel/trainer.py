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

    # ------------------------------------------------------------------ checkpoints
    def save(self, dirpath: str, *, step: int, config=None, asynchronous: bool = True):
        """Start a checkpoint of weights + sharded optimizer state; call ``.wait()`` on the returned
        handle (every rank) before relying on the files."""
        from .. import checkpoint
        names = self.model.parameter_names() if hasattr(self.model, "parameter_names") else None
        return checkpoint.save_dp(dirpath, self.dp, step=step, config=config, names=names, asynchronous=asynchronous)

    def load(self, dirpath: str) -> dict:
        """Resume from a checkpoint written at any world size; returns its manifest."""
        from .. import checkpoint
        return checkpoint.load_dp(dirpath, self.dp)

    def check(self) -> None:
        """Raise if a bounded device-side wait expired during the previous steps."""
        code = self.dp.check_status() | (K.gemm_status() if self.device.type == "cuda" else 0)
        if code:
            raise RuntimeError(f"device-side wait timed out (status 0x{code:x}); a peer did not signal in time")


class TPTrainer:
    """Training loop for tensor parallelism (optionally x data parallelism).

    Ranks are grouped as ``dp`` replicas of ``tp`` consecutive ranks. Every rank of a tensor-
    parallel group receives the same micro-batch; activations between the parallel regions are
    sharded on tokens and the collectives run inside the GEMM kernels. After backward the
    gradients of replicated parameters are summed over the tensor-parallel group, all gradients are
    averaged over the data-parallel group (NCCL), and a multi-tensor AdamW updates local weights.
    """

    def __init__(self, preset: str, *, tp_size: int, micro_batch: int, seq_len: int, lr: float = 2e-4,
                 weight_decay: float = 0.1, comm: str = "fused", dtype=torch.bfloat16, device=None):
        import torch.distributed as dist
        from ..models.gpt import PRESETS
        from ..optim import AdamW
        from . import tp as tpm
        from .tp_layers import TPGPT
        world = dist.get_world_size() if dist.is_initialized() else 1
        rank = dist.get_rank() if dist.is_initialized() else 0
        assert world % tp_size == 0
        self.tp_size, self.dp_size = tp_size, world // tp_size
        self.tp_group = self.dp_group = None
        if world > 1 and tp_size < world:
            for g in range(self.dp_size):
                grp = dist.new_group(list(range(g * tp_size, (g + 1) * tp_size)))
                if rank // tp_size == g:
                    self.tp_group = grp
            for t in range(tp_size):
                grp = dist.new_group(list(range(t, world, tp_size)))
                if rank % tp_size == t:
                    self.dp_group = grp
        self.device = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.ctx = tpm.TPContext(group=self.tp_group, comm=comm, device=self.device, single=(tp_size == 1))
        v, s, d, h, l, ff = PRESETS[preset] if isinstance(preset, str) else preset   # or an explicit 6-tuple
        self.model = TPGPT(self.ctx, v, s, d, h, l, ff, (micro_batch, seq_len), dtype=dtype, device=self.device)
        self.opt = AdamW(self.model.parameters(), lr=lr, weight_decay=weight_decay, beta2=0.95)
        self.micro_batch = micro_batch
        self.dp_rank = rank // tp_size

    def step_device(self, ids: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
        """ids [B_replica, S] / targets [B_replica * S]: this data-parallel replica's batch, identical on
        the ranks of its tensor-parallel group. Returns this rank's share of the replica's mean loss."""
        from .tp_layers import allreduce_replicated_grads
        B, S = ids.shape
        mb = min(self.micro_batch, B)
        n_micro = B // mb
        self.opt.zero_grad()
        total = None
        for i in range(n_micro):
            loss = self.model.loss(ids[i * mb:(i + 1) * mb], targets[i * mb * S:(i + 1) * mb * S])
            loss.backward()
            l = loss.data.reshape(1)
            total = l if total is None else K.ew("ADD", total, l)
        allreduce_replicated_grads(self.model.parameters(), self.ctx, self.dp_group, self.dp_size)
        self.opt.step(grad_scale=1.0 / (n_micro * self.dp_size))
        return K.ew("MUL_S", total, s0=1.0 / n_micro) if n_micro > 1 else total

    def save(self, dirpath: str, *, step: int, config=None, asynchronous: bool = True):
        from .. import checkpoint
        return checkpoint.save_tp(dirpath, self.model, self.opt, self.ctx, step=step, dp_rank=self.dp_rank,
                                  config=config, asynchronous=asynchronous)

    def load(self, dirpath: str) -> dict:
        from .. import checkpoint
        return checkpoint.load_tp(dirpath, self.model, self.opt, self.ctx)

    def check(self) -> None:
        code = self.ctx.check_status() | K.gemm_status()
        if code:
            raise RuntimeError(f"device-side wait timed out (status 0x{code:x})")
