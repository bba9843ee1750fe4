"""Checkpoint / resume.

The reference has no checkpointing at all (its Adam state is an in-memory map keyed by raw
pointer, src/optimizers.h:26); the one on-disk convention it uses is a headerless little-endian
float32 stream (src/mars.cpp:152-166). Two formats are therefore provided:

* ``save_parameters`` / ``load_parameters``: that raw stream, parameters concatenated in
  ``parameters()`` order (the same bytes the C++ shim's functions of the same names write).
* A checkpoint directory: ``manifest.json`` (parameter names / logical shapes / dtypes, step,
  optimizer step, RNG state, config) + per writing rank ``rankNNNNN.bin`` (fp32 pieces) and
  ``rankNNNNN.json`` (what each piece is). A piece is a part of a LOGICAL parameter - either a
  flat element range (ZeRO shards of the data-parallel engine) or a block along one dim (tensor-
  parallel shards) - so a checkpoint can be loaded into any DP x TP layout: the reader
  reassembles logical tensors and every loading rank cuts out what it owns.

Writes are asynchronous: the state is copied to pinned host memory on a side stream and a thread
writes the files, so the training step is not stalled; ``SaveHandle.wait()`` finishes the
checkpoint (collective: every rank calls it).
"""
from __future__ import annotations

import json
import os
import threading
from typing import Iterable, Sequence

import numpy as np
import torch
import torch.distributed as dist

FORMAT = "dummygrad_b200.checkpoint.v1"
KINDS = ("master", "m", "v")


# ----------------------------------------------------------------------------- raw .bin streams
def save_parameters(path: str, params: Iterable) -> None:
    """Raw little-endian fp32, parameters concatenated in the given order."""
    with open(path, "wb") as f:
        for p in params:
            t = p.data if hasattr(p, "data") and isinstance(p.data, torch.Tensor) else p
            f.write(t.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False).tobytes())


def load_parameters(path: str, params: Iterable) -> None:
    params = list(params)
    need = sum(int(p.data.numel()) for p in params)
    have = os.path.getsize(path) // 4
    if have < need:
        raise ValueError(f"{path}: holds {have} floats, the parameters need {need}")
    mm = np.memmap(path, dtype="<f4", mode="r")
    off = 0
    for p in params:
        n = int(p.data.numel())
        src = torch.from_numpy(np.array(mm[off:off + n])).view(p.data.shape)
        p.data.copy_(src.to(p.data.dtype))
        off += n


# ----------------------------------------------------------------------------- writer
class SaveHandle:
    def __init__(self, dirpath: str, thread: threading.Thread | None, manifest: dict | None, group=None):
        self.dirpath, self._thread, self._manifest, self._group = dirpath, thread, manifest, group
        self.error: BaseException | None = None

    def wait(self) -> None:
        """Join the writer, then (rank 0, after every rank is done) publish the manifest."""
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self.error is not None:
            raise RuntimeError(f"checkpoint write failed: {self.error}") from self.error
        if dist.is_initialized():
            dist.barrier(self._group)
        if self._manifest is not None:
            tmp = os.path.join(self.dirpath, "manifest.json.tmp")
            with open(tmp, "w") as f:
                json.dump(self._manifest, f, indent=1)
            os.replace(tmp, os.path.join(self.dirpath, "manifest.json"))
            self._manifest = None
        if dist.is_initialized():
            dist.barrier(self._group)


def _write_pieces(dirpath: str, writer_rank: int, pieces: list[tuple[dict, torch.Tensor]], manifest: dict | None,
                  group=None, asynchronous: bool = True) -> SaveHandle:
    """pieces: (meta, tensor). Stages everything into one pinned fp32 host buffer, then writes."""
    os.makedirs(dirpath, exist_ok=True)
    total = sum(int(t.numel()) for _, t in pieces)
    cuda = any(t.is_cuda for _, t in pieces)
    host = torch.empty(max(total, 1), dtype=torch.float32, pin_memory=cuda)
    index, off, done = [], 0, None
    if cuda:
        dev = next(t.device for _, t in pieces if t.is_cuda)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        ctx = torch.cuda.stream(side)
    else:
        import contextlib
        ctx = contextlib.nullcontext()
    with ctx:
        for meta, t in pieces:
            n = int(t.numel())
            src = t.detach().reshape(-1)
            host[off:off + n].copy_(src if src.dtype == torch.float32 else src.float(), non_blocking=cuda)
            index.append(dict(meta, offset=off * 4, numel=n))
            off += n
        if cuda:
            done = torch.cuda.Event()
            done.record(side)
            for _, t in pieces:          # the caller may overwrite these right after we return
                if t.is_cuda:
                    t.record_stream(side)
    handle = SaveHandle(dirpath, None, manifest, group)
    base = os.path.join(dirpath, f"rank{writer_rank:05d}")

    def work():
        try:
            if done is not None:
                done.synchronize()
            with open(base + ".bin.tmp", "wb") as f:
                f.write(host[:total].numpy().astype("<f4", copy=False).tobytes())
                f.flush()
                os.fsync(f.fileno())
            os.replace(base + ".bin.tmp", base + ".bin")
            with open(base + ".json.tmp", "w") as f:
                json.dump({"file": os.path.basename(base) + ".bin", "pieces": index}, f)
            os.replace(base + ".json.tmp", base + ".json")
        except BaseException as e:  # surfaced by wait()
            handle.error = e

    if total == 0 and not pieces:
        return handle
    if asynchronous:
        handle._thread = threading.Thread(target=work, name="dg-checkpoint-writer", daemon=True)
        handle._thread.start()
    else:
        work()
    return handle


def _rng_state() -> dict:
    st = {"torch_cpu": torch.get_rng_state().numpy().tobytes().hex()}
    if torch.cuda.is_available():
        st["torch_cuda"] = torch.cuda.get_rng_state().numpy().tobytes().hex()
    return st


def restore_rng(manifest: dict) -> None:
    st = manifest.get("rng", {})
    if "torch_cpu" in st:
        torch.set_rng_state(torch.from_numpy(np.frombuffer(bytes.fromhex(st["torch_cpu"]), dtype=np.uint8).copy()))
    if "torch_cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(torch.from_numpy(np.frombuffer(bytes.fromhex(st["torch_cuda"]), dtype=np.uint8).copy()))


def _manifest(params: Sequence, shapes: Sequence[Sequence[int]], names: Sequence[str] | None, step: int, opt_t: int,
              config, layout: dict, extra: dict | None) -> dict:
    names = list(names) if names is not None else [f"param{i:04d}" for i in range(len(params))]
    cfg = config.to_dict() if hasattr(config, "to_dict") else (config or {})
    return {"format": FORMAT, "step": int(step), "optimizer_t": int(opt_t), "layout": layout,
            "params": [{"name": n, "shape": [int(s) for s in sh], "dtype": str(p.dtype).replace("torch.", "")}
                       for n, sh, p in zip(names, shapes, params)],
            "rng": _rng_state(), "config": cfg, "extra": extra or {}}
