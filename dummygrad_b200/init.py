"""Initialisers with the reference's definitions (src/init.h).

``xavier`` is N(0, sqrt(1/fan_in)) and ``kaiming`` N(0, sqrt(2/fan_in)) over 2-D shapes,
exactly as the reference defines them (they are not the Glorot-uniform / He variants of
other libraries). ``randn/xavier/kaiming`` return tensors that require grad; ``ones``,
``zeros`` and ``one_hot`` do not. On CUDA the numbers come from the Philox kernel, seeded by
``manual_seed`` and advanced by one counter block per four elements; on CPU from a
``torch.Generator``. Bit-equality with the reference's ``std::mt19937`` stream is not a goal
(``std::normal_distribution`` is implementation-defined); parity tests inject weights.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch

from .ops import kernels as K
from .tensor import Tensor, default_device, default_dtype


class _Gen:
    """Global generator state (the reference's ``g_gen``, src/init.h:4)."""

    def __init__(self):
        self.seed = torch.seed() & 0x7FFFFFFFFFFFFFFF
        self.offset = 0
        self.cpu = torch.Generator()
        self.cpu.manual_seed(self.seed)


g_gen = _Gen()


def manual_seed(seed: int) -> None:
    g_gen.seed = int(seed)
    g_gen.offset = 0
    g_gen.cpu.manual_seed(int(seed))


def _normal(shape: Sequence[int], std: float, requires_grad: bool, dtype=None, device=None) -> Tensor:
    t = Tensor(shape, requires_grad, dtype=dtype or default_dtype(), device=device or default_device())
    n = t.size()
    if t.data.is_cuda:
        # draw in fp32 so bf16 parameters are a rounding of the same stream
        if t.dtype == torch.float32:
            K.randn_(t.data, g_gen.seed, g_gen.offset, 0.0, std)
        else:
            tmp = torch.empty(t.data.shape, dtype=torch.float32, device=t.data.device)
            K.randn_(tmp, g_gen.seed, g_gen.offset, 0.0, std)
            K.assign_(t.data, tmp)
        g_gen.offset += (n + 3) // 4
    else:
        K.randn_(t.data, g_gen.seed, g_gen.offset, 0.0, std, generator=g_gen.cpu)
    return t


def randn(shape: Sequence[int], dtype=None, device=None) -> Tensor:
    return _normal(shape, 1.0, True, dtype, device)


def xavier(shape: Sequence[int], dtype=None, device=None) -> Tensor:
    if len(shape) != 2:
        raise RuntimeError("xavier: 2-D shapes only")
    return _normal(shape, math.sqrt(1.0 / shape[0]), True, dtype, device)


def kaiming(shape: Sequence[int], dtype=None, device=None) -> Tensor:
    if len(shape) != 2:
        raise RuntimeError("kaiming: 2-D shapes only")
    return _normal(shape, math.sqrt(2.0 / shape[0]), True, dtype, device)


def ones(shape: Sequence[int], dtype=None, device=None) -> Tensor:
    t = Tensor(shape, False, dtype=dtype, device=device)
    K.fill_(t.data, 1.0)
    return t


def zeros(shape: Sequence[int], dtype=None, device=None) -> Tensor:
    return Tensor(shape, False, dtype=dtype, device=device)


def one_hot(idx, classes: int) -> Tensor:
    from .ops.functional import one_hot as _oh
    return _oh(idx, classes)
