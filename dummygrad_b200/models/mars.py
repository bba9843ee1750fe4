"""The "Mars" motion model of the reference's demo program (src/mars.cpp:60-146): a Linear
encoder over 156-dim pose frames, a learned positional table added to every sequence of the
batch, one causal TransformerBlock, the last time step sliced out, and a Linear decoder that
predicts the next frame; trained with MSE, value-clipped gradients and Adam."""
from __future__ import annotations

import torch

from .. import init
from ..ops import functional as F
from ..tensor import Tensor
from .layers import Embedding, Linear, Module, TransformerBlock


class Mars(Module):
    def __init__(self, d_in: int = 156, d_model: int = 256, n_heads: int = 8, max_seq: int = 128, n_layers: int = 1,
                 dtype=None, device=None, fused: bool = True):
        self.encoder = Linear(d_in, d_model, dtype=dtype, device=device, fused=fused)
        self.pos_emb = Embedding(max_seq, d_model, dtype=dtype, device=device, fused=fused)
        self.blocks = [TransformerBlock(d_model, n_heads, True, dtype=dtype, device=device, fused=fused)
                       for _ in range(n_layers)]
        self.decoder = Linear(d_model, d_in, dtype=dtype, device=device, fused=fused)
        self.max_seq, self.d_model = max_seq, d_model
        self.fused = fused

    def forward(self, x: Tensor) -> Tensor:
        """x [B, S, d_in] -> prediction of the next frame [B, d_in]."""
        B, S, _ = x.shape
        h = self.encoder.forward(x)
        pos = torch.arange(S, device=x.device, dtype=torch.int64)
        pe = self.pos_emb.forward(pos)                 # [S, d_model]
        h = F.cast_n_add(h, pe)                        # broadcast over the batch
        for blk in self.blocks:
            h = blk.forward(h)
        return self.decoder.forward(F.slice_last(h))

    def parameters(self) -> list[Tensor]:
        p = self.encoder.parameters() + self.pos_emb.parameters()
        for blk in self.blocks:
            p += blk.parameters()
        return p + self.decoder.parameters()
