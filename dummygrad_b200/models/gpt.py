"""Weight-tied pre-LN GPT decoder (src/transformer.h:69-144).

``GPT(vocab, max_seq, d_model, n_heads, n_layers)`` keeps the reference constructor, the
1/sqrt(2 * n_layers) rescale of every block's attention out-projection and second FFN
matrix, the parameter order (token table, position table, blocks, final LayerNorm) and
``forward(input_ids, pos_ids) -> logits``.

Beyond the reference: ``forward`` accepts a batch ([B, S] ids; the reference handles one
sequence per call because its embedding flattens), ``loss`` runs the fused
logits -> cross-entropy kernel, and ``d_ff`` can be set for the 350M / 1.3B presets.
"""
from __future__ import annotations

import math

import torch

from ..ops import functional as F
from ..ops import kernels as K
from ..tensor import Tensor
from .layers import Embedding, LayerNorm, Module, TransformerBlock, scale_


class GPT(Module):
    def __init__(self, vocab_size: int, max_seq_len: int, d_model: int, n_heads: int, n_layers: int, d_ff: int = 0,
                 dtype=None, device=None, fused: bool = True):
        self.token_emb = Embedding(vocab_size, d_model, dtype=dtype, device=device, fused=fused)
        self.pos_emb = Embedding(max_seq_len, d_model, dtype=dtype, device=device, fused=fused)
        self.blocks: list[TransformerBlock] = []
        scale = 1.0 / math.sqrt(2.0 * n_layers)
        for _ in range(n_layers):
            blk = TransformerBlock(d_model, n_heads, True, dtype=dtype, device=device, fused=fused, d_ff=d_ff)
            scale_(blk.attn.W_o.W, scale)
            scale_(blk.ffn.fc2.W, scale)
            self.blocks.append(blk)
        self.ln_f = LayerNorm(d_model, dtype=dtype, device=device, fused=fused)
        self.vocab_size, self.max_seq_len, self.d_model = vocab_size, max_seq_len, d_model
        self.n_heads, self.n_layers = n_heads, n_layers
        self.fused = fused

    # ------------------------------------------------------------------ forward
    def hidden(self, input_ids, pos_ids=None) -> Tensor:
        """Final-LayerNorm hidden states, [n, d] for flat ids or [B, S, d] for [B, S] ids."""
        ids = input_ids.data if isinstance(input_ids, Tensor) else input_ids
        batched = ids.dim() == 2
        B, S = (ids.shape[0], ids.shape[1]) if batched else (1, ids.numel())
        if pos_ids is None:
            pos = torch.arange(S, device=ids.device, dtype=torch.int64).repeat(B)
        else:
            pos = pos_ids.data if isinstance(pos_ids, Tensor) else pos_ids
        if self.fused:
            x = F.embedding(self.token_emb.weight, ids, self.pos_emb.weight, pos)
        else:
            x = F.add(self.token_emb.forward(ids), self.pos_emb.forward(pos))
        if batched:
            x = F.reshape(x, [B, S, self.d_model])
        for blk in self.blocks:
            x = blk.forward(x)
        return self.ln_f.forward(x)

    def forward(self, input_ids, pos_ids=None) -> Tensor:
        """Logits through the weight-tied head: x_norm @ token_emb.weight^T."""
        x = self.hidden(input_ids, pos_ids)
        return F.matmul(x, F.transpose(self.token_emb.weight, 0, 1))

    def loss(self, input_ids, targets, pos_ids=None, reduction: str = "mean") -> Tensor:
        """Next-token cross-entropy with integer targets (fused logits -> loss kernel)."""
        logits = self.forward(input_ids, pos_ids)
        if self.fused:
            return F.softmax_cross_entropy(logits, targets, reduction=reduction, inplace_grad=True)
        V = self.vocab_size
        probs = F.softmax(F.reshape(logits, [logits.size() // V, V]))
        onehot = F.one_hot(targets, V).to(probs.dtype)
        loss = F.cross_entropy(probs, onehot)
        return F.mul_scalar(loss, float(V)) if reduction == "mean" else loss

    def parameter_names(self) -> list[str]:
        return gpt_parameter_names(len(self.blocks))

    def parameters(self) -> list[Tensor]:
        p = self.token_emb.parameters() + self.pos_emb.parameters()
        for blk in self.blocks:
            p += blk.parameters()
        return p + self.ln_f.parameters()


def gpt_parameter_names(n_layers: int) -> list[str]:
    """Names of a GPT's parameters in parameters() order (used by checkpoints)."""
    out = ["token_emb.weight", "pos_emb.weight"]
    for i in range(n_layers):
        b = f"blocks.{i}."
        out += [b + "ln1.gamma", b + "ln1.beta"]
        out += [b + f"attn.W_{x}.{y}" for x in "qkvo" for y in "Wb"]
        out += [b + "ln2.gamma", b + "ln2.beta", b + "ffn.fc1.W", b + "ffn.fc1.b", b + "ffn.fc2.W", b + "ffn.fc2.b"]
    return out + ["ln_f.gamma", "ln_f.beta"]


PRESETS = {
    # name: (vocab, max_seq, d_model, n_heads, n_layers, d_ff)
    "toy": (256, 32, 64, 4, 2, 256),
    "gpt350m": (50304, 1024, 1024, 16, 24, 4096),
    "gpt1p3b": (50304, 2048, 2048, 16, 24, 8192),
}


def build_preset(name: str, dtype=None, device=None, fused: bool = True) -> GPT:
    v, s, d, h, l, ff = PRESETS[name]
    return GPT(v, s, d, h, l, d_ff=ff, dtype=dtype, device=device, fused=fused)
