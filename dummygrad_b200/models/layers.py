"""NN modules with the reference's names, parameter shapes, initialisation and
``parameters()`` order (src/linear.h, src/layernorm.h, src/embedding.h, src/attention.h,
src/transformer.h). Modules are plain classes exposing ``forward`` and ``parameters`` by
convention, like the reference.

Every module has two execution modes with identical mathematics:

* ``fused=True`` (default): one fused node per module step - GEMM with bias/GELU/residual
  epilogue, one-kernel LayerNorm, gather embedding, fused attention.
* ``fused=False``: the reference's op-by-op composition (e.g. LayerNorm as
  mean -> cast_n_sub -> var -> add_scalar -> sqrt -> cast_n_div -> scale_n_shift), which is
  what the parity tests compare the fused path against.
"""
from __future__ import annotations

import math

import torch

from .. import init
from ..ops import functional as F
from ..ops import kernels as K
from ..tensor import Tensor


class Module:
    """Minimal base: parameter listing, train-state helpers, raw fp32 parameter (de)serialisation."""

    fused = True

    def parameters(self) -> list[Tensor]:  # pragma: no cover - interface
        raise NotImplementedError

    def zero_grad(self) -> None:
        for p in self.parameters():
            p.zero_grad()

    def num_parameters(self) -> int:
        seen, n = set(), 0
        for p in self.parameters():
            if id(p) not in seen:
                seen.add(id(p))
                n += p.size()
        return n

    def __call__(self, *a, **kw):
        return self.forward(*a, **kw)


class Linear(Module):
    """y = x W + b with W [fan_in, fan_out] ~ kaiming and b [1, fan_out] = ``bias``."""

    def __init__(self, fan_in: int, fan_out: int, bias: float = 0.0, dtype=None, device=None, fused: bool = True):
        self.W = init.kaiming([fan_in, fan_out], dtype=dtype, device=device)
        self.b = Tensor([1, fan_out], True, dtype=dtype, device=device)
        if bias != 0.0:
            self.b.fill(float(bias))
        self.fused = fused

    def forward(self, x: Tensor, act: str | None = None, residual: Tensor | None = None) -> Tensor:
        if self.fused:
            return F.linear(x, self.W, self.b, act=act, residual=residual)
        y = F.cast_n_add(F.matmul(x, self.W), self.b)
        if act == "gelu":
            y = F.gelu(y)
        elif act == "relu":
            y = F.relu(y)
        if residual is not None:
            y = F.add(y, residual)
        return y

    def parameters(self) -> list[Tensor]:
        return [self.W, self.b]


class LayerNorm(Module):
    def __init__(self, features: int, eps: float = 1e-5, dtype=None, device=None, fused: bool = True):
        self.gamma = Tensor([1, features], True, dtype=dtype, device=device)
        self.beta = Tensor([1, features], True, dtype=dtype, device=device)
        self.gamma.fill(1.0)
        self.eps = eps
        self.fused = fused

    def forward(self, x: Tensor) -> Tensor:
        if self.fused:
            return F.layer_norm(x, self.gamma, self.beta, self.eps)
        mu = F.mean(x, 1)
        xmu = F.cast_n_sub(x, mu)
        variance = F.var(x, 1)
        std = F.sqrt(F.add_scalar(variance, self.eps))
        x_norm = F.cast_n_div(xmu, std)
        return F.scale_n_shift(x_norm, self.gamma, self.beta)

    def parameters(self) -> list[Tensor]:
        return [self.gamma, self.beta]


class Embedding(Module):
    """weight [N, D] ~ xavier; forward flattens indices and returns [n, D] (src/embedding.h:19-22)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, dtype=None, device=None, fused: bool = True):
        self.weight = init.xavier([num_embeddings, embedding_dim], dtype=dtype, device=device)
        self.num_embeddings = num_embeddings
        self.fused = fused

    def forward(self, idx) -> Tensor:
        if self.fused:
            return F.embedding(self.weight, idx)
        return F.matmul(F.one_hot(idx, self.num_embeddings).to(self.weight.dtype), self.weight)

    def parameters(self) -> list[Tensor]:
        return [self.weight]


class SelfAttention(Module):
    """Single head, d_k = d_model (src/attention.h:12-46)."""

    def __init__(self, d_model: int, causal: bool = False, dtype=None, device=None, fused: bool = True):
        self.W_q = Linear(d_model, d_model, dtype=dtype, device=device, fused=fused)
        self.W_k = Linear(d_model, d_model, dtype=dtype, device=device, fused=fused)
        self.W_v = Linear(d_model, d_model, dtype=dtype, device=device, fused=fused)
        self.d_k = d_model
        self.causal = causal
        self.fused = fused

    def forward(self, x: Tensor) -> Tensor:
        q, k, v = self.W_q.forward(x), self.W_k.forward(x), self.W_v.forward(x)
        scale = 1.0 / math.sqrt(self.d_k)
        if self.fused:
            return F.attention(q, k, v, causal=self.causal, scale=scale)
        scores = F.mul_scalar(F.matmul(q, F.transpose(k, -2, -1)), scale)
        if self.causal:
            scores = F.causal_mask(scores)
        return F.matmul(F.softmax(scores), v)

    def parameters(self) -> list[Tensor]:
        return self.W_q.parameters() + self.W_k.parameters() + self.W_v.parameters()


class MultiHeadAttention(Module):
    def __init__(self, d_model: int, n_heads: int, causal: bool = False, dtype=None, device=None, fused: bool = True):
        if d_model % n_heads:
            raise ValueError("d_model must be divisible by n_heads")
        self.W_q = Linear(d_model, d_model, dtype=dtype, device=device, fused=fused)
        self.W_k = Linear(d_model, d_model, dtype=dtype, device=device, fused=fused)
        self.W_v = Linear(d_model, d_model, dtype=dtype, device=device, fused=fused)
        self.W_o = Linear(d_model, d_model, dtype=dtype, device=device, fused=fused)
        self.d_model, self.n_heads, self.d_k, self.causal = d_model, n_heads, d_model // n_heads, causal
        self.fused = fused

    def forward(self, x_in: Tensor, residual: Tensor | None = None) -> Tensor:
        x = x_in
        is_2d = x.ndim() == 2
        if is_2d:
            x = F.reshape(x, [1, x.shape[0], x.shape[1]])
        B, S = x.shape[0], x.shape[1]
        H, dk = self.n_heads, self.d_k
        scale = 1.0 / math.sqrt(dk)
        merged = None
        if self.fused and self.W_q.b is not None:
            # projections + attention as one node (their three input gradients are summed in GEMM epilogues)
            merged = F.attention_block(x, self.W_q.W, self.W_q.b, self.W_k.W, self.W_k.b, self.W_v.W, self.W_v.b, H,
                                       causal=self.causal, scale=scale)
        if merged is None:
            q, k, v = self.W_q.forward(x), self.W_k.forward(x), self.W_v.forward(x)
        if merged is not None:
            pass
        elif self.fused:
            merged = F.mha_core(q, k, v, H, causal=self.causal, scale=scale)
        else:
            qs = F.transpose(F.reshape(q, [B, S, H, dk]), 1, 2)
            ks = F.transpose(F.reshape(k, [B, S, H, dk]), 1, 2)
            vs = F.transpose(F.reshape(v, [B, S, H, dk]), 1, 2)
            scores = F.mul_scalar(F.matmul(qs, F.transpose(ks, -2, -1)), scale)
            if self.causal:
                scores = F.causal_mask(scores)
            attn = F.matmul(F.softmax(scores), vs)
            merged = F.reshape(F.transpose(attn, 1, 2), [B, S, self.d_model])
        res = residual
        if res is not None and is_2d:
            res = F.reshape(res, [1, S, self.d_model])
        out = self.W_o.forward(merged, residual=res)
        if is_2d:
            out = F.reshape(out, [S, self.d_model])
        return out

    def parameters(self) -> list[Tensor]:
        return self.W_q.parameters() + self.W_k.parameters() + self.W_v.parameters() + self.W_o.parameters()


class FeedForward(Module):
    """fc2(gelu(fc1(x))) with d_ff defaulting to 4 * d_model (src/transformer.h:11-31)."""

    def __init__(self, d_model: int, d_ff: int = 0, dtype=None, device=None, fused: bool = True):
        d_ff = d_ff or 4 * d_model
        self.fc1 = Linear(d_model, d_ff, dtype=dtype, device=device, fused=fused)
        self.fc2 = Linear(d_ff, d_model, dtype=dtype, device=device, fused=fused)
        self.fused = fused

    def forward(self, x: Tensor, residual: Tensor | None = None) -> Tensor:
        if self.fused:
            return F.mlp(x, self.fc1.W, self.fc1.b, self.fc2.W, self.fc2.b, residual=residual)
        return self.fc2.forward(self.fc1.forward(x, act="gelu"), residual=residual)

    def parameters(self) -> list[Tensor]:
        return self.fc1.parameters() + self.fc2.parameters()


class TransformerBlock(Module):
    """Pre-LN block: x1 = x + attn(ln1(x)); out = x1 + ffn(ln2(x1)) (src/transformer.h:34-66)."""

    def __init__(self, d_model: int, n_heads: int, causal: bool = True, dtype=None, device=None, fused: bool = True,
                 d_ff: int = 0):
        self.ln1 = LayerNorm(d_model, dtype=dtype, device=device, fused=fused)
        self.attn = MultiHeadAttention(d_model, n_heads, causal, dtype=dtype, device=device, fused=fused)
        self.ln2 = LayerNorm(d_model, dtype=dtype, device=device, fused=fused)
        self.ffn = FeedForward(d_model, d_ff, dtype=dtype, device=device, fused=fused)
        self.fused = fused

    def forward(self, x: Tensor) -> Tensor:
        if self.fused:
            # residual adds run in the epilogue of the out-projection / fc2 GEMMs
            x1 = self.attn.forward(self.ln1.forward(x), residual=x)
            return self.ffn.forward(self.ln2.forward(x1), residual=x1)
        x1 = F.add(x, self.attn.forward(self.ln1.forward(x)))
        return F.add(x1, self.ffn.forward(self.ln2.forward(x1)))

    def parameters(self) -> list[Tensor]:
        return self.ln1.parameters() + self.attn.parameters() + self.ln2.parameters() + self.ffn.parameters()


def scale_(t: Tensor, s: float) -> None:
    """In-place t *= s on the parameter's own buffer (initialisation-time rescale)."""
    K.ew("MUL_S", t.data, s0=s, out=t.data)
