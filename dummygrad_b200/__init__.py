"""dummygrad_b200: a reverse-mode autograd and training framework for NVIDIA B200.

Public surface (reference names in parentheses are kept identical):

* ``Tensor``, ``Node``, ``Edge``, ``AccumulateGrad``, ``get_grad_edge``, ``backward`` - the engine
* ``ops`` / top-level functions - the 40 differentiable ops (``add`` ... ``gelu``) and fused nodes
* ``init`` - ``manual_seed randn xavier kaiming one_hot ones zeros``
* ``optim`` - ``SGD``, ``Adam``, ``AdamW``
* ``models`` - ``Linear LayerNorm Embedding SelfAttention MultiHeadAttention FeedForward
  TransformerBlock GPT`` + ``MLP``, ``Mars``
* ``parallel`` - data / tensor parallel training over NVLink with fused compute+collective kernels
* ``utils`` - checkpointing, config, metrics, profiler
"""
from . import _lib
from .tensor import (ONE, AccumulateGrad, Edge, Node, Tensor, backward, default_device, default_dtype, get_grad_edge,
                     make_contiguous, make_strides, set_default_device, set_default_dtype, tensor_add_inplace, unravel)
from .ops.functional import *  # noqa: F401,F403 - the op set is the API
from .ops import functional as _functional
from . import init, optim
from .init import kaiming, manual_seed, ones, randn, xavier, zeros
from .optim import SGD, Adam, AdamW, ParamState
from . import models
from .models import (GPT, MLP, Embedding, FeedForward, LayerNorm, Linear, Mars, MultiHeadAttention, SelfAttention,
                     TransformerBlock)

__version__ = "0.1.0"


def build(verbose: bool = False) -> None:
    """Compile the native libraries in-tree."""
    from . import _build
    _build.build_all(verbose=verbose)
