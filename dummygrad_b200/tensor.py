"""Tensor and the reverse-mode engine.

Capabilities follow the reference's core runtime (src/engine.h): a strided ``Tensor`` with
``requires_grad / grad / grad_fn / grad_accumulator``, ``Edge``/``Node`` graph vertices with a
public ``apply`` extension point (src/engine.h:22-42), ``AccumulateGrad`` leaf sinks whose
gradients accumulate across backward calls (src/engine.h:298-312) and a scalar-rooted
``backward(retain_graph)`` that walks the graph in topological (Kahn) order
(src/engine.h:325-399).

Design differences, on purpose:

* Storage is a device buffer (``torch.Tensor`` is used as allocator + strided view metadata
  with int64 sizes); every arithmetic step on CUDA is one of this package's sm_100a kernels
  enqueued on the current stream, so ``backward`` is a stream-ordered kernel sequence.
* Gradients are values: a gradient handed to two consumers is never accumulated into in place
  unless the engine owns it, and strided views are normalised at node boundaries. (The
  reference aliases the incoming gradient in add/sub and reads strided gradients as if they
  were contiguous: src/ops.h:8,49; src/transpose.h:13; src/engine.h:280-295.)
* In-degree counting is iterative, so graph depth is not limited by the Python stack
  (the reference recurses: src/engine.h:334-350).
* Leaf hooks fire when a parameter's gradient for the current backward is final; the data-
  parallel layer uses them to launch the fused reduce-scatter + optimizer per bucket while
  the rest of backward is still running.
"""
from __future__ import annotations

import math
import weakref
from collections import deque
from typing import Callable, Iterable, Sequence

import torch

from .ops import kernels as K

_DEFAULT_DEVICE: torch.device | None = None
_DEFAULT_DTYPE = torch.float32


def default_device() -> torch.device:
    global _DEFAULT_DEVICE
    if _DEFAULT_DEVICE is None:
        _DEFAULT_DEVICE = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() \
            else torch.device("cpu")
    return _DEFAULT_DEVICE


def set_default_device(dev) -> None:
    global _DEFAULT_DEVICE
    _DEFAULT_DEVICE = torch.device(dev)


def set_default_dtype(dt: torch.dtype) -> None:
    global _DEFAULT_DTYPE
    assert dt in (torch.float32, torch.bfloat16)
    _DEFAULT_DTYPE = dt


def default_dtype() -> torch.dtype:
    return _DEFAULT_DTYPE


class _ImplicitOne:
    """Seed gradient of exactly 1.0 for the backward root; nodes may skip the multiply."""

    def __repr__(self):
        return "ONE"


ONE = _ImplicitOne()


def materialize(g, shape, dtype, device) -> torch.Tensor:
    """Turn the implicit seed into a real tensor of ones."""
    if g is ONE:
        t = torch.empty(tuple(shape), dtype=dtype, device=device)
        return K.fill_(t, 1.0)
    return g


def make_strides(shape: Sequence[int]) -> list[int]:
    """Row-major strides (src/engine.h:52-60)."""
    if len(shape) == 0:
        raise ValueError("0-d tensors are not supported")
    strides = [1] * len(shape)
    for i in range(len(shape) - 2, -1, -1):
        strides[i] = strides[i + 1] * shape[i + 1]
    return strides


def unravel(flat: int, shape: Sequence[int]) -> list[int]:
    """Flat index -> multi-index (src/engine.h:63-73)."""
    idx = [0] * len(shape)
    for i in range(len(shape) - 1, -1, -1):
        idx[i] = flat % shape[i]
        flat //= shape[i]
    return idx


class Edge:
    __slots__ = ("function", "input_slot")

    def __init__(self, function: "Node | None", input_slot: int = 0):
        self.function = function
        self.input_slot = input_slot


class Node:
    """A vertex of the backward graph. Subclass and implement ``apply`` to add an op.

    ``apply(grads)`` receives ``[g]`` (one output-gradient slot; ``g`` is a contiguous
    ``torch.Tensor`` or :data:`ONE`) and returns one gradient (or ``None``) per entry of
    ``next_edges``.
    """

    # A node whose first returned gradient (the one for next_edges[0]) can absorb another gradient of
    # the same input sets this to True. The engine then offers the gradient that is already waiting
    # for that input in ``self._input_grad_addend``; a node that adds it inside its own kernel sets
    # the attribute back to None and returns the sum.
    fuse_input_grad = False

    def __init__(self):
        self.next_edges: list[Edge] = []
        self._grad_owned = False
        self._input_grad_addend = None

    def add_next_edge(self, function: "Node | None", slot: int = 0) -> None:
        self.next_edges.append(Edge(function, slot))

    def apply(self, grads: list):  # pragma: no cover - interface
        raise NotImplementedError

    def release_variables(self) -> None:
        pass

    @property
    def name(self) -> str:
        return type(self).__name__


class AccumulateGrad(Node):
    """Leaf sink: ``var.grad += g`` (src/engine.h:298-312)."""

    def __init__(self, var: "Tensor"):
        super().__init__()
        self.var = weakref.ref(var)

    def apply(self, grads: list):
        var = self.var()
        if var is None:
            return []
        g = grads[0]
        g = materialize(g, var.data.shape, var.data.dtype, var.data.device)
        if g.dtype != var.data.dtype:
            g = K.cast(g, var.data.dtype)
            self._grad_owned = True
        if tuple(g.shape) != tuple(var.data.shape):
            g = g.reshape(var.data.shape)
        sink = var._grad_sink
        if sink is not None:
            # pre-allocated gradient storage (e.g. a view into a data-parallel bucket)
            if g.data_ptr() == sink.data_ptr():
                pass    # the producing kernel wrote (or the engine summed) straight into the sink
            elif var._sink_filled:
                K.accumulate_(sink, K.contiguous(g))
            else:
                K.assign_(sink, K.contiguous(g))
                var._sink_filled = True
            if var.grad is None:
                var.grad = Tensor._wrap(sink, requires_grad=False)
        elif var.grad is None:
            if not (self._grad_owned and g.is_contiguous()):
                g = K.ew("COPY", K.contiguous(g))
            var.grad = Tensor._wrap(g, requires_grad=False)
        else:
            K.accumulate_(var.grad.data, K.contiguous(g))
        for hook in var._post_acc_hooks:
            hook(var)
        return []


def get_grad_edge(t: "Tensor") -> Edge:
    """Null edge if no grad is needed, else grad_fn, else the lazily created accumulator
    (src/engine.h:315-322)."""
    if not t.requires_grad:
        return Edge(None, 0)
    if t.grad_fn is not None:
        return Edge(t.grad_fn, 0)
    if t.grad_accumulator is None:
        t.grad_accumulator = AccumulateGrad(t)
    return Edge(t.grad_accumulator, 0)


class Tensor:
    """Strided n-d array with autograd metadata (src/engine.h:76-261)."""

    __slots__ = ("data", "requires_grad", "grad", "grad_fn", "grad_accumulator", "_post_acc_hooks", "_grad_sink",
                 "_sink_filled", "name", "__weakref__")

    def __init__(self, shape: Sequence[int], requires_grad: bool = True, dtype: torch.dtype | None = None,
                 device=None):
        shape = [int(s) for s in shape]
        if len(shape) == 0:
            raise ValueError("0-d tensors are not supported")
        self.data = torch.zeros(shape, dtype=dtype or _DEFAULT_DTYPE, device=device or default_device())
        self._init_meta(requires_grad)

    def _init_meta(self, requires_grad: bool) -> None:
        self.requires_grad = bool(requires_grad)
        self.grad: Tensor | None = None
        self.grad_fn: Node | None = None
        self.grad_accumulator: Node | None = None
        self._post_acc_hooks: list[Callable] = []
        self._grad_sink: torch.Tensor | None = None
        self._sink_filled = False
        self.name = None

    @classmethod
    def _wrap(cls, data: torch.Tensor, requires_grad: bool = False) -> "Tensor":
        t = cls.__new__(cls)
        t.data = data
        t._init_meta(requires_grad)
        return t

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_torch(cls, data: torch.Tensor, requires_grad: bool = False) -> "Tensor":
        if data.dim() == 0:
            data = data.reshape(1)
        return cls._wrap(data, requires_grad)

    @classmethod
    def from_list(cls, values, shape=None, requires_grad: bool = False, dtype=None, device=None) -> "Tensor":
        t = torch.tensor(values, dtype=torch.float32)
        if shape is not None:
            t = t.reshape(list(shape))
        if t.dim() == 0:
            t = t.reshape(1)
        t = t.to(device or default_device())
        if dtype is not None and dtype != torch.float32:
            t = K.cast(t, dtype)
        return cls._wrap(t, requires_grad)

    # ------------------------------------------------------------------ metadata
    @property
    def shape(self) -> list[int]:
        return list(self.data.shape)

    @property
    def strides(self) -> list[int]:
        return list(self.data.stride())

    @property
    def offset(self) -> int:
        return self.data.storage_offset()

    @property
    def dtype(self) -> torch.dtype:
        return self.data.dtype

    @property
    def device(self) -> torch.device:
        return self.data.device

    def ndim(self) -> int:
        return self.data.dim()

    def size(self) -> int:
        return self.data.numel()

    def is_contiguous(self) -> bool:
        return self.data.is_contiguous()

    def flat_idx(self, indices: Sequence[int]) -> int:
        return sum(int(i) * s for i, s in zip(indices, self.data.stride()))

    # ------------------------------------------------------------------ element access (host round trip)
    def _storage_view(self, t: torch.Tensor) -> torch.Tensor:
        n = t.untyped_storage().nbytes() // t.element_size() - t.storage_offset()
        return torch.as_strided(t, (n,), (1,), t.storage_offset())

    def data_at(self, i: int) -> float:
        """Element ``i`` in storage order from this view's offset (src/engine.h:111)."""
        return float(self._storage_view(self.data)[i].item())

    def grad_at(self, i: int) -> float:
        if self.grad is None:
            return 0.0
        return float(self.grad._storage_view(self.grad.data)[i].item())

    def item(self) -> float:
        if self.size() != 1:
            raise RuntimeError("item() needs a one-element tensor")
        return float(self.data.reshape(-1)[0].item())

    def tolist(self):
        return self.data.float().cpu().tolist()

    def numpy(self):
        return self.data.detach().float().cpu().numpy()

    # ------------------------------------------------------------------ mutation
    def zero_grad(self) -> None:
        """Drop the gradient (src/engine.h:138-140). A bucket-backed gradient keeps its storage."""
        self.grad = None
        self._sink_filled = False

    def fill(self, values) -> "Tensor":
        """Copy a flat sequence in logical order; stride-aware (src/engine.h:143-154)."""
        if isinstance(values, (int, float)):
            if self.data.is_contiguous():
                K.fill_(self.data, float(values))
            else:
                tmp = torch.empty(self.data.shape, dtype=self.data.dtype, device=self.data.device)
                K.strided_copy(self.data, K.fill_(tmp, float(values)))
            return self
        src = torch.as_tensor(values, dtype=torch.float32).reshape(-1)
        if src.numel() != self.size():
            raise RuntimeError(f"fill: got {src.numel()} values for a tensor of {self.size()} elements")
        src = src.reshape(self.data.shape).to(self.data.device)
        if src.dtype != self.data.dtype:
            src = K.cast(src, self.data.dtype)
        K.strided_copy(self.data, src)
        return self

    # ------------------------------------------------------------------ views without autograd
    def _view(self, shape: Sequence[int]) -> "Tensor":
        """Alias the storage with a new shape; contiguous tensors only (src/engine.h:157-170)."""
        if not self.data.is_contiguous():
            raise RuntimeError("view: tensor is not contiguous")
        if math.prod(shape) != self.size():
            raise RuntimeError("view: element count differs")
        return Tensor._wrap(self.data.view(list(shape)), self.requires_grad)

    def _reshape(self, shape: Sequence[int]) -> "Tensor":
        """View when contiguous, otherwise a stride-aware gather copy (src/engine.h:173-194)."""
        if math.prod(shape) != self.size():
            raise RuntimeError("reshape: element count differs")
        return Tensor._wrap(K.contiguous(self.data).view(list(shape)), self.requires_grad)

    def _transpose(self, d0: int = -2, d1: int = -1) -> "Tensor":
        """Swap two axes; zero-copy (src/engine.h:201-218)."""
        return Tensor._wrap(self.data.transpose(d0, d1), self.requires_grad)

    def contiguous(self) -> "Tensor":
        return self if self.data.is_contiguous() else Tensor._wrap(K.contiguous(self.data), self.requires_grad)

    def detach(self) -> "Tensor":
        return Tensor._wrap(self.data, False)

    def to(self, dtype: torch.dtype) -> "Tensor":
        return Tensor._wrap(K.cast(self.data, dtype), self.requires_grad)

    # autograd-aware forms live in ops; bound here for convenience
    def reshape(self, shape):
        from . import ops
        return ops.reshape(self, shape)

    def view(self, shape):
        from . import ops
        return ops.view(self, shape)

    def transpose(self, d0=-2, d1=-1):
        from . import ops
        return ops.transpose(self, d0, d1)

    # ------------------------------------------------------------------ printing
    def _format(self, t: torch.Tensor) -> str:
        def rec(x):
            if isinstance(x, list):
                return "[" + ", ".join(rec(v) for v in x) + "]"
            return f"{x:g}"
        shape = ",".join(str(s) for s in t.shape)
        return rec(t.float().cpu().tolist()) + f", shape=({shape})"

    def show(self) -> None:
        print(self._format(self.data))

    def show_grad(self) -> None:
        print("None" if self.grad is None else self._format(self.grad.data))

    def __repr__(self) -> str:
        return f"Tensor(shape={self.shape}, dtype={self.dtype}, device={self.device}, requires_grad={self.requires_grad})"

    # ------------------------------------------------------------------ hooks
    def register_post_accumulate_hook(self, fn: Callable[["Tensor"], None]) -> None:
        self._post_acc_hooks.append(fn)

    def set_grad_sink(self, buf: torch.Tensor | None) -> None:
        """Make gradients of this leaf accumulate into ``buf`` (same shape/dtype, contiguous)."""
        if buf is not None:
            assert tuple(buf.shape) == tuple(self.data.shape) and buf.dtype == self.data.dtype and buf.is_contiguous()
        self._grad_sink = buf
        self._sink_filled = False
        self.grad = None

    def claim_grad_sink(self) -> torch.Tensor | None:
        """For backward nodes that can write a parameter gradient anywhere: the gradient sink, if this
        leaf has one that holds nothing yet this step (the caller must then produce the COMPLETE
        gradient contribution in it and return it as the gradient), else None. Claiming marks the
        sink as filled, so a second use of the same parameter accumulates instead of overwriting."""
        if self._grad_sink is None or self._sink_filled:
            return None
        self._sink_filled = True
        return self._grad_sink

    # ------------------------------------------------------------------ backward
    def backward(self, retain_graph: bool = False) -> None:
        backward(self, retain_graph)


def _is_owned(og: torch.Tensor, incoming, outs: list) -> bool:
    if og is incoming:
        return False
    if og._base is not None:
        return False
    return sum(1 for o in outs if o is og) == 1


def backward(root: Tensor, retain_graph: bool = False) -> None:
    """Reverse-mode sweep from a one-element root (src/engine.h:325-399)."""
    if root.size() != 1:
        raise RuntimeError("backward() can only be called on a scalar (one-element) tensor")
    root.grad = Tensor._wrap(K.fill_(torch.empty_like(root.data, memory_format=torch.contiguous_format), 1.0), False)
    root_fn = root.grad_fn
    if root_fn is None:
        return
    # iterative in-degree count
    indeg: dict[Node, int] = {root_fn: 0}
    stack = [root_fn]
    while stack:
        n = stack.pop()
        for e in n.next_edges:
            f = e.function
            if f is None:
                continue
            if f in indeg:
                indeg[f] += 1
            else:
                indeg[f] = 1
                stack.append(f)
    ready: deque[Node] = deque([root_fn])
    slots: dict[Node, list] = {root_fn: [ONE, False]}
    while ready:
        node = ready.popleft()
        slot = slots.pop(node, None)
        edges = node.next_edges
        fused_first = False
        if slot is None:
            outs: list = [None] * len(edges)
            g = None
        else:
            g, owned = slot
            node._grad_owned = owned
            offered = None
            if node.fuse_input_grad and edges and edges[0].function is not None:
                waiting = slots.get(edges[0].function)
                if waiting is not None and waiting[0] is not ONE and waiting[0].is_contiguous():
                    offered = node._input_grad_addend = waiting[0]
            outs = list(node.apply([g]) or [])
            if offered is not None:
                if node._input_grad_addend is None and outs and outs[0] is not None:
                    fused_first = True          # outs[0] already contains the waiting gradient
                node._input_grad_addend = None
        for i, e in enumerate(edges):
            f = e.function
            if f is None:
                continue
            og = outs[i] if i < len(outs) else None
            if i == 0 and fused_first and og is not None:
                slots[f] = [og, True]
                og = None
            if og is not None:
                cur = slots.get(f)
                if cur is None:
                    if og is ONE:
                        slots[f] = [ONE, False]
                    else:
                        slots[f] = [og, _is_owned(og, g, outs)]
                else:
                    a = cur[0]
                    if a is ONE or og is ONE:
                        ref = og if a is ONE else a
                        a = materialize(a, ref.shape, ref.dtype, ref.device)
                        og = materialize(og, ref.shape, ref.dtype, ref.device)
                        cur[1] = cur[1] if cur[0] is not ONE else True
                    if og.dtype != a.dtype:
                        og = K.cast(og, a.dtype)
                    if cur[1] and a.is_contiguous():
                        K.accumulate_(a, K.contiguous(og))
                        cur[0] = a
                    else:
                        cur[0] = K.ew("ADD", K.contiguous(a), K.contiguous(og).reshape(a.shape))
                        cur[1] = True
            indeg[f] -= 1
            if indeg[f] == 0:
                ready.append(f)
        if not retain_graph:
            node.next_edges = []
            node.release_variables()


def tensor_add_inplace(dst: Tensor | None, src: Tensor) -> Tensor:
    """``dst += src`` honouring strides; clones ``src`` when ``dst`` is None (src/engine.h:280-295)."""
    if dst is None:
        return Tensor._wrap(K.ew("COPY", K.contiguous(src.data)), False)
    if dst.data.is_contiguous():
        K.accumulate_(dst.data, K.contiguous(src.data))
    else:
        tmp = K.ew("ADD", K.contiguous(dst.data), K.contiguous(src.data))
        K.strided_copy(dst.data, tmp)
    return dst


def make_contiguous(t: Tensor) -> Tensor:
    """Identity when contiguous, else a gather copy with no autograd node (src/engine.h:265-275)."""
    return t.contiguous()


def parameters_of(objs: Iterable) -> list[Tensor]:
    out: list[Tensor] = []
    for o in objs:
        out.extend(o.parameters())
    return out
