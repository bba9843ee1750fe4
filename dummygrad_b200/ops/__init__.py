"""Differentiable ops.

``kernels`` holds the device-level functions; ``functional`` holds the 40 autograd ops of the
reference API plus the fused nodes (linear, layer_norm, attention, softmax_cross_entropy).
``functional`` depends on :mod:`dummygrad_b200.tensor`, which itself uses ``kernels``, so the
functional names are resolved on first access (PEP 562) instead of at package import.
"""
from . import kernels  # noqa: F401


def __getattr__(name):
    import importlib
    functional = importlib.import_module(".functional", __name__)
    try:
        return getattr(functional, name)
    except AttributeError:
        raise AttributeError(f"module {__name__!r} has no attribute {name!r}") from None
