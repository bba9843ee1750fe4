"""Multi-GPU training on one NVLink/NVSwitch node: process-group plumbing, symmetric peer
memory, the data-parallel trainer with the fused reduce-scatter + optimizer kernel, and the
tensor-parallel layers built on the fused all-gather->GEMM / GEMM->reduce-scatter kernels."""
from . import dist  # noqa: F401
