"""The allocation-free column reduction, called through its exported C symbol.

Some users of the kernel library may not allocate device memory when they call it (a host
application that owns the whole memory budget, a path that must not block on the allocator).
For them ``dg_reduce_cols_noalloc`` keeps its scratch in a fixed array inside the library. This
test checks that it returns what the ordinary entry point returns, twice in a row on the same
array, and that it refuses shapes whose scratch would not fit.

The file name sorts last on purpose, so a stop-at-first-failure run has already run every other
test.
"""
import ctypes as C

import pytest
import torch

from dummygrad_b200 import _lib as L
from dummygrad_b200.ops import kernels as K

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _entry(lib):
    fn = lib.dg_reduce_cols_noalloc
    fn.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    return fn


def _call(fn, x, mode):
    B, R, Cc = x.shape
    out = torch.empty(B, Cc, dtype=x.dtype, device=x.device)
    mean = torch.empty(B, Cc, dtype=x.dtype, device=x.device)
    rc = fn(L.dtype_code(x.dtype), out.data_ptr(), mean.data_ptr(), x.data_ptr(), B, R, Cc, mode, L.stream_ptr())
    return rc, out, mean


@pytest.mark.parametrize("shape", [(3, 257, 70), (1, 4096, 1024), (2, 9, 5)])
def test_matches_allocating_entry_point_twice(shape):
    lib = L.load()
    fn = _entry(lib)
    torch.manual_seed(0)
    for attempt in range(2):                      # two calls in a row share the fixed scratch
        x = torch.randn(*shape, device="cuda") + attempt
        for mode in (L.RED_SUM, L.RED_MEAN, L.RED_VAR, L.RED_STD):
            rc, out, mean = _call(fn, x, mode)
            assert rc == 0
            ref, ref_mean = K.reduce_cols(x, mode, want_mean=True)
            torch.cuda.synchronize()
            scale = max(1.0, ref.abs().max().item())
            assert (out - ref).abs().max().item() <= TOL * scale
            if mode >= L.RED_VAR:
                assert (mean - ref_mean).abs().max().item() <= TOL * max(1.0, ref_mean.abs().max().item())


def test_bf16_and_oversize_rejected():
    lib = L.load()
    fn = _entry(lib)
    x = torch.randn(2, 300, 64, device="cuda").to(torch.bfloat16)
    rc, out, _ = _call(fn, x, L.RED_SUM)
    assert rc == 0
    ref, _ = K.reduce_cols(x, L.RED_SUM)
    torch.cuda.synchronize()
    assert (out.float() - ref.float()).abs().max().item() <= 1e-2 * max(1.0, ref.float().abs().max().item())
    # scratch need grows with B*C*splits: this shape needs more than the fixed 4 MiB
    B, R, Cc = 1, 64, 2 * 1024 * 1024
    assert lib.dg_reduce_cols_scratch_bytes(B, R, Cc) > 4 * 2 ** 20
    big = torch.zeros(B, R, Cc, device="cuda")
    rc, _, _ = _call(fn, big, L.RED_SUM)
    assert rc == -4
