"""Op-level profiler: device time per kernel entry point.

``with profile() as prof: ...`` wraps every launcher of the kernel library with a pair of CUDA
events on the launching stream and, on exit, reports total / count / mean microseconds per
entry point (elementwise launches are split by opcode). It replaces ``show()`` as the
debugging aid the reference offers (src/engine.h:221-258) and is what the per-step
fwd / bwd / comm / optimizer breakdown in the metrics log is built from. Profiling serialises
nothing, but the events add a few microseconds per launch: never quote timings taken under it
as benchmark numbers.
"""
from __future__ import annotations

import contextlib
from collections import defaultdict

import torch

from .. import _lib as L


class _Proxy:
    def __init__(self, lib, records, nvtx: bool = False):
        object.__setattr__(self, "_lib", lib)
        object.__setattr__(self, "_records", records)
        object.__setattr__(self, "_cache", {})
        object.__setattr__(self, "_nvtx", nvtx)

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not name.startswith("dg_") or name.endswith("_bytes") or name.endswith("_supported") or name in (
                "dg_version", "dg_device_sm_count"):
            return fn
        cached = self._cache.get(name)
        if cached is not None:
            return cached
        records = self._records
        nvtx = self._nvtx

        def wrapped(*args):
            key = name
            if name == "dg_elementwise":
                key = f"dg_elementwise[{L._EW_NAMES[args[0]]}]"
            elif name == "dg_gemm_sm100":
                g = args[0]._obj
                lay = ("n" if g.a_kmajor else "t") + ("t" if g.b_kmajor else "n")
                key = f"dg_gemm_sm100[{lay} {g.M}x{g.N}x{g.K}" + (f" b{g.batch}]" if g.batch > 1 else "]")
            if nvtx:     # a named range per launch for timeline tools; no events, no timing table
                torch.cuda.nvtx.range_push(key)
                try:
                    return fn(*args)
                finally:
                    torch.cuda.nvtx.range_pop()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            rc = fn(*args)
            e1.record()
            records.append((key, e0, e1))
            return rc

        self._cache[name] = wrapped
        return wrapped

    def __setattr__(self, name, value):
        setattr(self._lib, name, value)


class Profile:
    def __init__(self):
        self.records: list = []
        self.table: dict[str, list[float]] = {}

    def summarize(self) -> dict:
        torch.cuda.synchronize()
        agg = defaultdict(lambda: [0.0, 0])
        for key, e0, e1 in self.records:
            a = agg[key]
            a[0] += e0.elapsed_time(e1) * 1e3
            a[1] += 1
        self.table = {k: v for k, v in sorted(agg.items(), key=lambda kv: -kv[1][0])}
        return self.table

    def report(self, top: int = 40) -> str:
        if not self.table:
            self.summarize()
        total = sum(v[0] for v in self.table.values()) or 1.0
        lines = [f"{'kernel':44s} {'total_us':>12s} {'count':>8s} {'mean_us':>10s} {'share':>7s}"]
        for k, (us, n) in list(self.table.items())[:top]:
            lines.append(f"{k:44s} {us:12.1f} {n:8d} {us / n:10.2f} {100 * us / total:6.1f}%")
        lines.append(f"{'TOTAL':44s} {total:12.1f} {sum(v[1] for v in self.table.values()):8d}")
        return "\n".join(lines)


@contextlib.contextmanager
def profile(nvtx: bool = False):
    """Profile every kernel-library launch made inside the block (CUDA only). With ``nvtx=True`` each
    launch is wrapped in an NVTX range named like the table rows (kernel, layout, shape) instead of
    being timed, so that timelines of external tools are readable."""
    lib = L.load()
    prof = Profile()
    proxy = _Proxy(lib, prof.records, nvtx)
    saved = L._LIB
    L._LIB = proxy
    try:
        yield prof
    finally:
        L._LIB = saved
        prof.summarize()
