"""Microbenchmark of the fused tcgen05 attention kernels (forward and backward).

    python bench/attn_bench.py [--B 8] [--H 16] [--S 1024] [--dk 64] [--iters 10] [--no-causal]

Timing with CUDA events after warm-up; inputs are rotated over a pool so consecutive launches
do not hit the same lines in L2. FLOPs counted: forward 4*B*H*S^2*dk (halved when causal),
backward 2.5x forward. Fractions are against the measured cuBLAS bf16 peak.
"""
import argparse
import json
import math
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from dummygrad_b200.ops import kernels as K  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--H", type=int, default=16)
    ap.add_argument("--S", type=int, default=1024)
    ap.add_argument("--dk", type=int, default=64)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-causal", action="store_true")
    ap.add_argument("--fwd-only", action="store_true")
    a = ap.parse_args()
    causal = not a.no_causal
    D = a.H * a.dk
    pool = 3
    qs, ks, vs, gs = ([torch.randn(a.B, a.S, D, device="cuda").to(torch.bfloat16) for _ in range(pool)] for _ in range(4))
    scale = 1.0 / math.sqrt(a.dk)
    flops = 4.0 * a.B * a.H * a.S * a.S * a.dk * (0.5 if causal else 1.0)

    def timeit(fn):
        for i in range(2):
            fn(i % pool)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(a.iters):
            fn(i % pool)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / a.iters

    outs = [K.attention_fwd(qs[i], ks[i], vs[i], a.H, causal, scale) for i in range(pool)]
    ms_f = timeit(lambda i: K.attention_fwd(qs[i], ks[i], vs[i], a.H, causal, scale))
    rec = {"B": a.B, "H": a.H, "S": a.S, "dk": a.dk, "causal": causal, "fwd_ms": ms_f, "fwd_tflops": flops / ms_f / 1e9}
    if not a.fwd_only:
        ms_b = timeit(lambda i: K.attention_bwd(qs[i], ks[i], vs[i], outs[i][0], gs[i], outs[i][1], a.H, causal, scale))
        rec.update({"bwd_ms": ms_b, "bwd_tflops": 2.5 * flops / ms_b / 1e9})
    rec["status"] = K.gemm_status()
    print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
