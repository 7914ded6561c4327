"""GEMM microbenchmark: the tcgen05 kernel against cuBLAS (``torch.matmul``) on the 13B model's shapes.

Prints, per shape and operand layout, the time of both (CUDA events, L2 flushed between iterations by
rotating through operand copies larger than L2), TFLOP/s and the fraction of the measured bf16 peak
from ``MEASURED_PEAKS.json``.  Usage: ``python benchmarks/gemm_bench.py [--tokens 32656] [--iters 10]``.
"""

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from teletron_b200.ops import gemm_tcgen05 as G  # noqa: E402


def peak():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:
        return 1590.0


def timeit(fn, iters, rotate):
    for i in range(3):
        fn(i % rotate)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        fn(i % rotate)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32656)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    T = a.tokens
    H = 3072
    cases = [("qkv fwd", "nt", T, 3 * H, H), ("proj fwd", "nt", T, H, H), ("fc1 fwd", "nt", T, 4 * H, H),
             ("fc2 fwd", "nt", T, H, 4 * H), ("single proj_out fwd", "nt", T, H, 5 * H),
             ("qkv dgrad", "nn", T, H, 3 * H), ("fc1 dgrad", "nn", T, H, 4 * H), ("fc2 dgrad", "nn", T, 4 * H, H),
             ("qkv wgrad", "tn", 3 * H, H, T), ("fc1 wgrad", "tn", 4 * H, H, T), ("fc2 wgrad", "tn", H, 4 * H, T)]
    pk = peak()
    rows = []
    for name, layout, M, N, K in cases:
        shape_a = (M, K) if layout != "tn" else (K, M)
        shape_b = (N, K) if layout == "nt" else (K, N)
        nbytes = 2 * (shape_a[0] * shape_a[1] + shape_b[0] * shape_b[1] + M * N)
        rotate = max(2, min(8, int(300e6 // nbytes) + 1))          # working set of the rotation > L2 (126 MB)
        As = [torch.randn(*shape_a, device="cuda").bfloat16() for _ in range(rotate)]
        Bs = [(torch.randn(*shape_b, device="cuda") * 0.02).bfloat16() for _ in range(rotate)]
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)

        def ours(i):
            G.gemm(As[i], Bs[i], layout, out=out)

        def lib(i):
            if layout == "nt":
                torch.matmul(As[i], Bs[i].t(), out=out)
            elif layout == "nn":
                torch.matmul(As[i], Bs[i], out=out)
            else:
                torch.matmul(As[i].t(), Bs[i], out=out)
        t_lib = timeit(lib, a.iters, rotate)
        # the CTA-pair kernel (cluster of 2) and the single-CTA kernel, each forced in turn; the dispatcher's own choice
        # for this shape is whichever the library would pick (pairs when there is a tile per pair of SMs)
        keep = G.PAIR_KERNEL
        G.PAIR_KERNEL = False
        t_single = timeit(ours, a.iters, rotate)
        G.PAIR_KERNEL = True
        t_pair = timeit(ours, a.iters, rotate) if G.use_pair_kernel(M, N) else float("nan")
        G.PAIR_KERNEL = keep
        t_ours = timeit(ours, a.iters, rotate)
        G.check_status()
        fl = 2.0 * M * N * K / 1e12
        rows.append((name, layout, M, N, K, t_ours, fl / (t_ours / 1e3), t_lib, fl / (t_lib / 1e3)))
        print(f"{name:22s} {layout} M={M:6d} N={N:6d} K={K:6d} | 1-CTA {t_single:7.3f} ms  CTA pair {t_pair:7.3f} ms | tcgen05 {t_ours:7.3f} ms {fl / (t_ours / 1e3):7.1f} TF "
              f"({fl / (t_ours / 1e3) / pk:.2f} of measured peak) | cuBLAS {t_lib:7.3f} ms {fl / (t_lib / 1e3):7.1f} TF "
              f"| ratio {t_lib / t_ours:.2f}", flush=True)
        del As, Bs
    tot_o = sum(r[5] for r in rows)
    tot_l = sum(r[7] for r in rows)
    print(f"total: tcgen05 {tot_o:.2f} ms, cuBLAS {tot_l:.2f} ms, ratio {tot_l / tot_o:.3f}; peak used {pk} TFLOP/s")


if __name__ == "__main__":
    main()
