"""Attention microbenchmark: the tcgen05 kernels against torch SDPA (cuDNN and flash backends).

``python benchmarks/attn_bench.py [--seq 32656] [--heads 24] [--iters 5] [--backward]``; times with CUDA
events, reports TFLOP/s (4 * S^2 * 128 * heads forward, 2.5x that backward) and the fraction of the
measured bf16 peak.
"""

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from teletron_b200.ops import attn_tcgen05 as A  # noqa: E402
from teletron_b200.ops.gemm_tcgen05 import check_status  # noqa: E402


def peak():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:
        return 1590.0


def timeit(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32656)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--backward", action="store_true")
    a = ap.parse_args()
    S, H = a.seq, a.heads
    q, k, v = (torch.randn(1, H, S, 128, device="cuda").bfloat16() for _ in range(3))
    fl = 4.0 * S * S * 128 * H / 1e12
    pk = peak()
    t = timeit(lambda: A.forward(q, k, v, None, None), a.iters)
    check_status()
    print(f"tcgen05 fwd      S={S} H={H}: {t:8.3f} ms  {fl / (t / 1e3):7.1f} TFLOP/s  ({fl / (t / 1e3) / pk:.2f} of measured peak)")
    from torch.nn.attention import SDPBackend, sdpa_kernel
    for name, be in (("sdpa cudnn", SDPBackend.CUDNN_ATTENTION), ("sdpa flash", SDPBackend.FLASH_ATTENTION)):
        try:
            with sdpa_kernel([be]):
                t = timeit(lambda: F.scaled_dot_product_attention(q, k, v), a.iters)
            print(f"{name:16s} S={S} H={H}: {t:8.3f} ms  {fl / (t / 1e3):7.1f} TFLOP/s")
        except Exception as e:
            print(f"{name}: unavailable ({type(e).__name__}: {e})")
    if a.backward:
        qg, kg, vg = (x.clone().requires_grad_() for x in (q, k, v))
        d = torch.randn(1, S, H * 128, device="cuda").bfloat16()

        def ours():
            o = A.attention(qg, kg, vg)
            o.backward(d)
        t = timeit(ours, a.iters)
        print(f"tcgen05 fwd+bwd  : {t:8.3f} ms  {3.5 * fl / (t / 1e3):7.1f} TFLOP/s")
        # the backward alone, in both variants: one pass with dQ reduced in fp32 against the deterministic two-kernel split
        from teletron_b200.ops import attn_bwd_tcgen05 as AB
        out, lse, *_ = A.forward(q, k, v, None, None)
        for name, fused in (("one pass", True), ("two kernels", False)) * 2:
            was = AB.set_fused(fused)
            t = timeit(lambda: AB.backward(d, q, k, v, out, lse, 128 ** -0.5, S), a.iters)
            AB.set_fused(was)
            check_status()
            print(f"tcgen05 bwd {name:12s}: {t:8.3f} ms  {2.5 * fl / (t / 1e3):7.1f} useful TFLOP/s "
                  f"({2.5 * fl / (t / 1e3) / pk:.2f} of measured peak)")
        for name, be in (("sdpa cudnn", SDPBackend.CUDNN_ATTENTION), ("sdpa flash", SDPBackend.FLASH_ATTENTION)):
            try:
                with sdpa_kernel([be]):
                    def lib():
                        o = F.scaled_dot_product_attention(qg, kg, vg)
                        o.backward(d.view(1, S, H, 128).transpose(1, 2))
                    t = timeit(lib, a.iters)
                print(f"{name:16s} fwd+bwd: {t:8.3f} ms  {3.5 * fl / (t / 1e3):7.1f} TFLOP/s")
            except Exception as e:
                print(f"{name}: unavailable ({type(e).__name__}: {e})")


if __name__ == "__main__":
    main()
