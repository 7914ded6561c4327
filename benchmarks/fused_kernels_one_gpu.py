"""The fused compute+collective kernels on ONE GPU, with every "peer" buffer placed in this GPU's own memory.

A profiler must not wrap a multi-rank command, and kernels that wait on one another must not run as separate launches
on one GPU.  Each kernel here is a single launch that plays rank ``--rank`` of ``--ranks``: its peer pointer tables name
``--ranks`` local buffers, so the instruction stream, tile schedule, epilogue and flag protocol are those of the
multi-GPU run while the "remote" traffic stays in local HBM.  Times are therefore an upper bound on what the kernel
can do when NVLink is not the limit; the counters (tensor-pipe activity, stall reasons, bytes) are what this is for:

    python benchmarks/fused_kernels_one_gpu.py --tokens 16384 --ranks 4
    ncu --set full --clock-control none -k regex:gemm_kernel -c 3 -o prof python benchmarks/fused_kernels_one_gpu.py --tokens 16384 --ranks 4 --iters 1

Kernels: (a) QKV GEMM + QK-RMSNorm + RoPE + sequence->head scatter, (c) all-gather->GEMM with copier warps,
(c) GEMM->reduce-scatter push, (d) gradient reduce-scatter by peer loads.
"""

import argparse
import ctypes
import json
import os
import sys

import torch

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..")))

from teletron_b200.ops._lib import c_float, c_int, c_long, call, ptr, stream  # noqa: E402
from teletron_b200.ops.gemm_tcgen05 import check_status, status_tensor  # noqa: E402

BF16 = torch.bfloat16


def table(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def timeit(fn, iters):
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
    ap.add_argument("--tokens", type=int, default=16384, help="tokens held by the emulated rank")
    ap.add_argument("--ranks", type=int, default=4)
    ap.add_argument("--rank", type=int, default=1)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--hidden", type=int, default=3072)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--ffn", type=int, default=12288)
    a = ap.parse_args()
    n, me, s, H, heads = a.ranks, a.rank, a.tokens, a.hidden, a.heads
    if heads % n or not 0 <= me < n:
        raise SystemExit("heads must divide by ranks and 0 <= rank < ranks")
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *shape, scale=1.0: (torch.randn(*shape, device=dev, generator=g) * scale).to(BF16)  # noqa: E731
    st = status_tensor(dev)
    res = {"tokens": s, "ranks": n, "rank": me}

    # (a) fused QKV: every "owner rank" gets its own q / k / v buffer [heads / n, n * s, 128]
    x = rnd(s, H)
    w, b = rnd(heads * 384, H, scale=0.02), rnd(heads * 384, scale=0.02)
    qw, kw = torch.ones(128, device=dev, dtype=BF16), torch.ones(128, device=dev, dtype=BF16)
    cos, sin = torch.rand(s, 128, device=dev, generator=g), torch.rand(s, 128, device=dev, generator=g)
    S_tot = n * s
    qb, kb, vb = ([torch.empty(heads // n, S_tot, 128, device=dev, dtype=BF16) for _ in range(n)] for _ in range(3))
    aux = torch.empty(s, heads * 384, device=dev, dtype=BF16)

    def qkv():
        call("tt_qkv_gemm_fused", ptr(x), ptr(w), ptr(b), ptr(qw), ptr(kw), ptr(cos), ptr(sin), table(qb), table(kb), table(vb),
             c_int(n), c_int(me), ptr(aux), c_int(s), c_int(heads), c_int(H), c_int(s), c_int(S_tot), c_int(me * s), c_int(s),
             c_int(0), c_float(1e-6), ptr(st), stream())
    ms = timeit(qkv, a.iters)
    res["a_qkv_norm_rope_scatter"] = {"ms": ms, "tflops": 2.0 * s * H * heads * 384 / ms / 1e9,
                                      "checksum": sum(float(t[:, me * s:(me + 1) * s].float().abs().sum()) for t in qb + kb + vb)}

    # (c) all-gather -> GEMM: n row blocks of [s / n, H] (all local), column-parallel weight [ffn / n, H]
    rows = s // n // 8 * 8
    blocks = [rnd(rows, H) for _ in range(n)]
    w1 = rnd(a.ffn // n, H, scale=0.02)
    out = torch.empty(n * rows, a.ffn // n, device=dev, dtype=BF16)
    stage = torch.empty(n * rows, H, device=dev, dtype=BF16)
    flags = torch.zeros(n * ((rows + 127) // 128), dtype=torch.int32, device=dev)
    epoch = [0]

    def ag():
        epoch[0] += 1
        call("tt_gemm_ag_bf16", table(blocks), c_int(n), c_int(me), c_int(rows), ptr(w1), c_int(0), c_long(H), ptr(out),
             c_long(a.ffn // n), None, None, c_int(a.ffn // n), c_int(H), c_int(0), ptr(stage), ptr(flags), c_int(epoch[0]),
             ptr(st), stream())
    ms = timeit(ag, a.iters)
    res["c_all_gather_gemm"] = {"ms": ms, "tflops": 2.0 * n * rows * H * (a.ffn // n) / ms / 1e9}

    # (c) GEMM -> reduce-scatter: partial [n * rows, H] tiles pushed into the owners' landing zones [n, rows, H]
    xk = rnd(n * rows, a.ffn // n)
    w2 = rnd(H, a.ffn // n, scale=0.02)
    zones = [torch.empty(n, rows, H, device=dev, dtype=BF16) for _ in range(n)]

    def rs():
        call("tt_gemm_comm_bf16", table([xk]), c_int(n), c_int(0), c_long(n * rows), c_int(0), c_int(0), None, c_long(0),
             ptr(w2), c_int(0), c_long(a.ffn // n), None, c_long(0), None, c_int(n * rows), c_int(H), c_int(a.ffn // n),
             c_int(rows), c_int(me), c_int(2), table(zones), c_int(0), c_int(0), c_long(H), None, None, c_int(0), ptr(st), stream())
    ms = timeit(rs, a.iters)
    res["c_gemm_reduce_scatter_push"] = {"ms": ms, "tflops": 2.0 * n * rows * H * (a.ffn // n) / ms / 1e9,
                                         "checksum": sum(float(z[me].float().abs().sum()) for z in zones)}

    # (d) gradient reduce-scatter: this rank's shard of n "peer" gradient buffers
    count = 64 << 20
    grads = [rnd(count) for _ in range(n)]
    shard = count // n // 8 * 8
    red = torch.empty(shard, device=dev, dtype=BF16)

    def grs():
        call("tt_reduce_scatter_bf16", table(grads), c_int(n), c_long(me * shard), ptr(red), c_long(shard), c_float(1.0 / n), stream())
    ms = timeit(grs, a.iters)
    res["d_grad_reduce_scatter"] = {"ms": ms, "read_gbs": n * shard * 2 / ms / 1e6}

    check_status()
    print(json.dumps(res, indent=1))


if __name__ == "__main__":
    main()
