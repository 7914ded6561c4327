"""Memory-bound kernels against the HBM roofline, and against the reference's own CUDA kernels on the same GPU.

For every kernel: CUDA-event time over buffers rotated through more than the L2 (126 MB), the algorithmic bytes
(every operand read once, every result written once), the achieved GB/s and its fraction of the measured copy
bandwidth in ``MEASURED_PEAKS.json``.  Kernels: LayerNorm + modulation forward / backward (plain and fused with the
gated residual), gated residual, RMSNorm forward / backward, QKV post-processing forward / backward, GELU forward /
backward, AdamW (both state layouts), the fused reduce + AdamW + all-gather with local peers, and the gradient
reduce-scatter / parameter all-gather kernels with local peers.

``--build-reference`` compiles the reference's two extensions (``teletron_op/fused_adaln``, ``teletron_op/fused_rmsnorm``)
from their unmodified sources into ``baseline/_ref_ops`` for sm_100a (the only change is the ``-gencode`` flag of
``adaln_setup.py:23-24`` / ``rms_setup.py:19-22``); nvcc cross-compiles, so this runs without a GPU.  When the built
modules are present, ``torch_launch_adaln_forward / backward`` and ``torch_launch_rms_forward / backward`` are timed on
the same buffers, inside the domain where those kernels are defined: cols 3072 (AdaLN) / 128 (RMSNorm), one batch, row
counts that are multiples of 64, non-zero weights (``rms_forward.cu:58-99`` loops with a block-wide barrier over
``rows >> 4`` or ``rows >> 6`` blocks; ``rms_backward.cu:83-85`` divides by the weight).

    python benchmarks/norm_bench.py --build-reference --reference-src <path to the reference>/teletron_op
    python benchmarks/norm_bench.py [--tokens 32768] [--iters 10]
"""

import argparse
import ctypes
import importlib.util
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
REF_OPS = os.path.join(ROOT, "baseline", "_ref_ops")
BF16 = torch.bfloat16


def hbm_peak():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"], "of measured"
    except Exception:
        return 6650.0, "of fallback"


def build_reference(src: str) -> None:
    """nvcc + torch headers, no GPU needed.  Sources are compiled where they are (read-only is fine); objects and the
    two modules land in baseline/_ref_ops."""
    from torch.utils.cpp_extension import load
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    flags = ["-O3", "-DENABLE_BF16", "--use_fast_math", "-gencode=arch=compute_100a,code=sm_100a"]
    for name, sub, files in (("fused_adaln", "fused_adaln", ["adaln_ops.cpp", "adaln_forward.cu", "adaln_backward.cu", "scale_shift_backward.cu"]),
                             ("fused_rmsnorm", "fused_rmsnorm", ["rms_ops.cpp", "rms_forward.cu", "rms_backward.cu", "weight_backward.cu"])):
        out = os.path.join(REF_OPS, name)
        os.makedirs(out, exist_ok=True)
        d = os.path.join(src, sub)
        load(name=name, sources=[os.path.join(d, f) for f in files], extra_include_paths=[os.path.join(d, "include")],
             extra_cflags=["-O3"], extra_cuda_cflags=flags, build_directory=out, is_python_module=False, verbose=True)
        print("built", os.path.join(out, name + ".so"))


def load_reference():
    mods = {}
    for name in ("fused_adaln", "fused_rmsnorm"):
        path = os.path.join(REF_OPS, name, name + ".so")
        if not os.path.isfile(path):
            return None
        spec = importlib.util.spec_from_file_location(name, path)
        m = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(m)
        mods[name] = m
    return mods


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
    ap.add_argument("--tokens", type=int, default=32768, help="rows of the [tokens, 3072] activations (a multiple of 64)")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--build-reference", action="store_true")
    ap.add_argument("--reference-src", type=str, default=None, help="path of the reference's teletron_op directory")
    ap.add_argument("--json", type=str, default=None)
    ap.add_argument("--only", type=str, default=None, choices=["ln", "gate", "gelu", "rms", "qkvpost", "adam"],
                    help="run one kernel group only (keeps a profiler capture short)")
    a = ap.parse_args()
    want = lambda grp: a.only is None or a.only == grp  # noqa: E731
    if a.build_reference:
        if not a.reference_src:
            raise SystemExit("--build-reference needs --reference-src")
        build_reference(a.reference_src)
        return
    if a.tokens % 64:
        raise SystemExit("--tokens must be a multiple of 64 (the reference's RMSNorm kernels are only defined there)")
    from teletron_b200.ops import _lib
    from teletron_b200.ops._lib import c_float, c_int, c_long, call, ptr, stream
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    peak, peak_word = hbm_peak()
    ref = load_reference()
    g = torch.Generator(device=dev).manual_seed(0)
    R, C, H = a.tokens, 3072, 24
    act_bytes = R * C * 2
    rot = max(2, int(300e6 // act_bytes) + 1)                      # every rotation set exceeds the 126 MB L2
    rnd = lambda *s, scale=1.0: (torch.randn(*s, device=dev, generator=g) * scale).to(BF16)  # noqa: E731
    rows_out = []

    def report(name, ms, nbytes, ref_ms=None):
        gbs = nbytes / ms / 1e6
        line = f"{name:<58s} {ms * 1e3:9.1f} us  {nbytes / 1e6:9.1f} MB  {gbs:8.0f} GB/s  {gbs / peak:5.2f} {peak_word}"
        if ref_ms is not None:
            line += f" | reference kernel {ref_ms * 1e3:9.1f} us  ({ref_ms / ms:4.2f}x)"
        print(line, flush=True)
        rows_out.append({"kernel": name, "us": ms * 1e3, "mbytes": nbytes / 1e6, "gbs": gbs, "frac_hbm": gbs / peak,
                         "reference_us": None if ref_ms is None else ref_ms * 1e3})

    xs = [rnd(R, C) for _ in range(rot)]
    br = [rnd(R, C) for _ in range(rot)]
    dys = [rnd(R, C) for _ in range(rot)]
    ys = [torch.empty(R, C, device=dev, dtype=BF16) for _ in range(rot)]
    y2 = [torch.empty(R, C, device=dev, dtype=BF16) for _ in range(rot)]
    scale, shift, gate = rnd(1, C, scale=0.1), rnd(1, C, scale=0.1), rnd(1, C, scale=0.5)
    mean = torch.empty(R, dtype=torch.float32, device=dev)
    rstd = torch.empty(R, dtype=torch.float32, device=dev)
    nblk = _lib.lib().tt_norm_partial_blocks(c_long(R), c_int(1))
    partials = torch.empty(nblk * 3 * C, dtype=torch.float32, device=dev)
    dscale, dshift, dgate = (torch.empty(1, C, device=dev, dtype=BF16) for _ in range(3))

    # ---- LayerNorm + modulation -----------------------------------------------------------------------------------
    def ln_fwd(i):
        call("tt_ln_mod_fwd", ptr(xs[i]), None, None, ptr(scale), ptr(shift), None, ptr(ys[i]), ptr(mean), ptr(rstd), c_long(R),
             c_int(C), c_long(R), c_float(1e-6), stream())

    def ln_bwd(i):
        call("tt_ln_mod_bwd", ptr(dys[i]), None, ptr(xs[i]), None, None, ptr(scale), ptr(mean), ptr(rstd), ptr(ys[i]), None,
             ptr(partials), ptr(dscale), ptr(dshift), None, c_long(R), c_int(C), c_long(R), stream())
    ref_f = ref_b = None
    if ref is not None and want("ln"):
        xn = [torch.empty(R, C, device=dev, dtype=BF16) for _ in range(rot)]
        inv = torch.empty(R, dtype=torch.float32, device=dev)
        sc1, sh1 = scale.reshape(C).contiguous(), shift.reshape(C).contiguous()
        ds, dh = torch.empty(C, device=dev, dtype=BF16), torch.empty(C, device=dev, dtype=BF16)
        A = ref["fused_adaln"]
        ref_f = timeit(lambda i: A.torch_launch_adaln_forward(ys[i], xn[i], xs[i], sc1, sh1, R, C, 1e-6, inv), a.iters, rot)
        ref_b = timeit(lambda i: A.torch_launch_adaln_backward(y2[i], ds, dh, dys[i], xn[i], sc1, inv, R, C), a.iters, rot)
        del xn
    if want("ln"):
        report("LayerNorm + modulate forward [R, 3072]", timeit(ln_fwd, a.iters, rot), 2 * act_bytes + 8 * R, ref_f)
        ln_fwd(0)
        report("LayerNorm + modulate backward (dx, dscale, dshift)", timeit(ln_bwd, a.iters, rot), 3 * act_bytes + 8 * R, ref_b)

    def lnr_fwd(i):
        call("tt_ln_mod_fwd", ptr(xs[i]), ptr(br[i]), ptr(gate), ptr(scale), ptr(shift), ptr(y2[i]), ptr(ys[i]), ptr(mean), ptr(rstd),
             c_long(R), c_int(C), c_long(R), c_float(1e-6), stream())
    if want("ln"):
        report("gated residual + LayerNorm + modulate forward", timeit(lnr_fwd, a.iters, rot), 4 * act_bytes + 8 * R)

    def gr_fwd(i):
        call("tt_gate_residual_fwd", ptr(xs[i]), ptr(br[i]), ptr(gate), ptr(ys[i]), c_long(R), c_int(C), c_long(R), stream())

    def gr_bwd(i):
        call("tt_gate_residual_bwd", ptr(dys[i]), ptr(br[i]), ptr(gate), ptr(ys[i]), ptr(partials), ptr(dgate), c_long(R), c_int(C),
             c_long(R), stream())
    if want("gate"):
        report("gated residual forward", timeit(gr_fwd, a.iters, rot), 3 * act_bytes)
        report("gated residual backward (dbranch, dgate)", timeit(gr_bwd, a.iters, rot), 3 * act_bytes)

    # ---- GELU ------------------------------------------------------------------------------------------------------
    n_el = R * C
    if want("gelu"):
        report("GELU (tanh) forward", timeit(lambda i: call("tt_gelu_fwd", ptr(xs[i]), ptr(ys[i]), c_long(n_el), c_int(1), stream()), a.iters, rot),
               2 * act_bytes)
        report("GELU (tanh) backward", timeit(lambda i: call("tt_gelu_bwd", ptr(dys[i]), ptr(xs[i]), ptr(ys[i]), c_long(n_el), c_int(1), stream()),
                                              a.iters, rot), 3 * act_bytes)

    # ---- RMSNorm over heads: [R * 24, 128] -------------------------------------------------------------------------
    RR = R * H
    w = (1 + 0.1 * torch.randn(128, device=dev, generator=g)).to(BF16)
    rs = torch.empty(RR, dtype=torch.float32, device=dev)
    dw = torch.empty(128, device=dev, dtype=BF16)
    nb2 = _lib.lib().tt_norm_partial_blocks(c_long(RR), c_int(1))
    part2 = torch.empty(nb2 * 128, dtype=torch.float32, device=dev)

    def rms_fwd(i):
        call("tt_rmsnorm_fwd", ptr(xs[i]), ptr(w), ptr(ys[i]), ptr(rs), c_long(RR), c_int(128), c_float(1e-6), stream())

    def rms_bwd(i):
        call("tt_rmsnorm_bwd", ptr(dys[i]), ptr(xs[i]), ptr(w), ptr(rs), ptr(y2[i]), ptr(part2), ptr(dw), c_long(RR), c_int(128), stream())
    ref_f = ref_b = None
    if ref is not None and want("rms"):
        Rm = ref["fused_rmsnorm"]
        inv = torch.empty(RR, dtype=torch.float32, device=dev)
        ref_f = timeit(lambda i: Rm.torch_launch_rms_forward(ys[i], xs[i], w, RR, 128, 1e-6, inv), a.iters, rot)
        # the reference's backward takes the normalised OUTPUT (it divides by the weight to recover x_hat)
        ref_b = timeit(lambda i: Rm.torch_launch_rms_backward(y2[i], dw, dys[i], ys[i], w, inv, RR, 128), a.iters, rot)
    if want("rms"):
        report("RMSNorm forward [R * 24, 128]", timeit(rms_fwd, a.iters, rot), 2 * act_bytes + 4 * RR, ref_f)
        rms_fwd(0)
        report("RMSNorm backward (dx, dw)", timeit(rms_bwd, a.iters, rot), 3 * act_bytes + 4 * RR, ref_b)

    if want("qkvpost"):
        # ---- QKV post-processing (split + QK-RMSNorm + RoPE + head-major), one third of the tokens to bound memory ------
        Rq = R // 4
        qkv = [rnd(Rq, H * 384) for _ in range(rot)]
        dqkv = [torch.empty(Rq, H * 384, device=dev, dtype=BF16) for _ in range(rot)]
        q, k, v = (torch.empty(1, H, Rq, 128, device=dev, dtype=BF16) for _ in range(3))
        ang = torch.rand(Rq, 64, device=dev, generator=g) * 6.28
        cos, sin = ang.cos().repeat_interleave(2, 1).contiguous(), ang.sin().repeat_interleave(2, 1).contiguous()
        nw = _lib.lib().tt_qkv_partial_warps(c_long(Rq), c_int(H))
        part3 = torch.empty(nw * 256, dtype=torch.float32, device=dev)
        dqw, dkw = torch.empty(128, device=dev, dtype=BF16), torch.empty(128, device=dev, dtype=BF16)
        qkv_bytes = Rq * H * 384 * 2

        def post_fwd(i):
            call("tt_qkv_post_fwd", ptr(qkv[i]), ptr(w), ptr(w), ptr(cos), ptr(sin), ptr(q), ptr(k), ptr(v), c_long(Rq), c_int(H), c_long(Rq),
                 c_long(Rq), c_long(0), c_long(Rq), c_float(1e-6), stream())

        def post_bwd(i):
            call("tt_qkv_post_bwd", ptr(q), ptr(k), ptr(v), ptr(qkv[i]), ptr(w), ptr(w), ptr(cos), ptr(sin), ptr(dqkv[i]), ptr(part3), ptr(dqw),
                 ptr(dkw), c_long(Rq), c_int(H), c_long(Rq), c_long(Rq), c_long(0), c_long(Rq), c_float(1e-6), stream())
        report("QKV post-processing forward (norm, RoPE, head-major)", timeit(post_fwd, a.iters, rot), 2 * qkv_bytes + 2 * Rq * 128 * 4)
        report("QKV post-processing backward", timeit(post_bwd, a.iters, rot), 3 * qkv_bytes + 2 * Rq * 128 * 4)
        del qkv, dqkv

    if want("adam"):
        # ---- AdamW on a 128 Mi-element range ---------------------------------------------------------------------------
        n = 128 << 20
        p, gr = rnd(n), rnd(n, scale=0.01)
        for state_dtype, master_mode, per in ((torch.float32, "fp32", 2 + 4 + 4 + 4 + 2 + 4 + 4 + 4), (BF16, "split16", 2 + 2 + 2 + 2 + 2 + 2 + 2 + 2 + 2)):
            m = torch.zeros(n, device=dev, dtype=state_dtype)
            vv = torch.zeros(n, device=dev, dtype=state_dtype)
            master = p.float() if master_mode == "fp32" else None
            lo = torch.zeros(n, device=dev, dtype=torch.int16) if master_mode == "split16" else None
            step = [0]

            def adam(_i):
                step[0] += 1
                call("tt_adamw", ptr(p), ptr(gr), ptr(m), ptr(vv), ptr(master), ptr(lo), c_long(n), c_int(1 if state_dtype == BF16 else 0),
                     c_float(1e-5), c_float(0.9), c_float(0.999), c_float(1e-8), c_float(0.01), c_int(step[0]), c_float(1.0), stream())
            report(f"AdamW, {master_mode} master + {'bf16' if state_dtype == BF16 else 'fp32'} moments", timeit(adam, a.iters, 1), n * per)
            if master_mode == "fp32":
                # the fused reduce + AdamW + all-gather kernel with four local "peers": 4 gradient reads, 4 parameter writes
                peers_g = [gr] + [rnd(n, scale=0.01) for _ in range(3)]
                peers_p = [p] + [torch.empty(n, device=dev, dtype=BF16) for _ in range(3)]
                tg = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in peers_g])
                tp = (ctypes.c_void_p * 4)(*[t.data_ptr() for t in peers_p])

                def fused(_i):
                    step[0] += 1
                    call("tt_rs_adamw_ag", tg, c_int(4), tp, c_int(4), c_int(0), c_long(0), ptr(m), ptr(vv), ptr(master), None, c_long(n),
                         c_int(0), c_float(1e-5), c_float(0.9), c_float(0.999), c_float(1e-8), c_float(0.01), c_int(step[0]), c_float(0.25),
                         stream())
                report("reduce (4 local peers) + AdamW + all-gather (4), fp32 state", timeit(fused, a.iters, 1), n * (4 * 2 + 24 + 4 * 2))
                red = torch.empty(n, device=dev, dtype=BF16)
                report("gradient reduce-scatter kernel, 4 local peers", timeit(
                    lambda _i: call("tt_reduce_scatter_bf16", tg, c_int(4), c_long(0), ptr(red), c_long(n), c_float(0.25), stream()), a.iters, 1),
                    n * (4 * 2 + 2))
                report("parameter all-gather push kernel, 4 local peers", timeit(
                    lambda _i: call("tt_all_gather_push_bf16", tp, c_int(4), c_long(0), ptr(red), c_long(n), stream()), a.iters, 1), n * (2 + 4 * 2))
                del peers_g, peers_p, red
            del m, vv, master, lo
    print(f"HBM copy peak used: {peak:.1f} GB/s ({peak_word}); reference kernels {'timed' if ref is not None else 'not built'}")
    if a.json:
        json.dump(rows_out, open(a.json, "w"), indent=1)


if __name__ == "__main__":
    main()
