"""Collective-fusion microbenchmark (hidden 3072, 24 heads x 128, bf16) on N GPUs of one node.

Launch: ``python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P
benchmarks/collective_fusion_bench.py [--tokens 119056] [--iters 10]``.

Paths, each against the unfused NCCL + cuBLAS sequence the reference runs:
  (a) Ulysses seq->head all-to-all fused with the QKV GEMM + QK-RMSNorm + RoPE
  (b) head->seq all-to-all fused with the output projection, in two forms: the projection GEMM pulling its A operand
      per head from the owner rank, and (the form the model uses) the attention epilogue pushing every output row to the
      token's owner so that the projection is local
  (c) tensor-parallel all-gather->GEMM and GEMM->reduce-scatter on the 3072 x 12288 MLP
Times are CUDA events on each rank, max over ranks.  The roofline per path is the slower of
FLOPs / measured bf16 peak and NVLink bytes / 770 GB/s (measured peer copy, per direction per GPU).
"""

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from teletron_b200.ops import fused_comm as FC  # noqa: E402
from teletron_b200.ops import cuda_ops  # noqa: E402
from teletron_b200.parallel import mappings as M  # noqa: E402

LINK_GBS = 770.0


def peak():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"]
    except Exception:
        return 1590.0


def timeit(fn, iters):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=118800)
    ap.add_argument("--text", type=int, default=256)
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    g = dist.group.WORLD
    H, heads = 3072, 24
    s = (a.tokens + world - 1) // world
    s = (s + 7) // 8 * 8
    T = a.text
    pk = peak()
    gen = torch.Generator(device="cuda").manual_seed(rank)
    rnd = lambda *sh, k=1.0: (torch.randn(*sh, device="cuda", generator=gen) * k).bfloat16()  # noqa: E731
    out = {}

    # ---- (a) + (b): Ulysses all-to-alls fused into the QKV GEMM and the output projection ----
    if heads % world == 0:
        ws = FC.UlyssesWorkspace(g, heads, s, T)
        x, xt = rnd(1, s, H), rnd(1, T, H)
        w, b = rnd(3 * H, H, k=0.02), rnd(3 * H, k=0.02)
        qw, kw = rnd(128, k=0.1) + 1, rnd(128, k=0.1) + 1
        ang = torch.rand(s, 64, device="cuda", generator=gen) * 6.28
        cos, sin = ang.cos().repeat_interleave(2, 1).contiguous(), ang.sin().repeat_interleave(2, 1).contiguous()
        wo, bo = rnd(H, H, k=0.02), rnd(H, k=0.02)

        def fused_a():
            with torch.no_grad():
                FC.fused_qkv_a2a(ws, x, w, b, qw, kw, cos, sin, xt, w, b, qw, kw)

        def unfused_a():
            with torch.no_grad():
                q, k, v = cuda_ops.qkv_projection(x, w, b, qw, kw, cos, sin, heads)
                tq, tk, tv = cuda_ops.qkv_projection(xt, w, b, qw, kw, None, None, heads)
                q, k, v = (M._a2a_heads_to_seq(t, g) for t in (q, k, v))
                h = heads // world
                qq = torch.cat([q, tq[:, rank * h:(rank + 1) * h]], dim=2)
                kk = torch.cat([k, tk[:, rank * h:(rank + 1) * h]], dim=2)
                vv = torch.cat([v, tv[:, rank * h:(rank + 1) * h]], dim=2)
                return qq, kk, vv
        ta_f, ta_u = timeit(fused_a, a.iters), timeit(unfused_a, a.iters)
        fl = 2.0 * s * H * 3 * H
        nbytes = 3 * s * H * 2 * (world - 1) / world
        roof = max(fl / (pk * 1e12), nbytes / (LINK_GBS * 1e9)) * 1e3
        out["a_qkv_norm_rope_a2a"] = {"fused_ms": ta_f, "nccl_cublas_ms": ta_u, "speedup": ta_u / ta_f, "roofline_ms": roof,
                                      "roofline_fraction": roof / ta_f}
        o = ws.token_major("o")
        o.copy_(rnd(1, ws.S_tot, ws.h_loc * 128))

        def fused_b():
            with torch.no_grad():
                FC.fused_a2a_linear(ws, o, wo, bo, wo, bo)

        def unfused_b():
            with torch.no_grad():
                ov = o[:, T:].reshape(1, ws.S, ws.h_loc, 128).transpose(1, 2)
                ov = M._a2a_seq_to_heads(ov.contiguous(), g).transpose(1, 2).reshape(1, s, H)
                ot = M._gather(o[:, :T].contiguous(), g, 2, None)
                return cuda_ops.linear(ov, wo, bo), cuda_ops.linear(ot, wo, bo)
        tb_f, tb_u = timeit(fused_b, a.iters), timeit(unfused_b, a.iters)
        fl = 2.0 * s * H * H
        nbytes = s * H * 2 * (world - 1) / world
        roof = max(fl / (pk * 1e12), nbytes / (LINK_GBS * 1e9)) * 1e3
        out["b_a2a_outproj"] = {"fused_ms": tb_f, "nccl_cublas_ms": tb_u, "speedup": tb_u / tb_f, "roofline_ms": roof,
                                "roofline_fraction": roof / tb_f}
        # (b') push form used by the model: the attention epilogue performs the head -> sequence all-to-all (every output
        # row crosses NVLink once, while the tensor core is busy), then the projections are local
        qh, kh, vh = (ws.head_major(n) for n in ("q", "k", "v"))
        for t in (qh, kh, vh):
            t.copy_(rnd(1, ws.h_loc, ws.S_tot, 128))
        from teletron_b200.ops import attn_tcgen05 as AT

        def fused_bp():
            with torch.no_grad():
                FC.fused_attention_outproj(ws, qh, kh, vh, wo, bo, wo, bo)

        def unfused_bp():
            with torch.no_grad():
                oo = AT.forward(qh, kh, vh, None, None)[0]
                ov = oo[:, T:].reshape(1, ws.S, ws.h_loc, 128).transpose(1, 2)
                ov = M._a2a_seq_to_heads(ov.contiguous(), g).transpose(1, 2).reshape(1, s, H)
                ot = M._gather(oo[:, :T].contiguous(), g, 2, None)
                return cuda_ops.linear(ov, wo, bo), cuda_ops.linear(ot, wo, bo)
        it2 = max(2, a.iters // 4)
        tp_f, tp_u = timeit(fused_bp, it2), timeit(unfused_bp, it2)
        fl = 4.0 * ws.S_tot * ws.S_tot * 128 * ws.h_loc + 2.0 * s * H * H
        nbytes = s * H * 2 * (world - 1) / world
        roof = max(fl / (pk * 1e12), nbytes / (LINK_GBS * 1e9)) * 1e3
        out["b_attention_a2a_outproj_push"] = {"fused_ms": tp_f, "nccl_cublas_ms": tp_u, "speedup": tp_u / tp_f,
                                               "roofline_ms": roof, "roofline_fraction": roof / tp_f}
        ws.heap.check()

    # ---- (c): tensor-parallel AG->GEMM (fc1) and GEMM->RS (fc2) with sequence-sharded activations ----
    rows = (a.tokens // world + 127) // 128 * 128
    F = 4 * H
    tpw = FC.TPWorkspace(g, rows, H, H)
    xl = rnd(rows, H)
    w1 = rnd(F // world, H, k=0.02)
    w2 = rnd(H, F // world, k=0.02)
    hfull = rnd(rows * world, F // world)

    def fused_ag():
        FC.fused_all_gather_linear(tpw, xl, w1)

    def fused_ag_pull():
        FC.fused_all_gather_linear(tpw, xl, w1, staged=False)

    def unfused_ag():
        full = torch.empty(rows * world, H, device="cuda", dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, xl)
        return torch.nn.functional.linear(full, w1)

    def fused_rs():
        FC.fused_linear_reduce_scatter(tpw, hfull, w2)

    def unfused_rs():
        y = torch.nn.functional.linear(hfull, w2)
        o2 = torch.empty(rows, H, device="cuda", dtype=torch.bfloat16)
        dist.reduce_scatter_tensor(o2, y)
        return o2
    for name, f, u, fl, nb in (("c_tp_ag_gemm", fused_ag, unfused_ag, 2.0 * rows * world * H * F / world, rows * H * 2 * (world - 1)),
                               ("c_tp_ag_gemm_pull_every_tile", fused_ag_pull, unfused_ag, 2.0 * rows * world * H * F / world, rows * H * 2 * (world - 1)),
                               ("c_tp_gemm_rs", fused_rs, unfused_rs, 2.0 * rows * world * H * F / world, rows * H * 2 * (world - 1))):
        tf, tu = timeit(f, a.iters), timeit(u, a.iters)
        roof = max(fl / (pk * 1e12), nb / (LINK_GBS * 1e9)) * 1e3
        out[name] = {"fused_ms": tf, "nccl_cublas_ms": tu, "speedup": tu / tf, "roofline_ms": roof, "roofline_fraction": roof / tf}
    tpw.heap.check()
    if rank == 0:
        print(json.dumps({"n_gpus": world, "tokens": a.tokens, "local_tokens": s, "peak_tflops": pk, "link_gbs": LINK_GBS,
                          "paths": out}, indent=1), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
