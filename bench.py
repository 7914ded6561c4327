"""Headline benchmark: HunyuanVideo-13B 720P training throughput (samples/s) on N B200s of one node.

``python bench.py --gpus N --steps K --warmup W`` (for N > 1 launched under ``torch.distributed.run``,
one rank per GPU) trains the full 20 + 40 block, hidden-3072 MMDiT on synthetic 720P x 33-frame latents
(32 400 video tokens + 256 text tokens per sample) in bf16 with full activation recompute and AdamW,
and prints ONE JSON line from rank 0.  One sample is spread over all N GPUs (Ulysses context parallel,
plus tensor parallel where asked), so the measurement is strong scaling and ``value`` is whole-job
samples per second.

Timing: W untimed warm-up steps, then exactly K steps between a barrier + synchronize on both sides,
timed with CUDA events on the launching stream, max over ranks.  A second timed loop measures the same
metric end to end through the public training API (``train_step``): every step copies that step's
inputs from pinned host memory and reads the loss back to the host.

``--impl reference`` is the arm that would run the unmodified reference from ``baseline/_ref``; it
prints why it cannot (its Megatron-LM / TransformerEngine / diffusers dependencies are not installed).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
os.environ.setdefault("PYTORCH_CUDA_ALLOC_CONF", "expandable_segments:True")


def parse():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=3)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", type=str, default="ours", choices=["ours", "reference", "library"])
    p.add_argument("--frames", type=int, default=33)
    p.add_argument("--resolution", type=int, nargs=2, default=[1280, 720])
    p.add_argument("--text-len", type=int, default=256)
    p.add_argument("--layers", type=int, default=20)
    p.add_argument("--single-layers", type=int, default=40)
    p.add_argument("--tp", type=int, default=None)
    p.add_argument("--cp", type=int, default=None)
    p.add_argument("--model-type", type=str, default="t2v", choices=["t2v", "i2v"])
    p.add_argument("--no-recompute", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-save-attention", action="store_true")
    p.add_argument("--fused-comm", type=int, default=1, help="1: in-kernel NVLink collectives for context parallelism")
    p.add_argument("--seq-pad-multiple", type=int, default=8,
                   help="pad each context-parallel chunk to a multiple of this many tokens (8 keeps the weight-gradient GEMMs of "
                        "cp4 / cp8 runs on the tcgen05 kernel; the pad keys are masked)")
    p.add_argument("--op-profile", type=str, default=None,
                   help="after the timed loop, run one step under torch.profiler and write the eager-op table to this file")
    p.add_argument("--breakdown", type=str, default=None,
                   help="after the timed loops, run one more step with per-kernel-family device timing (CUDA events around "
                        "every native call and NCCL section) and write the table to this file")
    p.add_argument("--overlap-grad-reduce", type=int, default=0,
                   help="1: bucketed gradient reduce-scatter on a side stream during backward")
    p.add_argument("--sequence-parallel", type=int, default=None,
                   help="1: shard the residual stream's tokens over the tensor-parallel ranks, MLPs on the fused all-gather -> GEMM / "
                        "GEMM -> reduce-scatter kernels; 0: replicated activations with NCCL all-reduce.  Default: 1 whenever tp > 1 "
                        "and the fused collectives are on")
    return p.parse_args()


def reference_arm(a):
    """The reference cannot be imported offline: say so in the contract's form."""
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    why = None
    try:
        import teletron  # noqa: F401
    except Exception as e:  # the expected outcome on this image
        why = f"import teletron failed: {type(e).__name__}: {e} (Megatron-LM submodule empty; megatron/transformer_engine/diffusers/yunchang/apex not installed)"
    if why is None:
        why = "reference imported but its training entry needs Megatron-LM core_r0.6.0 + TransformerEngine, which are not installed"
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
    return 0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
        os.close(fd)
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for n, v in zip(names, f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.path)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def run_op_profile(step_fn, path, rank):
    """One more step under torch.profiler: the PyTorch eager ops (cat, add, sum, fill, copies) that remain between the
    native kernels, grouped by input shape and sorted by device time.  A diagnosis aid; nothing timed here is reported."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=True) as prof:
        step_fn()
        torch.cuda.synchronize()
    if rank == 0:
        with open(path, "w") as fh:
            fh.write(prof.key_averages(group_by_input_shape=True).table(sort_by="cuda_time_total", row_limit=70,
                                                                       max_name_column_width=60, max_shapes_column_width=100))


def run_breakdown(step_fn, dev):
    """One extra training step with CUDA events around every native call and NCCL / optimizer section.  Returns
    ``{"step_ms": ..., "phases": {name: (ms on this rank, launches, max ms over ranks)}}`` (rank 0 writes it)."""
    import torch
    import torch.distributed as dist
    from teletron_b200.ops import _lib
    step_fn()                                    # one untimed step so that nothing of the timed loops is still in flight
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    from teletron_b200.ops import status as _status
    _lib.profile_start()
    t_host0 = time.perf_counter()
    e0.record()
    step_fn()
    e1.record()
    # host time to enqueue forward + backward + gradient sync: up to the status check, the first point where the host waits
    host_enqueue_ms = (_status.LAST_CHECK_HOST_TIME - t_host0) * 1e3
    prof = _lib.profile_stop()
    step_ms = e0.elapsed_time(e1)
    names = sorted(prof)
    mine = torch.tensor([prof[n][0] for n in names] + [step_ms], dtype=torch.float64, device=dev)
    worst = mine.clone()
    if dist.is_initialized():
        # the ranks run the same program, so the same names in the same order
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    return {"step_ms": float(mine[-1]), "step_ms_max": float(worst[-1]), "host_enqueue_ms": host_enqueue_ms,
            "phases": {n: (prof[n][0], prof[n][1], float(worst[i])) for i, n in enumerate(names)}}


_FAMILIES = (("attention forward", ("tt_attn_fwd",)), ("attention backward", ("tt_attn_bwd",)),
             ("QKV GEMM + norm + RoPE + seq->head exchange (F1)", ("tt_qkv_gemm_fused",)),
             ("QKV backward: head->seq gather + RoPE^T + norm backward (F1b)", ("tt_qkv_post_bwd",)),
             ("GEMMs with a fused collective (F2b push, F3)", ("tt_gemm_comm", "tt_gemm_ag")),
             ("plain GEMMs", ("tt_gemm_bf16", "tt_gemm2_bf16")), ("QKV post-processing (unfused path)", ("tt_qkv_post_fwd",)),
             ("device barriers (includes waiting for the slowest peer)", ("tt_comm_barrier",)),
             ("norm / modulation / gate / GELU", ("tt_ln_mod", "tt_gate_residual", "tt_rmsnorm", "tt_gelu")),
             ("gradient reduce-scatter + parameter all-gather (own kernels)", ("tt_reduce_scatter", "tt_all_gather_push", "tt_rs_adamw")),
             ("AdamW", ("tt_adamw",)), ("peer copies / partial sums", ("tt_gather_cols", "tt_partial_sum")),
             ("NCCL tensor-parallel all-reduce", ("nccl tp",)), ("NCCL other", ("nccl",)))


def format_breakdown(b, line) -> str:
    """Text table: device time per kernel family of one training step, and what is left (PyTorch eager ops, host gaps)."""
    rows, used = [], set()
    for title, prefixes in _FAMILIES:
        ms = n = mx = 0
        for name, (t, c, w) in b["phases"].items():
            if name not in used and any(name.startswith(p) for p in prefixes):
                used.add(name)
                ms, n, mx = ms + t, n + c, mx + w
        if n:
            rows.append((title, ms, n, mx))
    for name, (t, c, w) in b["phases"].items():
        if name not in used:
            rows.append((name, t, c, w))
    total = sum(r[1] for r in rows)
    out = [f"per-phase device time of one training step (CUDA events around every native call / NCCL section; rank 0 and max over ranks)",
           f"config: {json.dumps(line['config'])}",
           f"step: {b['step_ms']:.1f} ms on rank 0 ({b['step_ms_max']:.1f} ms max over ranks); timed loop: {line['ms_per_step']:.1f} ms/step; "
           f"host needed {b['host_enqueue_ms']:.1f} ms to enqueue forward + backward + gradient sync (with the profiling events)",
           f"{'phase':<72}{'ms':>10}{'share':>8}{'calls':>8}{'max ms':>10}"]
    for title, ms, n, mx in sorted(rows, key=lambda r: -r[1]):
        out.append(f"{title:<72}{ms:>10.2f}{100 * ms / b['step_ms']:>7.1f}%{n:>8d}{mx:>10.2f}")
    out.append(f"{'not in any bracket: PyTorch eager ops (cat, add, sum, copies), host gaps':<72}{b['step_ms'] - total:>10.2f}"
               f"{100 * (b['step_ms'] - total) / b['step_ms']:>7.1f}%")
    return "\n".join(out) + "\n"


def _heap_bytes() -> int:
    from teletron_b200.parallel import symm_mem
    return int(symm_mem.ALLOCATED_BYTES)


def main():
    a = parse()
    if a.impl == "reference":
        return reference_arm(a)

    import torch
    import torch.distributed as dist

    from teletron_b200 import ops
    from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, hunyuan_13b
    from teletron_b200.ops import _lib
    from teletron_b200.parallel import state as ps
    from teletron_b200.training import initialize, setup_model_and_optimizer, train_step
    from teletron_b200.training.args import get_args
    from teletron_b200.training.logging import model_flops_per_sample

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != a.gpus:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {a.gpus}")
    if a.impl == "library":
        # the restated reference path: cuBLAS GEMMs, SDPA attention, unfused PyTorch elementwise ops, NCCL collectives
        ops.set_impl("torch")
        # the reference turns the cuDNN SDPA backend off and runs PyTorch's flash backend
        # (teletron/models/dit/dit_attention.py:312)
        torch.backends.cuda.enable_cudnn_sdp(False)
    tp = a.tp if a.tp is not None else (2 if a.gpus == 8 else 1)
    cp = a.cp if a.cp is not None else max(1, a.gpus // tp)
    single = a.gpus == 1
    argv = ["--bf16", "--model-size", "13b", "--model-type", a.model_type, "--num-frames", str(a.frames),
            "--video-resolution", str(a.resolution[0]), str(a.resolution[1]), "--tensor-model-parallel-size", str(tp),
            "--context-parallel-size", str(cp), "--use-distributed-optimizer", "--lr", "1e-5", "--weight-decay", "1e-2",
            "--train-iters", str(a.steps + a.warmup), "--flow-shift", "7.0", "--dit-num-layers", str(a.layers),
            "--dit-num-single-layers", str(a.single_layers), "--distributed-timeout-minutes", "10",
            # a single B200 holds the 13B model only with the compact optimizer state (6 bytes/param)
            "--master-weight-mode", "split16" if single else "fp32",
            "--optimizer-state-dtype", "bf16" if single else "fp32"]
    if not a.no_recompute:
        argv += ["--recompute-granularity", "full", "--recompute-method", "block"]
    if a.impl == "ours" and a.fused_comm and a.gpus > 1:
        argv += ["--fused-comm"]
    if a.overlap_grad_reduce and a.gpus > 1:
        argv += ["--overlap-grad-reduce"]
    if a.sequence_parallel is None:
        a.sequence_parallel = 1 if (a.impl == "ours" and a.fused_comm) else 0
    sp = bool(a.sequence_parallel) and tp > 1
    if sp:
        argv += ["--sequence-parallel"]
    args = initialize(argv=argv)
    dev = args.device
    rank = args.rank

    from teletron_b200.models.hunyuanvideo.config import HunyuanParams  # noqa: F401
    cfg = hunyuan_13b(in_channels=33 if a.model_type == "i2v" else 16, num_layers=a.layers,
                      num_single_layers=a.single_layers,
                      recompute_granularity=None if a.no_recompute else "full", seed=1234,
                      recompute_save_attention=not a.no_save_attention and a.impl == "ours", sequence_parallel=sp,
                      sequence_pad_multiple=a.seq_pad_multiple)
    if a.impl == "ours" and a.fused_comm and a.gpus > 1:
        from teletron_b200.models.hunyuanvideo import blocks
        blocks.set_fused_comm(True)
    flow = FlowConfig(shift=7.0, model_type=a.model_type)

    def model_provider():
        pipe = HunyuanPipeline(cfg, flow, device=dev, dtype=torch.bfloat16)
        pipe._placed = True
        return pipe

    model, optimizer, scheduler = setup_model_and_optimizer(model_provider, args)
    W, H = a.resolution
    f = (a.frames - 1) // 4 + 1
    tokens = f * (H // 16) * (W // 16)

    # synthetic sample of the named shape, in pinned host memory (the e2e loop copies it every step)
    g = torch.Generator().manual_seed(1234)
    n_valid = int(torch.randint(64, a.text_len + 1, (1,), generator=g))
    mask = torch.zeros(1, a.text_len, dtype=torch.bool)
    mask[:, :n_valid] = True
    host = {"latents": torch.randn(1, 16, f, H // 8, W // 8, generator=g).to(torch.bfloat16).pin_memory(),
            "prompt_embeds": torch.randn(1, a.text_len, 4096, generator=g).to(torch.bfloat16).pin_memory(),
            "clip_text_embed": torch.randn(1, 768, generator=g).to(torch.bfloat16).pin_memory(),
            "prompt_attention_mask": mask.pin_memory()}
    h2d_bytes = sum(t.numel() * t.element_size() for t in host.values())
    device_batch = {k: v.to(dev) for k, v in host.items()}

    def loss_func(out):
        loss = out[0].mean()
        return loss, {"loss": loss.detach()}

    def fwd_device(_it, m):
        return m(device_batch), loss_func

    def fwd_e2e(_it, m):
        batch = {k: v.to(dev, non_blocking=True) for k, v in host.items()}
        return m(batch), loss_func

    def barrier():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, read_loss):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.LAUNCHES
        t0 = time.perf_counter()
        e0.record()
        last = None
        for _ in range(steps):
            losses, _, _ = train_step(fn, None, model, optimizer, scheduler, args)
            if read_loss:
                last = float(losses["loss"])         # device -> host read of the step's result
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        wall = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([ms, wall], dtype=torch.float64, device=dev)
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), float(t[1]), _lib.LAUNCHES - l0, last

    for _ in range(a.warmup):
        train_step(fwd_device, None, model, optimizer, scheduler, args)
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    ms, _, launches, _ = timed(fwd_device, a.steps, read_loss=False)
    clocks = sampler.stop() if rank == 0 else None
    e2e = None
    if not a.no_e2e:
        e2e_ms, wall_ms, _, last_loss = timed(fwd_e2e, a.steps, read_loss=True)
        e2e = {"value": a.steps / (e2e_ms / 1e3), "unit": "samples/s", "h2d_bytes_per_step": h2d_bytes,
               "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / a.steps, "wall_ms_per_step": wall_ms / a.steps,
               "last_loss": last_loss}
    ms_per_step = ms / a.steps
    value = 1.0 / (ms_per_step / 1e3)
    fl = lambda rec: model_flops_per_sample(cfg.num_parameters(), tokens, a.text_len, cfg.num_attention_heads,  # noqa: E731
                                            cfg.attention_head_dim, cfg.num_layers + cfg.num_single_layers, rec,
                                            attention_recomputed=not cfg.recompute_save_attention)
    flops, flops_executed = fl(False), fl(not a.no_recompute)
    if a.op_profile:
        run_op_profile(lambda: train_step(fwd_device, None, model, optimizer, scheduler, args), a.op_profile, rank)
    breakdown = None
    if a.breakdown:
        breakdown = run_breakdown(lambda: train_step(fwd_device, None, model, optimizer, scheduler, args), dev)
    if rank == 0:
        from teletron_b200.ops import attention_backend as attn_mod
        from teletron_b200.ops import gemm as gemm_mod
        from teletron_b200.ops import attn_backward as attn_bwd_mod
        from teletron_b200.ops import fused_comm as fc_mod
        out = {"metric": "HunyuanVideo-13B 720P train samples/s", "value": value, "unit": "samples/s",
               "n_gpus": a.gpus, "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step,
               "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
               "data": "synthetic latents/embeddings, random-init weights", "impl": a.impl,
               "config": {"model": f"HunyuanVideo-13B {a.model_type.upper()} ({a.layers} dual + {a.single_layers} single blocks, hidden 3072)",
                          "global_batch": 1, "seq_len": tokens + a.text_len, "frames": a.frames,
                          "resolution": f"{W}x{H}", "parallelism": f"tp{tp}cp{cp}dp1" + ("+sp" if sp else ""),
                          "recompute": "none" if a.no_recompute else ("full (attention output kept)" if cfg.recompute_save_attention else "full"),
                          "collectives": "in-kernel NVLink (fused)" if (a.impl == "ours" and a.fused_comm and (cp > 1 or sp)) else "NCCL", "optimizer": "AdamW ZeRO-1",
                          "optimizer_state": "split16 master + bf16 moments" if single else "fp32 master + fp32 moments",
                          "l2": "inputs larger than L2: >25 GB of weights and >10 GB of activations stream through every step"},
               "s_per_step": ms_per_step / 1e3, "frames_per_s": value * a.frames,
               # useful = forward + backward of the model; executed adds what the recompute pass really runs again
               "model_tflops_per_gpu": flops * value / a.gpus / 1e12,
               "executed_tflops_per_gpu": flops_executed * value / a.gpus / 1e12, "clocks": clocks, "e2e": e2e,
               "gpu_launches": launches,
               "kernel_backends": {"gemm": dict(gemm_mod.COUNTERS), "attention": dict(attn_mod.COUNTERS),
                                   "attention_backward": dict(attn_bwd_mod.COUNTERS), "fused_collective": dict(fc_mod.COUNTERS)},
               # the symmetric heaps (parameter / gradient buffers and collective workspaces of the fused-collective mode)
               # are raw device allocations that the PyTorch allocator's peak does not see
               "peak_mem_gb": (torch.cuda.max_memory_allocated() + _heap_bytes()) / 2 ** 30,
               "peak_mem_torch_gb": torch.cuda.max_memory_allocated() / 2 ** 30}
        if breakdown is not None:
            with open(a.breakdown, "w") as fh:
                fh.write(format_breakdown(breakdown, out))
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
