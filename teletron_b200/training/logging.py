"""Timers, rank-0 printing and metric sinks (JSONL + optional TensorBoard).

Stands in for Megatron's ``Timers`` / ``training_log`` that the reference relies on
(``teletron/training/training.py:35-43, 178-228``).  Device phases are timed with CUDA events on
the launching stream; multi-rank figures are reduced as max (and min) over ranks on the device
side, never by wall clock.  Beyond the reference's log line (iteration, ms/iter, lr, loss) it
reports samples/s, video frames/s (the unit of the reference's published charts), tokens/s,
model TFLOP/s per GPU and MFU.
"""

from __future__ import annotations

import json
import os
import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


def is_rank_0() -> bool:
    return (not dist.is_initialized()) or dist.get_rank() == 0


def print_rank_0(*a, **kw) -> None:
    if is_rank_0():
        print(*a, **kw, flush=True)


def print_rank_last(*a, **kw) -> None:
    """Printed by the last DiT rank (encoder ranks sit behind it and report nothing)."""
    last = True
    if dist.is_initialized():
        from ..parallel import state as ps
        n = ps.state().dit_world_size if ps.model_parallel_is_initialized() else dist.get_world_size()
        last = dist.get_rank() == n - 1
    if last:
        print(*a, **kw, flush=True)


class _Timer:
    def __init__(self, name: str, use_cuda: bool):
        self.name, self.use_cuda = name, use_cuda
        self.elapsed_ms = 0.0
        self._pairs = []
        self._t0 = None
        self.count = 0

    def start(self):
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._t0 = ev
        else:
            self._t0 = time.perf_counter()

    def stop(self):
        if self._t0 is None:
            raise RuntimeError(f"timer {self.name} stopped before start")
        if self.use_cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._pairs.append((self._t0, ev))
        else:
            self.elapsed_ms += (time.perf_counter() - self._t0) * 1e3
        self._t0 = None
        self.count += 1

    def elapsed(self, reset: bool = True) -> float:
        """Milliseconds accumulated since the last reset (syncs on the recorded events)."""
        if self.use_cuda and self._pairs:
            self._pairs[-1][1].synchronize()
            self.elapsed_ms += sum(a.elapsed_time(b) for a, b in self._pairs)
            self._pairs = []
        v = self.elapsed_ms
        if reset:
            self.elapsed_ms = 0.0
            self.count = 0
        return v


class Timers:
    """``timers('name', log_level=1).start()`` / ``.stop()``, as in Megatron."""

    def __init__(self, log_level: int = 0, log_option: str = "minmax"):
        self.log_level, self.log_option = log_level, log_option
        self._timers: Dict[str, _Timer] = {}
        self._levels: Dict[str, int] = {}

    class _Null:
        def start(self, *a, **k):
            pass

        def stop(self, *a, **k):
            pass

    def __call__(self, name: str, log_level: int = 1):
        t = self._timers.get(name)
        if t is not None:
            return t                      # a later .stop() call need not repeat the level
        if log_level > self.log_level and log_level > 0:
            return Timers._Null()
        if t is None:
            t = self._timers[name] = _Timer(name, torch.cuda.is_available())
            self._levels[name] = log_level
        return t

    def collect(self, names: Optional[List[str]] = None, reset: bool = True) -> Dict[str, Dict[str, float]]:
        names = names or list(self._timers)
        out = {}
        for n in names:
            if n not in self._timers:
                continue
            v = self._timers[n].elapsed(reset)
            mx = mn = v
            if dist.is_initialized() and dist.get_world_size() > 1:
                from ..parallel import state as ps
                # encoder ranks never reach a timer report: reduce over the DiT ranks only
                group = ps.get_transformer_model_group() if ps.model_parallel_is_initialized() else None
                dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
                t = torch.tensor([v, -v], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
                mx, mn = float(t[0]), -float(t[1])
            out[n] = {"max_ms": mx, "min_ms": mn}
        return out

    def log(self, names: Optional[List[str]] = None, normalizer: float = 1.0) -> str:
        stats = self.collect(names)
        parts = [f"{n}: ({s['min_ms'] / normalizer:.2f}, {s['max_ms'] / normalizer:.2f})" for n, s in stats.items()]
        line = "time (ms) | " + " | ".join(parts)
        print_rank_last(line)
        return line


def model_flops_per_sample(num_params_blocks: int, video_tokens: int, text_tokens: int, heads: int, head_dim: int,
                           n_blocks: int, recompute: bool, attention_recomputed: bool = True) -> float:
    """FLOPs executed for one training sample: linears ``2 * P * tokens`` and attention
    ``4 * tokens^2 * head_dim * heads`` per block forward; backward = 2x forward (attention backward 2.5x); full
    recompute adds one more forward of the linears, and of attention too unless the attention output is kept
    (``attention_recomputed=False``).  ``recompute=False`` gives the useful (model) FLOPs that an MFU is quoted on."""
    n = video_tokens + text_tokens
    lin = 2.0 * num_params_blocks * n
    att = 4.0 * n * n * head_dim * heads * n_blocks
    total = 3.0 * lin + 3.5 * att
    if recompute:
        total += lin + (att if attention_recomputed else 0.0)
    return total


class MetricLogger:
    def __init__(self, jsonl_path: Optional[str] = None, tensorboard_dir: Optional[str] = None, queue_size: int = 10,
                 wandb_project: Optional[str] = None, wandb_name: Optional[str] = None, wandb_dir: Optional[str] = None,
                 config: Optional[dict] = None):
        self.jsonl = None
        self.wandb = None
        if wandb_project and is_rank_0():
            try:
                import wandb
                wandb.init(project=wandb_project, name=wandb_name, dir=wandb_dir,
                           config={k: v for k, v in (config or {}).items() if isinstance(v, (int, float, str, bool, type(None)))})
                self.wandb = wandb
            except Exception as e:      # wandb is optional
                print_rank_0(f"wandb unavailable ({e}); logging to stdout/JSONL only")
        if jsonl_path and is_rank_0():
            os.makedirs(os.path.dirname(os.path.abspath(jsonl_path)), exist_ok=True)
            self.jsonl = open(jsonl_path, "a")
        self.tb = None
        if tensorboard_dir and is_rank_0():
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tb = SummaryWriter(log_dir=tensorboard_dir, max_queue=queue_size)
            except Exception as e:      # tensorboard is optional
                print_rank_0(f"tensorboard unavailable ({e}); logging to stdout/JSONL only")

    def log(self, step: int, metrics: Dict[str, float]) -> None:
        if not is_rank_0():
            return
        if self.jsonl is not None:
            self.jsonl.write(json.dumps({"step": step, **metrics}) + "\n")
            self.jsonl.flush()
        if self.tb is not None:
            for k, v in metrics.items():
                if isinstance(v, (int, float)):
                    self.tb.add_scalar(k, v, step)
        if self.wandb is not None:
            self.wandb.log({k: v for k, v in metrics.items() if isinstance(v, (int, float))}, step=step)

    def close(self):
        if self.jsonl is not None:
            self.jsonl.close()
        if self.tb is not None:
            self.tb.close()
        if self.wandb is not None:
            self.wandb.finish()


def peak_bf16_tflops() -> float:
    """Sustained bf16 GEMM peak used as the MFU denominator (the measured one when the peaks file is present)."""
    from ..utils.perf import measured_peaks
    return measured_peaks()["bf16_tflops_sustained"]
