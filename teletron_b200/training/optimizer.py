"""AdamW with ZeRO-1 sharding over the DP x CP group, on flat buffers.

Stands in for Megatron's ``DistributedOptimizer`` + apex/TE ``FusedAdam`` + ``Float16Module``
that the reference wires up in ``teletron/core/training.py:33-44``: bf16 model weights, an
authoritative higher-precision copy owned by exactly one data-parallel rank per element,
Adam moments sharded the same way, gradient reduce-scatter before and parameter all-gather
after the update, optional global-norm clipping, and the Megatron rule of no weight decay on
biases / 1-D parameters.

Memory modes (sized for 180 GB of HBM3e):

* ``master_mode="fp32"``, ``state_dtype=fp32`` - the reference's 12 bytes/param of sharded state.
* ``master_mode="split16"`` - the fp32 master is stored as the bf16 weight itself plus a 16-bit
  remainder (``master_bits = (bf16_bits << 16) + int16_remainder``): exact fp32 master at
  2 extra bytes/param.  With ``state_dtype=bf16`` the whole optimizer costs 6 bytes/param, which
  is what lets the full 13B model train on a single B200.

The arithmetic is that of :func:`teletron_b200.ops.optim.adamw_update_reference`; on CUDA the update of
a shard is one launch of the fused sm_100a kernel (``csrc/optim.cu``).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..parallel.grad_buffer import DistributedDataParallel, ParamAndGradBuffer
from ..parallel import state as ps


from ..ops.optim import _pack16 as split16_pack, _unpack16 as split16_unpack  # noqa: E402,F401


class _ShardState:
    """Optimizer state for this rank's slice ``[start, end)`` of one bucket."""

    def __init__(self, buf: ParamAndGradBuffer, start: int, end: int, master_mode: str, state_dtype: torch.dtype):
        n = end - start
        self.start, self.end = start, end
        dev = buf.device
        self.exp_avg = torch.zeros(n, dtype=state_dtype, device=dev)
        self.exp_avg_sq = torch.zeros(n, dtype=state_dtype, device=dev)
        if master_mode == "fp32":
            self.master = buf.param_data[start:end].float()
            self.master_lo = None
        elif master_mode == "split16":
            self.master = None
            self.master_lo = torch.zeros(n, dtype=torch.int16, device=dev)
        else:
            self.master = None
            self.master_lo = None


class DistributedOptimizer:
    def __init__(self, ddp: DistributedDataParallel, lr: float = 1e-5, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.01, clip_grad: float = 0.0, master_mode: str = "fp32",
                 state_dtype: torch.dtype = torch.float32, model_parallel_group=None):
        if master_mode not in ("fp32", "split16", "none"):
            raise ValueError(master_mode)
        self.ddp = ddp
        self.lr, self.betas, self.eps, self.weight_decay = lr, betas, eps, weight_decay
        self.clip_grad = clip_grad
        self.master_mode, self.state_dtype = master_mode, state_dtype
        self.mp_group = model_parallel_group
        self.step_count = 0
        self.sharded = ddp.use_distributed_optimizer and ddp.world > 1
        self.shards: List[List[_ShardState]] = []
        for buf in ddp.buffers:
            if buf.dtype == torch.float32 and master_mode == "split16":
                raise ValueError("split16 master weights need bf16 parameters")
            states = []
            for b in buf.buckets:
                s, e = buf.shard_range(b, ddp.rank) if self.sharded else (b.start, b.end)
                mm = master_mode if buf.dtype != torch.float32 else "none"
                states.append(_ShardState(buf, s, e, mm, state_dtype))
            self.shards.append(states)
        self.last_grad_norm: Optional[float] = None
        # With the flat buffers in a symmetric heap, the whole update of a shard is one kernel: peers' gradients are
        # read and summed, AdamW runs, and the new weights are stored into every replica (csrc/optim.cu).  Without
        # clipping nothing needs the reduced gradients beforehand, so the separate reduce-scatter is dropped as well;
        # with overlapped reduction (side stream during backward) the kernel reads the already reduced local shard.
        self.fused_update = (self.sharded and getattr(ddp, "heap", None) is not None and len(ddp.buffers) == 1
                             and ddp.buffers[0].dtype == torch.bfloat16)
        self.reduce_here = self.fused_update and not (clip_grad and clip_grad > 0.0) and not ddp.overlap_grad_reduce
        ddp.reduce_in_optimizer = self.reduce_here

    # ---- helpers ------------------------------------------------------------------------
    def _segments(self, buf: ParamAndGradBuffer, st: _ShardState):
        """Intersections of a shard with the buffer's (weight-decay, tp-duplicate) regions."""
        for r in buf.regions:
            s, e = max(r.start, st.start), min(r.end, st.end)
            if s < e:
                yield s, e, r

    def grad_norm(self) -> float:
        """Global L2 norm of the (already averaged) gradients, each element counted once."""
        total = None
        tp_rank = ps.get_tensor_model_parallel_rank()
        for buf, states in zip(self.ddp.buffers, self.shards):
            for st in states:
                for s, e, r in self._segments(buf, st):
                    if r.tp_duplicate and tp_rank != 0:
                        continue
                    v = buf.grad_data[s:e].float().pow(2).sum()
                    total = v if total is None else total + v
        if total is None:
            total = torch.zeros((), device=self.ddp.buffers[0].device)
        if self.sharded:
            dist.all_reduce(total, group=self.ddp.group)
        if ps.get_tensor_model_parallel_world_size() > 1:
            dist.all_reduce(total, group=ps.get_tensor_model_parallel_group())
        return float(total.sqrt().item())

    # ---- step ---------------------------------------------------------------------------
    @torch.no_grad()
    def step(self) -> bool:
        """Update this rank's shards, then all-gather the new bf16 weights.  Gradients must
        already be synchronised (``ddp.finish_grad_sync()``)."""
        from .. import ops
        self.step_count += 1
        clip_coef = 1.0
        if self.clip_grad and self.clip_grad > 0.0:
            norm = self.grad_norm()
            self.last_grad_norm = norm
            if not math.isfinite(norm):
                return False
            clip_coef = min(1.0, self.clip_grad / (norm + 1e-6))
        b1, b2 = self.betas
        if self.fused_update:
            from ..ops import fused_comm as FC
            heap, (po, go) = self.ddp.heap, self.ddp.heap_offsets
            buf, states = self.ddp.buffers[0], self.shards[0]
            scale = clip_coef * (self.ddp.grad_scale if self.reduce_here else 1.0)
            for st in states:
                for s, e, r in self._segments(buf, st):
                    o0, o1 = s - st.start, e - st.start
                    FC.fused_reduce_adamw_all_gather(
                        heap, go, po, s, e - s, st.exp_avg[o0:o1], st.exp_avg_sq[o0:o1],
                        None if st.master is None else st.master[o0:o1],
                        None if st.master_lo is None else st.master_lo[o0:o1],
                        lr=self.lr, beta1=b1, beta2=b2, eps=self.eps,
                        weight_decay=self.weight_decay if r.weight_decay else 0.0, step=self.step_count,
                        grad_scale=scale, grads_reduced=not self.reduce_here)
            heap.barrier()         # peers have read this rank's gradients; every replica holds the new weights
            return True
        for buf, states in zip(self.ddp.buffers, self.shards):
            for st in states:
                for s, e, r in self._segments(buf, st):
                    o0, o1 = s - st.start, e - st.start
                    ops.optim.adamw_update(
                        param=buf.param_data[s:e], grad=buf.grad_data[s:e],
                        exp_avg=st.exp_avg[o0:o1], exp_avg_sq=st.exp_avg_sq[o0:o1],
                        master=None if st.master is None else st.master[o0:o1],
                        master_lo=None if st.master_lo is None else st.master_lo[o0:o1],
                        lr=self.lr, beta1=b1, beta2=b2, eps=self.eps,
                        weight_decay=self.weight_decay if r.weight_decay else 0.0,
                        step=self.step_count, grad_scale=clip_coef)
            if self.sharded and getattr(self.ddp, "heap", None) is not None:
                # parameter all-gather by peer stores: every rank writes its updated shard into all replicas
                from ..ops import fused_comm as FC
                for st in states:
                    FC.fused_param_all_gather(self.ddp.heap, self.ddp.heap_offsets[0], st.start, buf.param_data[st.start:st.end])
                self.ddp.heap.barrier()
            elif self.sharded:
                from ..ops import _lib
                with _lib.phase("nccl parameter all-gather"):
                    for b, st in zip(buf.buckets, states):
                        dist.all_gather_into_tensor(buf.param_data[b.start:b.end], buf.param_data[st.start:st.end],
                                                    group=self.ddp.group)
        return True

    def zero_grad(self, set_to_none: bool = False):
        self.ddp.zero_grad_buffer()

    # ---- checkpoint ---------------------------------------------------------------------
    def state_dict(self) -> Dict:
        """Small replicated part (hyper-parameters, step)."""
        return {"step": self.step_count, "lr": self.lr, "betas": self.betas, "eps": self.eps,
                "weight_decay": self.weight_decay, "master_mode": self.master_mode,
                "state_dtype": str(self.state_dtype)}

    def load_state_dict(self, sd: Dict):
        self.step_count = sd.get("step", 0)
        self.lr = sd.get("lr", self.lr)

    def sharded_state_dict(self) -> Dict:
        """This rank's shard of the moments / master weights (``distrib_optim.pt`` payload)."""
        out = []
        for states in self.shards:
            out.append([{"start": st.start, "end": st.end, "exp_avg": st.exp_avg.cpu(),
                         "exp_avg_sq": st.exp_avg_sq.cpu(),
                         "master": None if st.master is None else st.master.cpu(),
                         "master_lo": None if st.master_lo is None else st.master_lo.cpu()} for st in states])
        return {"buffers": out}

    def load_sharded_state_dict(self, sd: Dict):
        for states, saved in zip(self.shards, sd["buffers"]):
            for st, s in zip(states, saved):
                if (st.start, st.end) != (s["start"], s["end"]):
                    raise ValueError("optimizer shard layout changed between save and load")
                st.exp_avg.copy_(s["exp_avg"])
                st.exp_avg_sq.copy_(s["exp_avg_sq"])
                if st.master is not None and s["master"] is not None:
                    st.master.copy_(s["master"])
                if st.master_lo is not None and s["master_lo"] is not None:
                    st.master_lo.copy_(s["master_lo"])

    def reload_model_params(self):
        """Refresh master weights from the (just loaded) bf16 parameters."""
        for buf, states in zip(self.ddp.buffers, self.shards):
            for st in states:
                if st.master is not None:
                    st.master.copy_(buf.param_data[st.start:st.end].float())
                if st.master_lo is not None:
                    st.master_lo.zero_()


class OptimizerParamScheduler:
    """Learning-rate schedule: warmup then constant / linear / cosine / inverse-square-root decay (Megatron flag names)."""

    def __init__(self, optimizer: DistributedOptimizer, max_lr: float, min_lr: float = 0.0,
                 lr_warmup_steps: int = 0, lr_decay_steps: int = 1, lr_decay_style: str = "constant"):
        self.optimizer = optimizer
        self.max_lr, self.min_lr = max_lr, min_lr
        self.warmup, self.decay_steps, self.style = lr_warmup_steps, max(1, lr_decay_steps), lr_decay_style
        self.num_steps = 0
        self.step(0)

    def get_lr(self) -> float:
        n = self.num_steps
        if self.warmup > 0 and n <= self.warmup:
            return self.max_lr * n / self.warmup
        if self.style == "constant":
            return self.max_lr
        if self.style == "inverse-square-root":
            # max_lr * sqrt(warmup) / sqrt(step), floored at min_lr (Megatron's formula; warmup 0 counts as 1)
            w = max(self.warmup, 1)
            return max(self.min_lr, self.max_lr * math.sqrt(w) / math.sqrt(max(n, w)))
        if n > self.decay_steps:
            return self.min_lr
        ratio = (n - self.warmup) / max(1, self.decay_steps - self.warmup)
        delta = self.max_lr - self.min_lr
        if self.style == "linear":
            coeff = 1.0 - ratio
        elif self.style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        else:
            raise ValueError(f"unknown lr decay style {self.style}")
        return self.min_lr + coeff * delta

    def step(self, increment: int = 1):
        self.num_steps += increment
        self.optimizer.lr = self.get_lr()

    def state_dict(self):
        return {"num_steps": self.num_steps, "max_lr": self.max_lr, "min_lr": self.min_lr,
                "warmup": self.warmup, "decay_steps": self.decay_steps, "style": self.style}

    def load_state_dict(self, sd):
        self.num_steps = sd.get("num_steps", 0)
        self.optimizer.lr = self.get_lr()
