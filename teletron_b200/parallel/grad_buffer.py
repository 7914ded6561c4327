"""Contiguous parameter / gradient buffers and the data-parallel wrapper.

What the reference gets from Megatron's ``ParamAndGradBuffer`` + its own
``DistributedDataParallel`` (``teletron/core/distributed/distributed_data_parallel.py:14-298``):
bucketed contiguous gradient storage in the *parameter dtype* (bf16, ``:104-106``), gradient
pre-scaling by ``1 / (dp * cp)`` (``:133-147``), reduce-scatter (ZeRO-1) or all-reduce over the
DP x CP group, optional overlap of the bucket collectives with backward.

Design differences:

* Parameters are re-pointed into one flat bf16 ``param_data`` buffer and their ``.grad`` *is* a
  view of the flat ``grad_data`` buffer, so autograd accumulates in place - there is no
  ``main_grad`` copy hook (``:181-205``) and no second copy of any gradient.
* The buffer is laid out in four contiguous regions ordered by (tensor-parallel duplicate?,
  weight-decay?), so the sharded optimizer and the grad-norm code can treat each rank's shard
  as at most four plain ranges instead of walking per-parameter maps.
* Buckets are sized for launch latency / overlap on NVSwitch (default 512 MiB), not link count.
"""

from __future__ import annotations

import contextlib
import dataclasses
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import nn


def _align(n: int, a: int) -> int:
    return (n + a - 1) // a * a


@dataclasses.dataclass
class Region:
    start: int
    end: int
    weight_decay: bool
    tp_duplicate: bool


@dataclasses.dataclass
class Bucket:
    start: int
    end: int
    params: List[nn.Parameter]
    pending: int = 0
    handle: Optional[object] = None
    late: bool = False          # holds TP-partial gradients: synchronised only after their TP reduction


def param_uses_weight_decay(name: str, p: nn.Parameter) -> bool:
    """Megatron's rule: no decay for biases and 1-D parameters (norm weights)."""
    return not (name.endswith(".bias") or p.dim() == 1)


class ParamAndGradBuffer:
    """Flat storage for all trainable parameters of one dtype and their gradients."""

    def __init__(self, named_params: List[Tuple[str, nn.Parameter]], shard_count: int,
                 bucket_bytes: int = 512 << 20, grad_dtype: Optional[torch.dtype] = None, storage=None):
        if not named_params:
            raise ValueError("no parameters")
        self.dtype = named_params[0][1].dtype
        self.grad_dtype = grad_dtype or self.dtype
        self.device = named_params[0][1].device
        self.shard_count = shard_count

        def key(item):
            name, p = item
            dup = not getattr(p, "tensor_model_parallel", False)
            # parameters whose gradients are partial sums over TP sit at the very end: only the last bucket(s) have to
            # wait for that reduction when bucket collectives are overlapped with backward
            return (dup, not param_uses_weight_decay(name, p), bool(getattr(p, "tp_partial_grad", False)))
        ordered = sorted(named_params, key=key)            # stable: keeps model order inside a region
        self.param_index: Dict[nn.Parameter, Tuple[int, int]] = {}
        self.names: Dict[nn.Parameter, str] = {}
        self.regions: List[Region] = []
        off = 0
        cur_key, region_start = None, 0
        for name, p in ordered:
            k = key((name, p))
            if cur_key is not None and k != cur_key:
                self.regions.append(Region(region_start, off, not cur_key[1], cur_key[0]))
                region_start = off
            cur_key = k
            self.param_index[p] = (off, off + p.numel())
            self.names[p] = name
            off = _align(off + p.numel(), 8)              # keep every parameter 16-byte aligned
        self.regions.append(Region(region_start, off, not cur_key[1], cur_key[0]))
        # every shard boundary stays 16-byte aligned
        self.numel = _align(off, 8 * shard_count)
        self.regions[-1].end = self.numel
        if storage is None:
            self.param_data = torch.zeros(self.numel, dtype=self.dtype, device=self.device)
            self.grad_data = torch.zeros(self.numel, dtype=self.grad_dtype, device=self.device)
        else:
            # caller-provided storage (a symmetric heap, so that peers can read gradients and write parameters)
            self.param_data, self.grad_data = storage(self.numel, self.dtype, self.grad_dtype)
            self.param_data.zero_()
            self.grad_data.zero_()
        for _, p in ordered:
            s, e = self.param_index[p]
            view = self.param_data[s:e].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.grad = self.grad_data[s:e].view(p.shape)
        self.params = [p for _, p in ordered]
        # buckets in reverse buffer order approximate backward order; each bucket is a multiple of
        # shard_count * 8 elements so reduce-scatter shards stay aligned
        elems = max(_align(bucket_bytes // self.param_data.element_size(), 8 * shard_count), 8 * shard_count)
        self.buckets: List[Bucket] = []
        b0 = 0
        while b0 < self.numel:
            b1 = min(self.numel, b0 + elems)
            ps_ = [p for p in self.params if self.param_index[p][0] < b1 and self.param_index[p][1] > b0]
            self.buckets.append(Bucket(b0, b1, ps_))
            b0 = b1
        self.param_buckets: Dict[nn.Parameter, List[Bucket]] = {p: [] for p in self.params}
        for b in self.buckets:
            for p in b.params:
                self.param_buckets[p].append(b)

    def shard_range(self, bucket: Bucket, rank: int) -> Tuple[int, int]:
        n = (bucket.end - bucket.start) // self.shard_count
        return bucket.start + rank * n, bucket.start + (rank + 1) * n

    def rebind_grads(self) -> None:
        """Make sure every ``param.grad`` still aliases the flat buffer (after ``zero_grad(set_to_none)``)."""
        for p in self.params:
            s, e = self.param_index[p]
            if p.grad is None or p.grad.data_ptr() != self.grad_data[s:e].data_ptr():
                p.grad = self.grad_data[s:e].view(p.shape)


def allreduce_tp_partial_grads(params, tp_group) -> None:
    """Sum over tensor-parallel ranks the gradients of replicated parameters whose gradient is only a
    per-rank share (``param.tp_partial_grad``: the per-head q/k RMSNorm weights)."""
    if tp_group is None or dist.get_world_size(tp_group) == 1:
        return
    grads = [p.grad for p in params if getattr(p, "tp_partial_grad", False) and p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=tp_group)
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()


class DistributedDataParallel(nn.Module):
    """Data-parallel wrapper over the DP x CP group with bucketed, optionally overlapped sync."""

    def __init__(self, module: nn.Module, group=None, use_distributed_optimizer: bool = True,
                 overlap_grad_reduce: bool = False, bucket_bytes: int = 512 << 20,
                 grad_dtype: Optional[torch.dtype] = None, check_for_nan_in_grad: bool = False, tp_group=None,
                 fused_comm: bool = False):
        super().__init__()
        self.module = module
        self.group = group
        self.world = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        self.use_distributed_optimizer = use_distributed_optimizer
        self.overlap_grad_reduce = overlap_grad_reduce and self.world > 1
        self.check_for_nan_in_grad = check_for_nan_in_grad
        named = [(n, p) for n, p in module.named_parameters() if p.requires_grad]
        by_dtype: Dict[torch.dtype, List[Tuple[str, nn.Parameter]]] = {}
        for n, p in named:
            by_dtype.setdefault(p.dtype, []).append((n, p))
        self.heap = None
        self.heap_offsets = None
        storage = None
        from . import state as _ps
        if (fused_comm and self.world > 1 and len(by_dtype) == 1 and named[0][1].is_cuda and named[0][1].dtype == torch.bfloat16
                and _ps.group_is_single_node(group)):          # peers on other hosts cannot be mapped: NCCL path
            # gradient reduce-scatter and parameter all-gather by in-kernel NVLink loads / stores: both flat
            # buffers live in a symmetric heap mapped into every data-parallel peer
            from .symm_mem import SymmetricHeap

            def storage(numel, dtype, grad_dtype):
                nbytes = numel * 2
                self.heap = SymmetricHeap(group, 2 * nbytes + 4096)
                po, go = self.heap.alloc(nbytes), self.heap.alloc(nbytes)
                self.heap_offsets = (po, go)
                return self.heap.tensor(po, (numel,), dtype), self.heap.tensor(go, (numel,), grad_dtype)
        self.buffers = [ParamAndGradBuffer(v, self.world, bucket_bytes, grad_dtype, storage) for v in by_dtype.values()]
        self.grad_scale = 1.0 / self.world
        # Set by the optimizer when it reduces the gradients itself, inside its fused reduce-scatter + AdamW + all-gather
        # kernel: finish_grad_sync then only makes every rank's gradients complete and visible.
        self.reduce_in_optimizer = False
        self._sync_enabled = True
        self._hooks = []
        self.tp_group = tp_group
        self._tp_partial = [p for _, p in named if getattr(p, "tp_partial_grad", False)]
        partial = set(self._tp_partial)
        for buf in self.buffers:
            for b in buf.buckets:
                # a bucket that holds TP-partial gradients is synchronised in finish_grad_sync, after their TP reduction
                b.late = any(p in partial for p in b.params)
        # with the symmetric heap, overlapped bucket reductions (and every barrier of this heap that belongs to them) run on
        # one side stream: the barrier's flags only ever grow if the barriers of a heap execute in the order of issue
        self._side = torch.cuda.Stream() if (self.overlap_grad_reduce and self.heap is not None) else None
        if self.overlap_grad_reduce:
            for buf in self.buffers:
                for p in buf.params:
                    self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(buf, p)))
        self._reset_pending()

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    # ---- sync control -------------------------------------------------------------------
    @contextlib.contextmanager
    def no_sync(self):
        prev, self._sync_enabled = self._sync_enabled, False
        try:
            yield
        finally:
            self._sync_enabled = prev

    def _reset_pending(self):
        for buf in self.buffers:
            for b in buf.buckets:
                b.pending = len(b.params)
                b.handle = None

    def _make_hook(self, buf: ParamAndGradBuffer, p: nn.Parameter):
        def hook(_):
            if not self._sync_enabled:
                return
            for b in buf.param_buckets[p]:
                b.pending -= 1
                if b.pending == 0 and not b.late:
                    self._launch(buf, b, async_op=True)
        return hook

    def _launch(self, buf: ParamAndGradBuffer, b: Bucket, async_op: bool):
        g = buf.grad_data[b.start:b.end]
        if self.check_for_nan_in_grad and not torch.isfinite(g.float().sum()):
            raise RuntimeError("non-finite gradient in bucket [%d, %d)" % (b.start, b.end))
        if self.world == 1:
            return
        if self.heap is not None and self.use_distributed_optimizer:
            # peers' buckets are read over NVLink and summed in fp32 with the 1/(dp*cp) scale folded in
            from ..ops import fused_comm as FC
            s, e = buf.shard_range(b, self.rank)
            if self._side is not None:
                # overlapped with backward: once this bucket's gradients are complete on the compute stream, the side
                # stream meets the peers at a barrier (their copies of the bucket are complete too) and reduces this
                # rank's shard.  The shard it writes is the part of this rank's bucket that no peer reads.
                ready = torch.cuda.Event()
                ready.record()
                with torch.cuda.stream(self._side):
                    self._side.wait_event(ready)
                    self.heap.barrier()
                    FC.fused_grad_reduce_scatter(self.heap, self.heap_offsets[1], s, e - s, buf.grad_data[s:e], self.grad_scale)
                b.handle = "fused-side"
                return
            FC.fused_grad_reduce_scatter(self.heap, self.heap_offsets[1], s, e - s, buf.grad_data[s:e], self.grad_scale)
            b.handle = "fused"
            return
        from ..ops import _lib
        with _lib.phase("nccl gradient reduce"):
            g.mul_(self.grad_scale)
            if self.use_distributed_optimizer:
                s, e = buf.shard_range(b, self.rank)
                b.handle = dist.reduce_scatter_tensor(buf.grad_data[s:e], g, group=self.group, async_op=async_op)
            else:
                b.handle = dist.all_reduce(g, group=self.group, async_op=async_op)

    def start_grad_sync(self):
        for buf in self.buffers:
            for b in buf.buckets:
                if b.handle is None and not b.late:
                    self._launch(buf, b, async_op=True)

    def finish_grad_sync(self):
        """Wait for (or issue) every bucket collective; afterwards each rank's shard holds the
        averaged gradient (ZeRO-1) or the whole buffer does (all-reduce mode)."""
        allreduce_tp_partial_grads(self._tp_partial, self.tp_group)
        if self._side is not None:
            # buckets not yet launched (those with TP-partial gradients, or all of them after no_sync micro-batches) go
            # through the same side-stream path; the closing barrier is issued there as well, then the compute stream joins
            for buf in self.buffers:
                for b in buf.buckets:
                    if b.handle is None:
                        self._launch(buf, b, async_op=True)
            with torch.cuda.stream(self._side):
                self.heap.barrier()    # all peers have read this rank's buckets; they may be overwritten again
            torch.cuda.current_stream().wait_stream(self._side)
            self._reset_pending()
            return
        if self.heap is not None:
            self.heap.barrier()        # every rank's gradients are complete before anyone reads them
        if self.reduce_in_optimizer and self.heap is not None:
            if self.check_for_nan_in_grad:
                for buf in self.buffers:
                    if not torch.isfinite(buf.grad_data.float().sum()):
                        raise RuntimeError("non-finite gradient")
            self._reset_pending()
            return
        for buf in self.buffers:
            for b in buf.buckets:
                if b.handle is None:
                    self._launch(buf, b, async_op=False)
                elif hasattr(b.handle, "wait"):
                    b.handle.wait()
        if self.heap is not None:
            self.heap.barrier()        # all peers have read this rank's buckets; they may be overwritten again
        self._reset_pending()

    def zero_grad_buffer(self):
        for buf in self.buffers:
            buf.grad_data.zero_()
            buf.rebind_grads()
        self._reset_pending()

    def broadcast_params(self):
        """Make every DP x CP replica start from rank 0's weights."""
        if self.world == 1:
            return
        src = dist.get_global_rank(self.group, 0)
        for buf in self.buffers:
            dist.broadcast(buf.param_data, src=src, group=self.group)

    def state_dict_for_save_checkpoint(self, prefix: str = "", keep_vars: bool = False):
        m = self.module
        if hasattr(m, "state_dict_for_save_checkpoint"):
            return m.state_dict_for_save_checkpoint(prefix=prefix, keep_vars=keep_vars)
        return m.state_dict(prefix=prefix, keep_vars=keep_vars)

    def load_state_dict(self, state_dict, strict: bool = True):
        return self.module.load_state_dict(state_dict, strict=strict)
