"""Autograd-aware collectives for context and tensor parallelism.

Public names follow the reference (``teletron/core/tensor_parallel/mappings.py:9-58``)
plus the Ulysses all-to-all that the reference borrows from ``yunchang``
(``teletron/models/dit/dit_attention.py:276-279``) and Megatron's TP region mappings.

All functions degrade to identity when the group is ``None`` / has one rank, so the
model code has a single path for every parallel configuration.  The transports here
are ``torch.distributed`` (NCCL on GPU, gloo on CPU); the in-kernel NVLink variants
live in :mod:`teletron_b200.ops.fused_comm` and share these autograd contracts.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _phase(name: str):
    from ..ops import _lib
    return _lib.phase(name)


def _size(group) -> int:
    return 1 if group is None else dist.get_world_size(group)


def _rank(group) -> int:
    return 0 if group is None else dist.get_rank(group)


def _scale(grad: torch.Tensor, mode: Optional[str], n: int) -> torch.Tensor:
    if mode == "up":
        return grad * n
    if mode == "down":
        return grad / n
    if mode is None:
        return grad
    raise ValueError(f"grad_scale must be 'up', 'down' or None, got {mode!r}")


def _split(x: torch.Tensor, group, dim: int, sizes: Optional[List[int]]) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    r = _rank(group)
    if sizes is None:
        if x.size(dim) % n:
            raise ValueError(f"dim {dim} of size {x.size(dim)} is not divisible by {n}")
        step = x.size(dim) // n
        return x.narrow(dim, r * step, step).contiguous()
    start = sum(sizes[:r])
    return x.narrow(dim, start, sizes[r]).contiguous()


def _gather(x: torch.Tensor, group, dim: int, sizes: Optional[List[int]]) -> torch.Tensor:
    n = _size(group)
    if n == 1:
        return x
    x = x.contiguous()
    if sizes is None and dim == 0:
        out = torch.empty((n * x.size(0),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out
    if sizes is None:
        # gather on dim 0 of a staging buffer, then fold into `dim` with one permute
        out = torch.empty((n * x.size(0),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return torch.cat(out.view((n,) + tuple(x.shape)).unbind(0), dim=dim)
    parts = []
    for s in sizes:
        shape = list(x.shape)
        shape[dim] = s
        parts.append(torch.empty(shape, dtype=x.dtype, device=x.device))
    dist.all_gather(parts, x, group=group)
    return torch.cat(parts, dim=dim)


class _SplitFwdGatherBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim, sizes, grad_scale):
        ctx.group, ctx.dim, ctx.sizes, ctx.grad_scale = group, dim, sizes, grad_scale
        return _split(x, group, dim, sizes)

    @staticmethod
    def backward(ctx, g):
        g = _scale(g, ctx.grad_scale, _size(ctx.group))
        return _gather(g, ctx.group, ctx.dim, ctx.sizes), None, None, None, None


class _GatherFwdSplitBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim, sizes, grad_scale):
        ctx.group, ctx.dim, ctx.sizes, ctx.grad_scale = group, dim, sizes, grad_scale
        return _gather(x, group, dim, sizes)

    @staticmethod
    def backward(ctx, g):
        g = _scale(g, ctx.grad_scale, _size(ctx.group))
        return _split(g, ctx.group, ctx.dim, ctx.sizes), None, None, None, None


def split_forward_gather_backward(x, group, dim: int, split_sizes: Optional[List[int]] = None,
                                  grad_scale: Optional[str] = "down"):
    """Keep this rank's chunk along ``dim``; backward all-gathers (scaled) grads."""
    if _size(group) == 1:
        return x
    return _SplitFwdGatherBwd.apply(x, group, dim, split_sizes, grad_scale)


def gather_forward_split_backward(x, group, dim: int, gather_sizes: Optional[List[int]] = None,
                                  grad_scale: Optional[str] = "up"):
    """All-gather along ``dim``; backward keeps this rank's (scaled) grad chunk."""
    if _size(group) == 1:
        return x
    return _GatherFwdSplitBwd.apply(x, group, dim, gather_sizes, grad_scale)


# ---------------------------------------------------------------------------------------------
# Ulysses sequence <-> head all-to-all
# ---------------------------------------------------------------------------------------------

def _a2a_heads_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    """``[B, H, s, D]`` (all heads, local tokens) -> ``[B, H/P, s*P, D]`` (local heads, all tokens)."""
    P = _size(group)
    B, H, s, D = x.shape
    if H % P:
        raise ValueError(f"{H} heads cannot be scattered over {P} context-parallel ranks")
    # send buffer: [P, B, H/P, s, D], chunk p goes to rank p
    send = x.reshape(B, P, H // P, s, D).permute(1, 0, 2, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[p] holds tokens of source rank p: concatenate along the sequence in rank order
    return recv.permute(1, 2, 0, 3, 4).reshape(B, H // P, P * s, D)


def _a2a_seq_to_heads(x: torch.Tensor, group) -> torch.Tensor:
    """Inverse of :func:`_a2a_heads_to_seq`: ``[B, H/P, s*P, D]`` -> ``[B, H, s, D]``."""
    P = _size(group)
    B, h, S, D = x.shape
    if S % P:
        raise ValueError(f"sequence {S} is not divisible by {P}")
    s = S // P
    send = x.reshape(B, h, P, s, D).permute(2, 0, 1, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 0, 2, 3, 4).reshape(B, P * h, s, D)


class _ScatterHeadsGatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a_heads_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a_seq_to_heads(g.contiguous(), ctx.group), None


class _ScatterSeqGatherHeads(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _a2a_seq_to_heads(x, group)

    @staticmethod
    def backward(ctx, g):
        return _a2a_heads_to_seq(g.contiguous(), ctx.group), None


def ulysses_scatter_heads(x: torch.Tensor, group) -> torch.Tensor:
    """Sequence-sharded ``[B, H, s, D]`` -> head-sharded ``[B, H/P, S, D]`` (autograd: inverse a2a)."""
    if _size(group) == 1:
        return x
    return _ScatterHeadsGatherSeq.apply(x, group)


def ulysses_gather_heads(x: torch.Tensor, group) -> torch.Tensor:
    """Head-sharded ``[B, H/P, S, D]`` -> sequence-sharded ``[B, H, s, D]``."""
    if _size(group) == 1:
        return x
    return _ScatterSeqGatherHeads.apply(x, group)


# ---------------------------------------------------------------------------------------------
# Tensor-parallel region mappings (Megatron semantics, no sequence parallelism)
# ---------------------------------------------------------------------------------------------

class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        with _phase("nccl tp all-reduce (bwd)"):
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        # reduced in place when the partial product is a dense tensor of its own (the usual case: a fresh GEMM output);
        # no copy of the activation is made
        if x.is_contiguous() and x._base is None and not x.is_leaf:
            ctx.mark_dirty(x)
        else:
            x = x.contiguous().clone()
        with _phase("nccl tp all-reduce (fwd)"):
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _GatherFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather(x, group, x.dim() - 1, None)

    @staticmethod
    def backward(ctx, g):
        return _split(g, ctx.group, g.dim() - 1, None), None


def copy_to_tensor_model_parallel_region(x, group):
    """Identity forward, all-reduce backward (input of a column-parallel linear)."""
    if _size(group) == 1:
        return x
    return _CopyToTP.apply(x, group)


def reduce_from_tensor_model_parallel_region(x, group):
    """All-reduce forward, identity backward (output of a row-parallel linear)."""
    if _size(group) == 1:
        return x
    return _ReduceFromTP.apply(x, group)


def gather_from_tensor_model_parallel_region(x, group):
    """All-gather along the last dim forward, split backward (modulation vectors)."""
    if _size(group) == 1:
        return x
    return _GatherFromTP.apply(x, group)


# ---------------------------------------------------------------------------------------------
# Sequence parallelism over the tensor-parallel group: the residual stream is sharded along the
# token dim between the column- and row-parallel linears (all-gather in, reduce-scatter out)
# ---------------------------------------------------------------------------------------------

def _reduce_scatter(x: torch.Tensor, group, dim: int) -> torch.Tensor:
    """Sum over the group, keep this rank's chunk of ``dim``."""
    n = _size(group)
    if n == 1:
        return x
    if x.size(dim) % n:
        raise ValueError(f"dim {dim} of size {x.size(dim)} is not divisible by {n}")
    if dim != 0:
        step = x.size(dim) // n
        x = torch.cat(x.split(step, dim=dim), dim=0)        # chunk r of `dim` becomes row block r
    x = x.contiguous()
    out = torch.empty((x.size(0) // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.reduce_scatter_tensor(out, x, group=group)
    return out


class _GatherSeqFwdReduceScatterBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _gather(x, group, dim, None)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter(g, ctx.group, ctx.dim), None, None


class _ReduceScatterSeqFwdGatherBwd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        return _reduce_scatter(x, group, dim)

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.group, ctx.dim, None), None, None


class _GatherFromTPReduceGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather(x, group, x.dim() - 1, None)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter(g, ctx.group, g.dim() - 1), None


def scatter_to_sequence_parallel_region(x, group, dim: int = 1):
    """Keep this rank's token block; backward all-gathers the blocks' gradients."""
    return split_forward_gather_backward(x, group, dim, grad_scale=None)


def gather_from_sequence_parallel_region(x, group, dim: int = 1):
    """All-gather token blocks (input of a column-parallel linear); backward reduce-scatters."""
    if _size(group) == 1:
        return x
    return _GatherSeqFwdReduceScatterBwd.apply(x, group, dim)


def reduce_scatter_to_sequence_parallel_region(x, group, dim: int = 1):
    """Sum the partial outputs of a row-parallel linear and keep this rank's token block."""
    if _size(group) == 1:
        return x
    return _ReduceScatterSeqFwdGatherBwd.apply(x, group, dim)


def gather_from_tensor_model_parallel_region_reduce_grad(x, group):
    """All-gather along the last dim; backward sums the gradients over the group before the split.  For a replicated
    result (modulation vectors) whose consumers each see only part of the tokens."""
    if _size(group) == 1:
        return x
    return _GatherFromTPReduceGrad.apply(x, group)


class _SplitTokens(torch.autograd.Function):
    """``x[:, :n], x[:, n:]`` whose backward is one concatenation.  Two plain slices would each get a zero-filled
    full-size gradient with the slice copied in, and the two would then be added: three passes over the whole tensor
    where one copy suffices (measured at 450 us against 65 us per split of a [1, 32656, 3072] bf16 tensor)."""

    @staticmethod
    def forward(ctx, x, n):
        ctx.n = n
        return x[:, :n], x[:, n:]

    @staticmethod
    def backward(ctx, da, db):
        return torch.cat([da, db], dim=1), None


def split_tokens(x: torch.Tensor, n: int):
    """Split ``[B, N, ...]`` after ``n`` tokens (views of ``x``; do not modify them in place)."""
    if not x.requires_grad or not torch.is_grad_enabled():
        return x[:, :n], x[:, n:]
    return _SplitTokens.apply(x, n)
