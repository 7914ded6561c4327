"""Dual-stream and single-stream MMDiT blocks with tensor + Ulysses context parallelism.

Behaviour follows ``teletron/models/dit/dit_layerspec.py:81-186`` (dual block),
``:248-358`` (single block), ``teletron/models/dit/dit_attention.py:43-338`` /
``:340-504`` (joint / single attention) and ``teletron/models/dit/dit_fusedlayers.py:155-272``
(AdaLN-zero modulation).  Parameter names match the reference's Megatron/TE modules so
its converted checkpoints load: ``norm1.linear``, ``self_attention.linear_qkv``,
``self_attention.added_linear_qkv``, ``self_attention.linear_proj``,
``self_attention.{q,k,added_q,added_k}_layernorm.weight``, ``mlp.linear_fc1/2``,
``ff_context.linear_fc1/2``, ``norm.linear``, ``proj_mlp``, ``proj_out``.

The structure is not Megatron's: blocks are plain modules over the functional op layer
(:mod:`teletron_b200.ops`), and the hot sequence is expressed with the fused ops that
the sm_100a kernels implement (LayerNorm+modulate, QKV GEMM + QK-RMSNorm + RoPE,
projection GEMM + gate + residual, GEMM + GELU).
"""

from __future__ import annotations

import collections
import os
from typing import Optional, Sequence, Tuple

import torch
from torch import nn
import torch.nn.functional as F

from ... import ops
from ...parallel import mappings as M
from ...parallel import state as ps
from ...parallel.pad import SeqPad


# ---------------------------------------------------------------------------------------------
# Tensor-parallel linears
# ---------------------------------------------------------------------------------------------

def _mark(param: nn.Parameter, *, partition_dim: Optional[int], full_shape: Sequence[int],
          init: str, partitions: Optional[Sequence[int]] = None) -> None:
    """Attach sharding / init metadata used by init, checkpointing and the converter."""
    param.partition_dim = partition_dim          # None = replicated over tensor-parallel ranks
    param.full_shape = tuple(full_shape)
    param.init_kind = init                       # "normal" | "scaled_normal" | "zeros" | "ones"
    param.partitions = tuple(partitions) if partitions else None
    param.tensor_model_parallel = partition_dim is not None


def tp_region_input(x: torch.Tensor, sequence_parallel: bool) -> torch.Tensor:
    """What a column-parallel linear consumes: the replicated activation (gradients all-reduced), or with sequence
    parallelism the all-gather of the token blocks (gradients reduce-scattered)."""
    g = ps.get_tensor_model_parallel_group()
    if sequence_parallel:
        return M.gather_from_sequence_parallel_region(x, g, dim=1)
    return M.copy_to_tensor_model_parallel_region(x, g)


def tp_region_output(y: torch.Tensor, sequence_parallel: bool, row_splits: Optional[Sequence[int]] = None) -> torch.Tensor:
    """Sum of the row-parallel partial products: all-reduce, or with sequence parallelism a reduce-scatter over the
    token dim.  ``row_splits`` names token groups (video, text) that are sharded separately."""
    g = ps.get_tensor_model_parallel_group()
    if not sequence_parallel:
        return M.reduce_from_tensor_model_parallel_region(y, g)
    if row_splits is None:
        return M.reduce_scatter_to_sequence_parallel_region(y, g, dim=1)
    parts = [M.reduce_scatter_to_sequence_parallel_region(t, g, dim=1) for t in y.split(list(row_splits), dim=1)]
    return torch.cat(parts, dim=1)


class ColumnParallelLinear(nn.Module):
    """``y = act(x W^T + b)`` with ``W`` sharded over output features (rows)."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, tp: int = 1,
                 sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        self.sequence_parallel = sequence_parallel and tp > 1
        if out_features % tp:
            raise ValueError(f"out_features {out_features} not divisible by tp {tp}")
        self.in_features, self.out_features, self.tp = in_features, out_features, tp
        self.weight = nn.Parameter(torch.empty(out_features // tp, in_features, device=device, dtype=dtype))
        _mark(self.weight, partition_dim=0 if tp > 1 else None, full_shape=(out_features, in_features), init="normal")
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features // tp, device=device, dtype=dtype))
            _mark(self.bias, partition_dim=0 if tp > 1 else None, full_shape=(out_features,), init="zeros")
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor, activation: Optional[str] = None, in_region: bool = False) -> torch.Tensor:
        """``in_region``: the caller already applied :func:`tp_region_input` (one gather shared by several linears)."""
        if not in_region:
            x = tp_region_input(x, self.sequence_parallel)
        return ops.linear(x, self.weight, self.bias, activation)


class RowParallelLinear(nn.Module):
    """``y = x W^T + b`` with ``W`` sharded over input features; output all-reduced over TP.

    ``input_partitions`` describes an input made of several concatenated feature
    groups that are *each* sharded (the single block's ``proj_out`` consumes
    ``[attn 3072/tp | mlp 12288/tp]``, ``convert_hunyuanvideo.py:578-589``).
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, tp: int = 1,
                 input_partitions: Optional[Sequence[int]] = None, sequence_parallel: bool = False,
                 device=None, dtype=None):
        super().__init__()
        self.sequence_parallel = sequence_parallel and tp > 1
        if in_features % tp:
            raise ValueError(f"in_features {in_features} not divisible by tp {tp}")
        self.in_features, self.out_features, self.tp = in_features, out_features, tp
        self.weight = nn.Parameter(torch.empty(out_features, in_features // tp, device=device, dtype=dtype))
        _mark(self.weight, partition_dim=1 if tp > 1 else None, full_shape=(out_features, in_features),
              init="scaled_normal", partitions=input_partitions)
        if bias:
            self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype))
            _mark(self.bias, partition_dim=None, full_shape=(out_features,), init="zeros")
            # with sequence parallelism every rank adds the bias to its token block only: the gradient is a partial sum
            self.bias.tp_partial_grad = self.sequence_parallel
        else:
            self.register_parameter("bias", None)

    def forward(self, x: torch.Tensor, row_splits: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Projection, TP all-reduce (or reduce-scatter over tokens), bias (added once, after the reduction)."""
        if self.tp == 1:
            return ops.linear(x, self.weight, self.bias)
        y = ops.linear(x, self.weight, None)
        y = tp_region_output(y, self.sequence_parallel, row_splits)
        return y if self.bias is None else y + self.bias

    def forward_merged(self, x1: torch.Tensor, x2: torch.Tensor, row_splits: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Same for an input given as its two feature groups (``input_partitions``): ``cat([x1, x2], -1)`` is projected,
        and the backward keeps the two gradients apart (:func:`teletron_b200.ops.linear_merged`)."""
        if self.tp == 1:
            return ops.linear_merged(x1, x2, self.weight, self.bias)
        y = ops.linear_merged(x1, x2, self.weight, None)
        y = tp_region_output(y, self.sequence_parallel, row_splits)
        return y if self.bias is None else y + self.bias



class RMSNorm(nn.Module):
    """Per-head RMSNorm.  ``tp_partial`` marks a weight that is shared by heads living on different
    tensor-parallel ranks: each rank then sees only its heads' share of the gradient, and the shares
    must be summed over TP before the optimizer step (the reference omits this reduction, so its
    q/k norm weights drift apart between TP ranks)."""

    def __init__(self, dim: int, eps: float = 1e-6, tp_partial: bool = False, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        _mark(self.weight, partition_dim=None, full_shape=(dim,), init="ones")
        self.weight.tp_partial_grad = tp_partial

    def forward(self, x):
        return ops.rmsnorm(x, self.weight, self.eps)


class AdaLNModulation(nn.Module):
    """``Linear(SiLU(temb))`` producing ``n_chunks`` modulation vectors.

    Column-parallel over TP followed by an all-gather of the (tiny) output, as in
    ``dit_fusedlayers.py:216-218``.  The LayerNorm itself is applied by the caller
    through :func:`teletron_b200.ops.layernorm_modulate`.
    """

    def __init__(self, dim: int, n_chunks: int, tp: int = 1, sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        self.n_chunks = n_chunks
        self.sequence_parallel = sequence_parallel and tp > 1
        # temb is replicated (never token-sharded): the linear itself takes no sequence-parallel gather
        self.linear = ColumnParallelLinear(dim, n_chunks * dim, bias=True, tp=tp, device=device, dtype=dtype)

    def forward(self, temb: torch.Tensor) -> Tuple[torch.Tensor, ...]:
        emb = self.linear(F.silu(temb))
        g = ps.get_tensor_model_parallel_group()
        if self.sequence_parallel:
            # each rank modulates its own token block, so the vectors' gradients are partial sums over TP
            emb = M.gather_from_tensor_model_parallel_region_reduce_grad(emb, g)
        else:
            emb = M.gather_from_tensor_model_parallel_region(emb, g)
        return emb.chunk(self.n_chunks, dim=1)


class ParallelMLP(nn.Module):
    """``linear_fc1`` (column-parallel) -> activation -> ``linear_fc2`` (row-parallel)."""

    def __init__(self, dim: int, hidden: int, activation: str, tp: int = 1, sequence_parallel: bool = False,
                 device=None, dtype=None):
        super().__init__()
        self.activation = activation
        kw = dict(tp=tp, sequence_parallel=sequence_parallel, device=device, dtype=dtype)
        self.linear_fc1 = ColumnParallelLinear(dim, hidden, **kw)
        self.linear_fc2 = RowParallelLinear(hidden, dim, **kw)

    def forward(self, x):
        if _use_fused_tp(x, self.linear_fc1.sequence_parallel, self.activation):
            # token-sharded input: all-gather -> GEMM (+ activation), then GEMM -> reduce-scatter, both in-kernel over NVLink
            from ...ops import fused_comm as FC
            ws = _tp_workspace(x.shape[1], self.linear_fc1.in_features, self.linear_fc2.out_features)
            h = FC.sp_column_linear(ws, x[0], self.linear_fc1.weight, self.linear_fc1.bias, self.activation)
            return FC.sp_row_linear(ws, h, self.linear_fc2.weight, self.linear_fc2.bias)[None]
        return self.linear_fc2(self.linear_fc1(x, activation=self.activation))


# ---------------------------------------------------------------------------------------------
# Attention with Ulysses context parallelism
# ---------------------------------------------------------------------------------------------

def _joint_attention(q, k, v, text_len: int, kv_valid_len: Optional[int]):
    """Single-rank case: q, k, v already hold ``cat(video, text)`` as ``[B, h, S + T, D]``."""
    S = q.shape[2] - text_len
    o = ops.attention(q, k, v, kv_valid_len=None if kv_valid_len is None else S + kv_valid_len)
    return M.split_tokens(o, S)


def _ulysses_attention(q, k, v, tq, tk, tv, pad: Optional[SeqPad], kv_valid_len: Optional[int]):
    """Joint attention over ``cat(video, text)`` with the Ulysses exchange.

    ``q, k, v``: video ``[B, H/tp, s, D]`` (sequence-sharded over CP); ``tq, tk, tv``: text
    ``[B, H/tp, T, D]`` (replicated over CP).  Returns token-major video ``[B, s, H/tp*D]``
    and text ``[B, T, H/tp*D]`` (call sites X1-X4 of the reference:
    ``dit_attention.py:275-297, 321-327``).
    """
    cp_group = ps.get_context_parallel_group()
    cp = ps.get_context_parallel_world_size()
    T = tq.shape[2]
    if cp > 1:
        q = M.ulysses_scatter_heads(q, cp_group)
        k = M.ulysses_scatter_heads(k, cp_group)
        v = M.ulysses_scatter_heads(v, cp_group)
        tq = M.split_forward_gather_backward(tq, cp_group, dim=1, grad_scale="down")
        tk = M.split_forward_gather_backward(tk, cp_group, dim=1, grad_scale="down")
        tv = M.split_forward_gather_backward(tv, cp_group, dim=1, grad_scale="down")
        if pad is not None and pad.pad:
            q, k, v = (pad.remove(t, 2) for t in (q, k, v))
    S = q.shape[2]
    o = ops.attention(torch.cat([q, tq], dim=2), torch.cat([k, tk], dim=2), torch.cat([v, tv], dim=2),
                      kv_valid_len=None if kv_valid_len is None else S + kv_valid_len)
    o_v, o_t = o[:, :S], o[:, S:]
    if cp > 1:
        B, _, hd = o_v.shape
        D = q.shape[-1]
        if pad is not None and pad.pad:
            o_v = pad.add(o_v, 1)
        o_v = M.ulysses_gather_heads(o_v.reshape(B, o_v.shape[1], hd // D, D).transpose(1, 2), cp_group)
        o_v = o_v.transpose(1, 2).reshape(B, -1, cp * hd)
        o_t = M.gather_forward_split_backward(o_t.contiguous(), cp_group, dim=2, grad_scale="up")
    return o_v, o_t.reshape(o_t.shape[0], T, -1)


_FUSED_COMM = False
# Collective workspaces (symmetric heaps) by kind, least recently used first.  One workspace per kind serves every clip
# length (it is re-laid-out in place, see _workspace); the cache bound only matters for models with several head counts or
# widths.  Every rank of a group sees the same sequence of shapes, so all of them make the same decisions.
_WORKSPACES = collections.OrderedDict()
_MAX_WORKSPACES = int(os.environ.get("TELETRON_B200_MAX_WORKSPACES", "8"))


def _cached_workspace(key, make):
    ws = _WORKSPACES.get(key)
    if ws is not None:
        _WORKSPACES.move_to_end(key)
        return ws
    while len(_WORKSPACES) >= max(1, _MAX_WORKSPACES):
        _, old = _WORKSPACES.popitem(last=False)
        # the last kernels that used the workspace touch the peers' slabs without a closing barrier: a rank may only
        # free its slab once every peer's work on it has finished, and only after the peers have unmapped it
        old.heap.close(collective=True)
    ws = _WORKSPACES[key] = make()
    return ws


def set_fused_comm(enabled: bool) -> None:
    """Route the Ulysses all-to-alls through the compute + collective fused kernels
    (:mod:`teletron_b200.ops.fused_comm`) instead of NCCL ``all_to_all_single``."""
    global _FUSED_COMM
    _FUSED_COMM = bool(enabled)


def fused_comm_enabled() -> bool:
    return _FUSED_COMM


def _use_fused(x: torch.Tensor, head_dim: int) -> bool:
    return (_FUSED_COMM and ps.get_context_parallel_world_size() > 1 and x.is_cuda and x.dtype == torch.bfloat16
            and x.shape[0] == 1 and head_dim == 128 and ops.get_impl() != "torch"
            and ps.group_is_single_node(ps.get_context_parallel_group()))


_FUSED_TP_MIN_ROWS = 1024      # below this (the text stream) two device barriers cost more than the NCCL collectives


def _use_fused_tp(x: torch.Tensor, sequence_parallel: bool, activation) -> bool:
    """Sequence-parallel MLP through the fused all-gather -> GEMM / GEMM -> reduce-scatter kernels."""
    return (_FUSED_COMM and sequence_parallel and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3
            and x.shape[0] == 1 and x.shape[1] >= _FUSED_TP_MIN_ROWS and ops.get_impl() != "torch"
            and activation in (None, "gelu", "gelu_tanh")
            and ps.group_is_single_node(ps.get_tensor_model_parallel_group()))


# Collective workspaces are sized with head-room (TELETRON_B200_WORKSPACE_HEADROOM, default 1.0 = exactly the first shape)
# and re-laid-out in place when the clip length changes; only a sequence longer than everything seen before makes every
# rank close the slab (collectively) and allocate a larger one.
_HEADROOM = float(os.environ.get("TELETRON_B200_WORKSPACE_HEADROOM", "1.0"))


def _tp_workspace(rows: int, k_max: int, n_max: int):
    from ...ops.fused_comm import TPWorkspace
    width = max(k_max, n_max)
    key = ("tp", width)
    ws = _WORKSPACES.get(key)
    if ws is not None and not ws.fits(rows):
        del _WORKSPACES[key]
        ws.heap.close(collective=True)
        ws = None
    if ws is None:
        ws = _cached_workspace(key, lambda: TPWorkspace(ps.get_tensor_model_parallel_group(), rows, width, width,
                                                        capacity_rows=int(rows * _HEADROOM)))
    elif ws.rows != rows:
        ws.configure(rows)
    return _cached_workspace(key, lambda: ws)


def _workspace(heads_local: int, s: int, T: int):
    from ...ops.fused_comm import UlyssesWorkspace
    key = ("ulysses", heads_local)
    ws = _WORKSPACES.get(key)
    if ws is not None and not ws.fits(s, T):
        del _WORKSPACES[key]
        ws.heap.close(collective=True)
        ws = None
    if ws is None:
        group = ps.get_context_parallel_group()
        cp = ps.get_context_parallel_world_size()
        cap = int(UlyssesWorkspace.bytes_needed(heads_local, cp, s, T) * _HEADROOM)
        ws = _cached_workspace(key, lambda: UlyssesWorkspace(group, heads_local, s, T, capacity_bytes=cap))
    elif (ws.s, ws.T) != (s, T):
        ws.configure(s, T)
    return _cached_workspace(key, lambda: ws)


def _fused_kv_len(ws, pad: Optional[SeqPad], kv_valid_len):
    """``(kv_len, mask_range)`` for the fused layout ``[text | video of rank 0 | video of rank 1 | ...]``: context-parallel
    padding is the sequence tail (a key length), padded text tokens ``[kv_valid_len, T)`` are a range of their own."""
    kv_len = None if pad is None or pad.pad == 0 else ws.T + pad.origin
    mask = None if kv_valid_len is None or kv_valid_len >= ws.T else (int(kv_valid_len), ws.T)
    return kv_len, mask


class JointAttention(nn.Module):
    """Dual-stream attention: separate QKV / out projections for video and text tokens."""

    def __init__(self, dim: int, heads: int, head_dim: int, tp: int, eps: float, qkv_bias: bool = True,
                 sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.heads_local, self.head_dim, self.eps = heads // tp, head_dim, eps
        self.sequence_parallel = sp = sequence_parallel and tp > 1
        self.linear_qkv = ColumnParallelLinear(dim, 3 * dim, bias=qkv_bias, tp=tp, sequence_parallel=sp, **kw)
        self.added_linear_qkv = ColumnParallelLinear(dim, 3 * dim, bias=qkv_bias, tp=tp, sequence_parallel=sp, **kw)
        self.linear_proj = RowParallelLinear(dim, dim, tp=tp, sequence_parallel=sp, **kw)
        self.added_linear_proj = RowParallelLinear(dim, dim, tp=tp, sequence_parallel=sp, **kw)
        self.q_layernorm = RMSNorm(head_dim, eps, tp > 1, **kw)
        self.k_layernorm = RMSNorm(head_dim, eps, tp > 1, **kw)
        self.added_q_layernorm = RMSNorm(head_dim, eps, tp > 1, **kw)
        self.added_k_layernorm = RMSNorm(head_dim, eps, tp > 1, **kw)

    def forward(self, x, ctx, cos, sin, pad, kv_valid_len):
        x = tp_region_input(x, self.sequence_parallel)
        ctx = tp_region_input(ctx, self.sequence_parallel)
        if _use_fused(x, self.head_dim):
            return self._forward_fused(x, ctx, cos, sin, pad, kv_valid_len)
        if ps.get_context_parallel_world_size() == 1:
            q, k, v = ops.joint_qkv_projection(
                x, self.linear_qkv.weight, self.linear_qkv.bias, self.q_layernorm.weight, self.k_layernorm.weight,
                cos, sin, ctx, self.added_linear_qkv.weight, self.added_linear_qkv.bias,
                self.added_q_layernorm.weight, self.added_k_layernorm.weight, self.heads_local, self.eps)
            return _joint_attention(q, k, v, ctx.shape[1], kv_valid_len)
        q, k, v = ops.qkv_projection(x, self.linear_qkv.weight, self.linear_qkv.bias, self.q_layernorm.weight,
                                     self.k_layernorm.weight, cos, sin, self.heads_local, self.eps)
        tq, tk, tv = ops.qkv_projection(ctx, self.added_linear_qkv.weight, self.added_linear_qkv.bias,
                                        self.added_q_layernorm.weight, self.added_k_layernorm.weight,
                                        None, None, self.heads_local, self.eps)
        return _ulysses_attention(q, k, v, tq, tk, tv, pad, kv_valid_len)


    def _forward_fused(self, x, ctx, cos, sin, pad, kv_valid_len):
        """QKV GEMM -> (RMSNorm, RoPE, seq->head all-to-all in the epilogue) -> attention; the caller finishes with
        :meth:`project_fused` (head->seq all-to-all inside the output projections)."""
        from ...ops import fused_comm as FC
        ws = _workspace(self.heads_local, x.shape[1], ctx.shape[1])
        q, k, v = FC.fused_qkv_a2a(ws, x, self.linear_qkv.weight, self.linear_qkv.bias, self.q_layernorm.weight,
                                   self.k_layernorm.weight, cos, sin, ctx, self.added_linear_qkv.weight,
                                   self.added_linear_qkv.bias, self.added_q_layernorm.weight,
                                   self.added_k_layernorm.weight, self.eps)
        return ("fused", ws, (q, k, v), _fused_kv_len(ws, pad, kv_valid_len)), None

    def project_fused(self, handle):
        """Attention (its epilogue does the head->seq all-to-all) followed by the two output projections."""
        from ...ops import fused_comm as FC
        _, ws, (q, k, v), (kv_len, mask) = handle
        tp = self.linear_proj.tp
        y, yt = FC.fused_attention_outproj(ws, q, k, v, self.linear_proj.weight, self.linear_proj.bias if tp == 1 else None,
                                           self.added_linear_proj.weight, self.added_linear_proj.bias if tp == 1 else None,
                                           kv_len=kv_len, mask_range=mask)
        if tp > 1:
            y = tp_region_output(y, self.sequence_parallel) + self.linear_proj.bias
            yt = tp_region_output(yt, self.sequence_parallel) + self.added_linear_proj.bias
        return y, yt


class SingleAttention(nn.Module):
    """Single-stream attention: one QKV over ``cat(video, text)``; no output projection."""

    def __init__(self, dim: int, heads: int, head_dim: int, tp: int, eps: float, qkv_bias: bool = True,
                 sequence_parallel: bool = False, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        self.heads_local, self.head_dim, self.eps = heads // tp, head_dim, eps
        self.linear_qkv = ColumnParallelLinear(dim, 3 * dim, bias=qkv_bias, tp=tp, sequence_parallel=sequence_parallel, **kw)
        self.q_layernorm = RMSNorm(head_dim, eps, tp > 1, **kw)
        self.k_layernorm = RMSNorm(head_dim, eps, tp > 1, **kw)

    def forward(self, h, text_len, cos, sin, pad, kv_valid_len, in_region: bool = False):
        if not in_region:
            h = M.copy_to_tensor_model_parallel_region(h, ps.get_tensor_model_parallel_group())
        s = h.shape[1] - text_len
        q, k, v = ops.qkv_projection(h, self.linear_qkv.weight, self.linear_qkv.bias, self.q_layernorm.weight,
                                     self.k_layernorm.weight, cos, sin, self.heads_local, self.eps, rope_len=s)
        if ps.get_context_parallel_world_size() == 1:
            return _joint_attention(q, k, v, text_len, kv_valid_len)
        return _ulysses_attention(q[:, :, :s], k[:, :, :s], v[:, :, :s], q[:, :, s:], k[:, :, s:], v[:, :, s:],
                                  pad, kv_valid_len)


# ---------------------------------------------------------------------------------------------
# Blocks
# ---------------------------------------------------------------------------------------------

class HunyuanDiTLayer(nn.Module):
    """Dual-stream block: video and text keep separate weights and meet in attention."""

    def __init__(self, cfg, tp: int = 1, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        H = cfg.hidden_size
        self.eps = cfg.layernorm_epsilon
        sp = bool(getattr(cfg, "sequence_parallel", False)) and tp > 1
        self.norm1 = AdaLNModulation(H, 6, tp, sp, **kw)
        self.norm1_context = AdaLNModulation(H, 6, tp, sp, **kw)
        self.self_attention = JointAttention(H, cfg.num_attention_heads, cfg.attention_head_dim, tp, self.eps,
                                             cfg.add_qkv_bias, sp, **kw)
        self.mlp = ParallelMLP(H, cfg.mlp_hidden, cfg.dual_mlp_activation, tp, sp, **kw)
        self.ff_context = ParallelMLP(H, cfg.mlp_hidden, cfg.dual_mlp_activation, tp, sp, **kw)

    def forward(self, x, ctx, temb, cos, sin, pad: Optional[SeqPad] = None, kv_valid_len: Optional[int] = None):
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = self.norm1(temb)
        c_shift_msa, c_scale_msa, c_gate_msa, c_shift_mlp, c_scale_mlp, c_gate_mlp = self.norm1_context(temb)
        xn = ops.layernorm_modulate(x, scale_msa, shift_msa, self.eps)
        cn = ops.layernorm_modulate(ctx, c_scale_msa, c_shift_msa, self.eps)
        attn, c_attn = self.self_attention(xn, cn, cos, sin, pad, kv_valid_len)
        if isinstance(attn, tuple):
            a, ca = self.self_attention.project_fused(attn)
        else:
            a = self.self_attention.linear_proj(attn)
            ca = self.self_attention.added_linear_proj(c_attn)
        # residual update and the next LayerNorm + modulation in one pass over the tokens
        x, xn = ops.gate_residual_layernorm_modulate(x, a, gate_msa, scale_mlp, shift_mlp, self.eps)
        ctx, cn = ops.gate_residual_layernorm_modulate(ctx, ca, c_gate_msa, c_scale_mlp, c_shift_mlp, self.eps)
        x = ops.gate_residual(x, self.mlp(xn), gate_mlp)
        ctx = ops.gate_residual(ctx, self.ff_context(cn), c_gate_mlp)
        return x, ctx


class HunyuanSingleDiTLayer(nn.Module):
    """Single-stream block: one set of weights over ``cat(video, text)``; attention and MLP
    run in parallel and are merged by one projection."""

    def __init__(self, cfg, tp: int = 1, device=None, dtype=None):
        super().__init__()
        kw = dict(device=device, dtype=dtype)
        H = cfg.hidden_size
        self.eps = cfg.layernorm_epsilon
        self.activation = cfg.single_mlp_activation
        self.sequence_parallel = sp = bool(getattr(cfg, "sequence_parallel", False)) and tp > 1
        self.norm = AdaLNModulation(H, 3, tp, sp, **kw)
        self.proj_mlp = ColumnParallelLinear(H, cfg.mlp_hidden, tp=tp, sequence_parallel=sp, **kw)
        self.self_attention = SingleAttention(H, cfg.num_attention_heads, cfg.attention_head_dim, tp, self.eps,
                                              cfg.add_qkv_bias, sp, **kw)
        self.proj_out = RowParallelLinear(H + cfg.mlp_hidden, H, tp=tp, input_partitions=(H, cfg.mlp_hidden),
                                          sequence_parallel=sp, **kw)

    def forward(self, x, ctx, temb, cos, sin, pad: Optional[SeqPad] = None, kv_valid_len: Optional[int] = None):
        T_own = ctx.shape[1]                       # text rows held by this rank (all of them without sequence parallelism)
        h = torch.cat([x, ctx], dim=1)
        shift, scale, gate = self.norm(temb)
        hn = ops.layernorm_modulate(h, scale, shift, self.eps)
        sp = self.sequence_parallel
        T, splits = T_own, None
        if sp:
            # video and text token blocks are gathered separately so that the result is [all video | all text]
            hn = torch.cat([tp_region_input(hn[:, :-T_own], True), tp_region_input(hn[:, -T_own:], True)], dim=1)
            T = T_own * self.proj_out.tp
            splits = (hn.shape[1] - T, T)
        mlp = self.proj_mlp(hn, activation=self.activation, in_region=sp)
        if _use_fused(hn, self.self_attention.head_dim):
            proj = self._attention_and_projection_fused(hn, mlp, T, cos, sin, pad, kv_valid_len, in_region=sp)
        else:
            attn, c_attn = self.self_attention(hn, T, cos, sin, pad, kv_valid_len, in_region=sp)
            proj = self.proj_out.forward_merged(torch.cat([attn, c_attn], dim=1), mlp, row_splits=splits)
        h = ops.gate_residual(h, proj, gate)
        return M.split_tokens(h, h.shape[1] - T_own)

    def _attention_and_projection_fused(self, hn, mlp, T, cos, sin, pad, kv_valid_len, in_region: bool = False):
        """Single-stream block with both Ulysses all-to-alls fused: the QKV epilogue scatters heads to their owners and
        the merged projection gathers them back per K block, taking the MLP half of its input from local memory."""
        from ...ops import fused_comm as FC
        sa = self.self_attention
        s = hn.shape[1] - T
        ws = _workspace(sa.heads_local, s, T)
        if not in_region:
            hn = M.copy_to_tensor_model_parallel_region(hn, ps.get_tensor_model_parallel_group())
        xv, xt = hn[:, :s], hn[:, s:]
        w, b = sa.linear_qkv.weight, sa.linear_qkv.bias
        q, k, v = FC.fused_qkv_a2a(ws, xv, w, b, sa.q_layernorm.weight, sa.k_layernorm.weight, cos, sin,
                                   xt, w, b, sa.q_layernorm.weight, sa.k_layernorm.weight, sa.eps)
        tp = self.proj_out.tp
        wo, bo = self.proj_out.weight, (self.proj_out.bias if tp == 1 else None)
        kv_len, mask = _fused_kv_len(ws, pad, kv_valid_len)
        y, yt = FC.fused_attention_outproj(ws, q, k, v, wo, bo, wo, bo, extra=mlp[:, :s], extra_t=mlp[:, s:],
                                           kv_len=kv_len, mask_range=mask)
        proj = torch.cat([y, yt], dim=1)
        if tp > 1:
            proj = tp_region_output(proj, self.sequence_parallel, (s, T) if self.sequence_parallel else None) + self.proj_out.bias
        return proj


class AdaLNContinuous(nn.Module):
    """Output head norm: ``LN(x) * (1 + scale) + shift`` with ``(scale, shift) = Linear(SiLU(temb))``
    (``dit_layerspec.py:55-78``; the linear is ``adaLN_modulation.1``)."""

    def __init__(self, dim: int, cond_dim: int, eps: float = 1e-6, device=None, dtype=None):
        super().__init__()
        self.eps = eps
        self.adaLN_modulation = nn.Sequential(nn.SiLU(), nn.Linear(cond_dim, 2 * dim, device=device, dtype=dtype))

    def forward(self, x, temb):
        scale, shift = self.adaLN_modulation(temb).chunk(2, dim=1)
        return ops.layernorm_modulate(x, scale, shift, self.eps)
