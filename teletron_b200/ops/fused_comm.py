"""Compute + collective fused ops over the symmetric heap (NVLink peer loads / stores from inside the kernels).

* :class:`UlyssesWorkspace` + :func:`fused_qkv_a2a` - QKV GEMM whose epilogue applies bias, QK-RMSNorm and RoPE
  and stores every head tile straight into the buffer of the context-parallel rank that owns the head (the
  sequence -> head all-to-all of ``dit_attention.py:277-279`` fused into the GEMM).  Backward: the inverse
  all-to-all is fused into the RoPE-transpose / RMSNorm-backward kernel, which reads dq / dk / dv from their owners.
* :func:`fused_a2a_linear` - output projection whose A operand is fetched per head from the rank that computed
  that head's attention output (the head -> sequence all-to-all of ``dit_attention.py:325`` fused into the GEMM's
  TMA loads).  Backward: the data-gradient GEMM pushes each head's columns to the head's owner.
* :func:`fused_all_gather_linear` / :func:`fused_linear_reduce_scatter` - tensor-parallel all-gather -> GEMM and
  GEMM -> reduce-scatter on sequence-sharded activations.
* :func:`fused_grad_reduce_scatter` / :func:`fused_param_all_gather` - data-parallel gradient reduce-scatter with the
  1/(dp*cp) scale folded in, and the parameter all-gather by peer stores.

All of them take micro-batch 1 (the only mode the reference's launch scripts use).  Every cross-rank hand-over is
a bounded device-side barrier on the heap (:meth:`SymmetricHeap.barrier`); call ``heap.check()`` at a
synchronisation point to turn a timed-out barrier into :class:`CommTimeoutError`.
"""

from __future__ import annotations

import contextlib
import ctypes
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..parallel.symm_mem import SymmetricHeap
from . import _lib, gemm
from ._lib import c_float, c_int, c_long, check, ptr, stream
from ._lib import call as _call
from .gemm_tcgen05 import status_tensor

BF16 = torch.bfloat16


def _table(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


# Every layer of a model shares one workspace per shape, and q / k / v and the gathered attention output are views
# of that workspace.  Tensors saved for backward may therefore alias it only while nothing else can run between the
# forward that wrote them and the backward that reads them: that is the replay of ONE checkpointed block, which is
# followed at once by that block's backward.  Everywhere else (no recompute, layers beyond --recompute-num-layers,
# a uniform chunk of several blocks) the next layer's forward would overwrite them behind autograd's back, so the
# ops below save private copies instead.
_SINGLE_BLOCK_REPLAY = 0
COUNTERS = {"qkv_gemm_fused": 0, "attn_fwd_push": 0, "gemm_comm": 0, "gemm_ag": 0, "private_saves": 0}


_COUNTED = {"tt_qkv_gemm_fused": "qkv_gemm_fused", "tt_attn_fwd_push": "attn_fwd_push", "tt_gemm_comm_bf16": "gemm_comm",
            "tt_gemm_ag_bf16": "gemm_ag"}


def call(fn_name: str, *args) -> None:
    """Native call that also counts the fused compute + collective launches by kind (reported by the benchmark)."""
    k = _COUNTED.get(fn_name)
    if k is not None:
        COUNTERS[k] += 1
    _call(fn_name, *args)


@contextlib.contextmanager
def single_block_replay():
    """Entered by the block checkpoint while it re-runs exactly one block for that block's own backward."""
    global _SINGLE_BLOCK_REPLAY
    _SINGLE_BLOCK_REPLAY += 1
    try:
        yield
    finally:
        _SINGLE_BLOCK_REPLAY -= 1


def saves_need_private_copies() -> bool:
    return torch.is_grad_enabled() and _SINGLE_BLOCK_REPLAY == 0


class UlyssesWorkspace:
    """Symmetric buffers of one context-parallel group.  The slab is sized once (for the largest sequence it has to hold)
    and :meth:`configure` lays the buffers out for the current ``(local sequence, text length)``: clips of different
    lengths reuse one slab and one set of IPC mappings instead of allocating a heap per shape."""

    NAMES = ("q", "k", "v", "o", "dq", "dk", "dv", "do")

    @staticmethod
    def bytes_needed(heads: int, cp: int, s_local: int, text_len: int) -> int:
        n_qkv = (heads // cp) * (cp * s_local + text_len) * 128 * 2
        n_g = (text_len + s_local) * heads * 128 * 2
        return 8 * (n_qkv + 1024) + n_g + 1024

    def __init__(self, group, heads: int, s_local: int, text_len: int, device=None, heap: Optional[SymmetricHeap] = None,
                 capacity_bytes: Optional[int] = None):
        self.group = group
        self.cp = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        if heads % self.cp:
            raise ValueError(f"{heads} heads cannot be split over {self.cp} context-parallel ranks")
        self.heads, self.h_loc = heads, heads // self.cp
        need = self.bytes_needed(heads, self.cp, s_local, text_len)
        self.capacity = max(need, capacity_bytes or 0)
        self.heap = heap or SymmetricHeap(group, self.capacity, device)
        self.configure(s_local, text_len)

    def fits(self, s_local: int, text_len: int) -> bool:
        return self.bytes_needed(self.heads, self.cp, s_local, text_len) <= self.capacity

    def configure(self, s_local: int, text_len: int) -> None:
        """Lay the buffers out for these sequence lengths (same call on every rank: the offsets stay symmetric).  The first
        fused op that follows starts with a barrier, so no peer still reads the previous layout when it is overwritten."""
        if not self.fits(s_local, text_len):
            raise MemoryError("sequence does not fit the workspace it was sized for")
        self.s, self.T = s_local, text_len
        self.S = self.cp * s_local
        self.S_tot = self.S + text_len
        # token order inside the buffers: [text | video of rank 0 | video of rank 1 | ...].  Text goes first so
        # that context-parallel padding (at the end of the last rank's video tokens) is the tail of the sequence
        # and a plain key-length mask removes it.
        self.text_off = 0
        self.video_off = text_len
        n_qkv = self.h_loc * self.S_tot * 128 * 2                  # bytes of one of q / k / v (batch 1)
        n_g = (text_len + s_local) * self.heads * 128 * 2          # gathered attention output: my tokens, all heads
        self.heap.reset()
        self.off = {n: self.heap.alloc(n_qkv) for n in self.NAMES}
        self.off["g"] = self.heap.alloc(n_g)

    def head_major(self, name: str, rank: Optional[int] = None) -> torch.Tensor:
        return self.heap.tensor(self.off[name], (1, self.h_loc, self.S_tot, 128), BF16, rank)

    def token_major(self, name: str, rank: Optional[int] = None) -> torch.Tensor:
        return self.heap.tensor(self.off[name], (1, self.S_tot, self.h_loc * 128), BF16, rank)

    def table(self, name: str):
        return self.heap.ptr_table(self.off[name])

    def local_table(self, name: str):
        """Every slot points at this rank's buffer (stores that must stay local)."""
        p = self.heap.local_ptr + self.off[name]
        return _table([p] * self.cp)


# ---------------------------------------------------------------------------------------------
# F1: QKV GEMM + QK-RMSNorm + RoPE + sequence -> head all-to-all
# ---------------------------------------------------------------------------------------------

def _qkv_fused_launch(ws: UlyssesWorkspace, x2, w, b, qw, kw, cos, sin, out_off, rope_len, only_local, aux, names=("q", "k", "v")):
    M, K = x2.shape
    tabs = [ws.local_table(n) if only_local else ws.table(n) for n in names]
    call("tt_qkv_gemm_fused", ptr(x2), ptr(w), ptr(b), ptr(qw), ptr(kw), ptr(cos), ptr(sin), tabs[0], tabs[1], tabs[2],
         c_int(ws.cp), c_int(ws.rank), ptr(aux), c_int(M), c_int(ws.heads), c_int(K), c_int(M), c_int(ws.S_tot),
         c_int(out_off), c_int(rope_len), c_int(1 if only_local else 0), c_float(1e-6), ptr(status_tensor(x2.device)),
         stream())


class _FusedQKVAllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ws, eps, cos, sin, x, w, b, qw, kw, xt, wt, bt, qwt, kwt):
        s, T = x.shape[1], xt.shape[1]
        if x.shape[0] != 1 or s != ws.s or T != ws.T:
            raise _lib.NativeError("fused Ulysses ops take micro-batch 1 and the workspace's sequence lengths")
        x2 = check(x.reshape(s, -1).contiguous(), BF16, "x")
        xt2 = check(xt.reshape(T, -1).contiguous(), BF16, "xt")
        cosf = check(cos.float().contiguous(), torch.float32, "cos")
        sinf = check(sin.float().contiguous(), torch.float32, "sin")
        need_grad = any(ctx.needs_input_grad)
        aux = torch.empty(s, ws.heads * 384, dtype=BF16, device=x.device) if need_grad else None
        auxt = torch.empty(T, ws.heads * 384, dtype=BF16, device=x.device) if need_grad else None
        ws.heap.barrier()          # peers have finished reading q / k / v of the previous use
        _qkv_fused_launch(ws, x2, w, b, qw, kw, cosf, sinf, ws.video_off + ws.rank * s, s, False, aux)
        _qkv_fused_launch(ws, xt2, wt, bt, qwt, kwt, None, None, ws.text_off, 0, True, auxt)
        ws.heap.barrier()          # every rank's tiles have landed
        ctx.ws, ctx.eps = ws, eps
        ctx.save_for_backward(x2, xt2, aux, auxt, cosf, sinf, w, qw, kw, wt, qwt, kwt)
        ctx.has_bias = (b is not None, bt is not None)
        ctx.shapes = (x.shape, xt.shape)
        q, k, v = (ws.head_major(n) for n in ("q", "k", "v"))
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        ws: UlyssesWorkspace = ctx.ws
        x2, xt2, aux, auxt, cosf, sinf, w, qw, kw, wt, qwt, kwt = ctx.saved_tensors
        s, T = ws.s, ws.T
        pending = [(ws.head_major(name), g) for name, g in (("dq", dq), ("dk", dk), ("dv", dv))
                   if g.data_ptr() != ws.head_major(name).data_ptr()]
        if pending:
            # gradients that were not produced inside the workspace (every rank takes the same branch: it depends on
            # the producer op only)
            ws.heap.barrier()      # previous readers of the gradient buffers are done
            for dst, g in pending:
                dst.copy_(g)
        ws.heap.barrier()          # every rank's head-sharded gradients are in place
        outs = []
        for (xx, raw, ww, q_w, k_w, off, rl, scale, hb) in ((x2, aux, w, qw, kw, ws.video_off + ws.rank * s, s, 1.0, ctx.has_bias[0]),
                                                        (xt2, auxt, wt, qwt, kwt, ws.text_off, 0, 1.0 / ws.cp, ctx.has_bias[1])):
            rows = raw.shape[0]
            dqkv = torch.empty_like(raw)
            nw = _lib.lib().tt_qkv_partial_warps(c_long(rows), c_int(ws.heads))
            partials = torch.empty(nw * 256, dtype=torch.float32, device=raw.device)
            dqw = torch.empty(128, dtype=BF16, device=raw.device)
            dkw = torch.empty_like(dqw)
            call("tt_qkv_post_bwd_peer", ws.table("dq"), ws.table("dk"), ws.table("dv"), c_int(ws.cp), ptr(raw),
                 ptr(q_w.contiguous()), ptr(k_w.contiguous()), ptr(cosf if rl else None), ptr(sinf if rl else None),
                 ptr(dqkv), ptr(partials), ptr(dqw), ptr(dkw), c_long(rows), c_int(ws.heads), c_long(rows),
                 c_long(ws.S_tot), c_long(off), c_long(rl), c_float(ctx.eps), stream())
            if scale != 1.0:
                # replicated text tokens: every rank rebuilds the full gradient; the 1/cp keeps the DP x CP average exact
                dqkv.mul_(scale)
                dqw.mul_(scale)
                dkw.mul_(scale)
            dx = gemm.gemm_nn(dqkv, ww)
            dw = gemm.gemm_tn(dqkv, xx)
            db = dqkv.sum(dim=0, dtype=torch.float32).to(BF16) if hb else None
            outs.append((dx, dw, db, dqw, dkw))
        (dx, dw, db, dqw, dkw), (dxt, dwt, dbt, dqwt, dkwt) = outs
        xs, xts = ctx.shapes
        return (None, None, None, None, dx.view(xs), dw, db, dqw, dkw, dxt.view(xts), dwt, dbt, dqwt, dkwt)


def fused_qkv_a2a(ws: UlyssesWorkspace, x, w, b, qw, kw, cos, sin, xt, wt, bt, qwt, kwt, eps: float = 1e-6):
    """Video tokens ``x [1, s, H]`` (sequence-sharded, RoPE applied) and replicated text tokens ``xt [1, T, H]`` ->
    ``q, k, v [1, heads / cp, T + cp * s, 128]`` for this rank's heads over the whole sequence (text tokens first)."""
    return _FusedQKVAllToAll.apply(ws, eps, cos, sin, x, w, b, qw, kw, xt, wt, bt, qwt, kwt)


# ---------------------------------------------------------------------------------------------
# F2: head -> sequence all-to-all + output projection
# ---------------------------------------------------------------------------------------------

def _a2a_gemm(ws: UlyssesWorkspace, src_name: str, row_off: int, M: int, w, bias, extra=None):
    N, K = w.shape
    out = torch.empty(M, N, dtype=BF16, device=w.device)
    call("tt_gemm_comm_bf16", ws.table(src_name), c_int(ws.cp), c_int(1), c_long(ws.S_tot), c_int(ws.h_loc * 128),
         c_int(row_off), ptr(extra), c_long(0 if extra is None else extra.stride(0)), ptr(w), c_int(0), c_long(w.stride(0)),
         ptr(out), c_long(N), ptr(bias), c_int(M), c_int(N), c_int(K), c_int(0), c_int(ws.rank), c_int(0), None, c_int(0),
         c_int(0), c_long(0), None, None, c_int(0), ptr(status_tensor(w.device)), stream())
    return out


def _gather_heads(ws: UlyssesWorkspace, rows: int, row_off: int) -> torch.Tensor:
    """``[rows, cp * span]``: every rank's head columns of ``o`` for ``rows`` tokens starting at ``row_off`` (peer loads)."""
    span = ws.h_loc * 128
    a = torch.empty(rows, ws.cp * span, dtype=BF16, device=ws.heap.device)
    call("tt_gather_cols_bf16", ws.table("o"), c_int(ws.cp), c_long(rows), c_int(span), c_long(row_off), ptr(a), stream())
    return a


class _FusedAllToAllLinear(torch.autograd.Function):
    """``y_video = gather_heads(o)[rank's tokens] @ W^T + b`` and ``y_text = gather_heads(o)[text] @ Wt^T + bt`` with the
    gather fused into the GEMM operand fetch.  ``extra`` / ``extra_t`` are optional local tensors concatenated to
    the gathered heads along K (the MLP half of the single block's merged projection)."""

    @staticmethod
    def forward(ctx, ws, private, o, w, b, wt, bt, extra, extra_t):
        dst = ws.token_major("o")
        ws.heap.barrier()                      # peers are done with the previous contents of `o`
        if o.data_ptr() != dst.data_ptr():
            dst.copy_(o)
        ws.heap.barrier()
        ex = None if extra is None else check(extra.reshape(ws.s, -1).contiguous(), BF16, "extra")
        ext = None if extra_t is None else check(extra_t.reshape(ws.T, -1).contiguous(), BF16, "extra_t")
        y = _a2a_gemm(ws, "o", ws.video_off + ws.rank * ws.s, ws.s, w, b, ex)
        yt = _a2a_gemm(ws, "o", ws.text_off, ws.T, wt, bt, ext)
        ctx.ws = ws
        a = at = None
        if private and any(ctx.needs_input_grad):
            # the weight gradients need the gathered activations; `o` of the workspace will not survive the next layer
            COUNTERS["private_saves"] += 1
            a, at = _gather_heads(ws, ws.s, ws.video_off + ws.rank * ws.s), _gather_heads(ws, ws.T, ws.text_off)
        ctx.save_for_backward(w, wt, ex, ext, a, at)
        ctx.has = (b is not None, bt is not None, extra is not None, extra_t is not None)
        ctx.extra_shapes = (None if extra is None else extra.shape, None if extra_t is None else extra_t.shape)
        return y.view(1, ws.s, -1), yt.view(1, ws.T, -1)

    @staticmethod
    def backward(ctx, dy, dyt):
        ws: UlyssesWorkspace = ctx.ws
        w, wt, ex, ext, a, at = ctx.saved_tensors
        hb, hbt, hex_, hext = ctx.has
        span = ws.h_loc * 128
        G = ws.cp * span                                        # gathered K columns
        dy2 = check(dy.reshape(ws.s, -1).contiguous(), BF16, "dy")
        dyt2 = check(dyt.reshape(ws.T, -1).contiguous(), BF16, "dyt")
        dev = dy2.device
        if a is None:
            # weight gradients need the gathered activations: collect them with the peer-reading copy kernel
            a, at = _gather_heads(ws, ws.s, ws.video_off + ws.rank * ws.s), _gather_heads(ws, ws.T, ws.text_off)
        a_full = a if ex is None else torch.cat([a, ex], dim=1)
        at_full = at if ext is None else torch.cat([at, ext], dim=1)
        dw = gemm.gemm_tn(dy2, a_full)
        dwt = gemm.gemm_tn(dyt2, at_full)
        db = dy2.sum(0, dtype=torch.float32).to(BF16) if hb else None
        dbt = dyt2.sum(0, dtype=torch.float32).to(BF16) if hbt else None
        # data gradient: each head's columns go to the head's owner (sequence -> head all-to-all fused in the epilogue)
        K = w.shape[1]
        dex = torch.empty(ws.s, K - G, dtype=BF16, device=dev) if hex_ else None
        ws.heap.barrier()                      # peers are done reading the previous contents of `do`
        call("tt_gemm_comm_bf16", _table([dy2.data_ptr()]), c_int(ws.cp), c_int(0), c_long(ws.s), c_int(0), c_int(0), None,
             c_long(0), ptr(w), c_int(1), c_long(w.stride(0)), ptr(dex), c_long(0 if dex is None else dex.stride(0)), None,
             c_int(ws.s), c_int(K), c_int(w.shape[0]), c_int(0), c_int(ws.rank), c_int(1), ws.table("do"), c_int(span),
             c_int(ws.video_off + ws.rank * ws.s), c_long(span), None, None, c_int(0), ptr(status_tensor(dev)), stream())
        # text rows: every rank holds the full gradient; keep this rank's heads, scaled by cp (the gather's "up" rule)
        dot_full = gemm.gemm_nn(dyt2, wt)
        do_local = ws.token_major("do")
        do_local[0, ws.text_off:ws.text_off + ws.T, :].copy_(dot_full[:, ws.rank * span:(ws.rank + 1) * span] * float(ws.cp))
        dext = dot_full[:, G:].contiguous().view(ctx.extra_shapes[1]) if hext else None
        ws.heap.barrier()                      # all pushed gradient tiles have landed
        return (None, None, do_local, dw, db, dwt, dbt, None if dex is None else dex.view(ctx.extra_shapes[0]), dext)


def fused_a2a_linear(ws: UlyssesWorkspace, o, w, b, wt, bt, extra=None, extra_t=None):
    """``o [1, S_tot, heads/cp * 128]`` (this rank's heads, all tokens) -> projections of this rank's video tokens
    (weights ``w``) and of the replicated text tokens (weights ``wt``)."""
    return _FusedAllToAllLinear.apply(ws, saves_need_private_copies(), o, w, b, wt, bt, extra, extra_t)


# ---------------------------------------------------------------------------------------------
# F2 (push form): attention whose epilogue performs the head -> sequence all-to-all, then local projections
# ---------------------------------------------------------------------------------------------

def _local_gemm_extra(ws: UlyssesWorkspace, a_rows: torch.Tensor, extra, w, bias):
    """``[a_rows | extra] @ w^T + bias`` without materialising the concatenation (the K loop switches source)."""
    M, G = a_rows.shape
    N, K = w.shape
    if extra is None:
        return gemm.gemm_nt(a_rows, w, bias)
    out = torch.empty(M, N, dtype=BF16, device=w.device)
    call("tt_gemm_comm_bf16", _table([a_rows.data_ptr()]), c_int(1), c_int(1), c_long(M), c_int(G), c_int(0), ptr(extra),
         c_long(extra.stride(0)), ptr(w), c_int(0), c_long(w.stride(0)), ptr(out), c_long(N), ptr(bias), c_int(M), c_int(N),
         c_int(K), c_int(0), c_int(0), c_int(0), None, c_int(0), c_int(0), c_long(0), None, None, c_int(0),
         ptr(status_tensor(w.device)), stream())
    return out


class _FusedAttentionOutProj(torch.autograd.Function):
    """Attention over this rank's heads with the head -> sequence all-to-all done by the attention epilogue (every
    output row is stored straight into the gathered buffer of the rank that owns the token, crossing NVLink once),
    followed by the local output projections of the video and the text stream."""

    @staticmethod
    def forward(ctx, ws, kv_len, mask_range, scale, private, q, k, v, w, b, wt, bt, extra, extra_t):
        from . import attn_tcgen05 as A
        import math
        H_all = ws.heads
        T, s = ws.T, ws.s
        sc = (1.0 / math.sqrt(128)) if scale is None else float(scale)
        kvl = ws.S_tot if kv_len is None else int(kv_len)
        mlo, mhi = (0, 0) if mask_range is None else (int(mask_range[0]), int(mask_range[1]))
        q, k, v = (check(t.contiguous(), BF16, n) for t, n in ((q, "q"), (k, "k"), (v, "v")))
        g = ws.heap.tensor(ws.off["g"], (T + s, H_all * 128), BF16)
        ws.heap.barrier()                  # peers are done with the previous gathered buffer / o
        cached = A._CACHE.pop(0) if (A._CACHE_MODE == "replay" and A._CACHE) else None
        if cached is None:
            out = torch.empty(1, ws.S_tot, ws.h_loc * 128, dtype=BF16, device=q.device)
            pitch = (ws.S_tot + 63) // 64 * 64
            lse = torch.full((1, ws.h_loc, pitch), float("inf"), dtype=torch.float32, device=q.device)
            call("tt_attn_fwd_push", ptr(q), ptr(k), ptr(v), ptr(out), ptr(lse), c_int(ws.h_loc), c_int(ws.S_tot), c_int(kvl),
                 c_int(mlo), c_int(mhi), c_int(pitch), c_float(sc), ptr(status_tensor(q.device)), stream(), ws.table("g"), c_int(ws.cp),
                 c_int(ws.rank), c_int(T), c_int(s), c_long(H_all * 128))
            if A._CACHE_MODE == "record":
                A._CACHE.append((out, lse))
            ws.heap.barrier()              # every rank's rows have landed
        else:
            # recompute pass with the attention output kept: redo only the all-to-all (peer-reading copy)
            out, lse = cached
            ws.token_major("o").copy_(out)
            ws.heap.barrier()
            span = ws.h_loc * 128
            call("tt_gather_cols_bf16", ws.table("o"), c_int(ws.cp), c_long(T), c_int(span), c_long(ws.text_off), ptr(g[:T]), stream())
            call("tt_gather_cols_bf16", ws.table("o"), c_int(ws.cp), c_long(s), c_int(span), c_long(ws.video_off + ws.rank * s),
                 ptr(g[T:]), stream())
        ex = None if extra is None else check(extra.reshape(s, -1).contiguous(), BF16, "extra")
        ext = None if extra_t is None else check(extra_t.reshape(T, -1).contiguous(), BF16, "extra_t")
        y = _local_gemm_extra(ws, g[T:], ex, w, b)
        yt = _local_gemm_extra(ws, g[:T], ext, wt, bt)
        ctx.ws, ctx.sc, ctx.kvl, ctx.mask = ws, sc, kvl, (mlo, mhi)
        if private and any(ctx.needs_input_grad):
            # q / k / v and g live in the workspace every layer shares: keep copies that the next layer cannot overwrite
            COUNTERS["private_saves"] += 1
            q, k, v, g = q.clone(), k.clone(), v.clone(), g.clone()
        ctx.save_for_backward(q, k, v, out, lse, w, wt, ex, ext, g)
        ctx.has = (b is not None, bt is not None)
        ctx.extra_shapes = (None if extra is None else extra.shape, None if extra_t is None else extra_t.shape)
        return y.view(1, s, -1), yt.view(1, T, -1)

    @staticmethod
    def backward(ctx, dy, dyt):
        from . import attn_backward
        ws: UlyssesWorkspace = ctx.ws
        q, k, v, out, lse, w, wt, ex, ext, g = ctx.saved_tensors
        T, s = ws.T, ws.s
        span = ws.h_loc * 128
        G = ws.cp * span
        K = w.shape[1]
        dev = q.device
        dy2 = check(dy.reshape(s, -1).contiguous(), BF16, "dy")
        dyt2 = check(dyt.reshape(T, -1).contiguous(), BF16, "dyt")
        # weight gradients: the gathered activations are local
        dw = torch.empty_like(w)
        gemm.gemm_tn_into(dy2, g[T:], dw[:, :G])
        dwt_same = wt.data_ptr() == w.data_ptr()
        dwt = torch.empty_like(wt)
        gemm.gemm_tn_into(dyt2, g[:T], dwt[:, :G])
        if ex is not None:
            gemm.gemm_tn_into(dy2, ex, dw[:, G:])
        if ext is not None:
            gemm.gemm_tn_into(dyt2, ext, dwt[:, G:])
        db = dy2.sum(0, dtype=torch.float32).to(BF16) if ctx.has[0] else None
        dbt = dyt2.sum(0, dtype=torch.float32).to(BF16) if ctx.has[1] else None
        # data gradient of the video rows: every head's columns are pushed to the head's owner by the GEMM epilogue
        dex = torch.empty(s, K - G, dtype=BF16, device=dev) if ex is not None else None
        ws.heap.barrier()                  # peers are done reading the previous contents of `do`
        call("tt_gemm_comm_bf16", _table([dy2.data_ptr()]), c_int(ws.cp), c_int(0), c_long(s), c_int(0), c_int(0), None,
             c_long(0), ptr(w), c_int(1), c_long(w.stride(0)), ptr(dex), c_long(0 if dex is None else dex.stride(0)), None,
             c_int(s), c_int(K), c_int(w.shape[0]), c_int(0), c_int(ws.rank), c_int(1), ws.table("do"), c_int(span),
             c_int(ws.video_off + ws.rank * s), c_long(span), None, None, c_int(0), ptr(status_tensor(dev)), stream())
        # text rows are replicated: keep this rank's heads, scaled by cp
        dot_full = gemm.gemm_nn(dyt2, wt)
        do_local = ws.token_major("do")
        do_local[0, ws.text_off:ws.text_off + T, :].copy_(dot_full[:, ws.rank * span:(ws.rank + 1) * span] * float(ws.cp))
        dext = dot_full[:, G:].contiguous().view(ctx.extra_shapes[1]) if ext is not None else None
        ws.heap.barrier()                  # all pushed gradient tiles have landed
        # dq / dk / dv are written straight into the workspace regions that the peers read in the QKV backward.  Their
        # last readers (the peers' QKV backward of the layer above) finished before the two barriers of this function.
        dq, dk, dv = attn_backward.backward(do_local, q, k, v, out, lse, ctx.sc, ctx.kvl,
                                            outs=tuple(ws.head_major(n) for n in ("dq", "dk", "dv")), mask_range=ctx.mask)
        del dwt_same
        return (None, None, None, None, None, dq, dk, dv, dw, db, dwt, dbt, None if dex is None else dex.view(ctx.extra_shapes[0]), dext)


def fused_attention_outproj(ws: UlyssesWorkspace, q, k, v, w, b, wt, bt, extra=None, extra_t=None, kv_len=None, scale=None,
                            mask_range=None):
    """``q, k, v [1, heads/cp, T + cp*s, 128]`` -> (projection of this rank's video tokens with ``w``, projection of the
    text tokens with ``wt``); ``extra`` / ``extra_t`` are local tensors concatenated to the attention output along K.
    Keys at and beyond ``kv_len`` (context-parallel padding, the sequence tail) and keys in ``mask_range`` (padded text
    tokens, which come first in this layout) are masked."""
    return _FusedAttentionOutProj.apply(ws, kv_len, mask_range, scale, saves_need_private_copies(), q, k, v, w, b, wt, bt,
                                        extra, extra_t)


# ---------------------------------------------------------------------------------------------
# F3: tensor-parallel all-gather -> GEMM and GEMM -> reduce-scatter
# ---------------------------------------------------------------------------------------------

class TPWorkspace:
    """Symmetric staging for sequence-sharded tensor parallelism: a gather source and a reduce-scatter landing zone, sized
    for ``rows_local`` rows (or more, ``capacity_rows``) and laid out per call of :meth:`configure`."""

    def __init__(self, group, rows_local: int, k_max: int, n_max: int, device=None, capacity_rows: Optional[int] = None):
        self.group = group
        self.tp = 1 if group is None else dist.get_world_size(group)
        self.rank = 0 if group is None else dist.get_rank(group)
        self.k_max, self.n_max = k_max, n_max
        self.capacity_rows = max(rows_local, capacity_rows or 0)
        a_bytes = self.capacity_rows * k_max * 2
        s_bytes = self.tp * self.capacity_rows * n_max * 2
        self.heap = SymmetricHeap(group, a_bytes + s_bytes + 4096, device)
        dev = self.heap.device
        self.stage = torch.empty(self.tp * self.capacity_rows * k_max, dtype=BF16, device=dev)
        self.flags = torch.zeros(self.tp * ((self.capacity_rows + 127) // 128), dtype=torch.int32, device=dev)
        self.epoch = 0
        self.configure(rows_local)

    def fits(self, rows_local: int) -> bool:
        return rows_local <= self.capacity_rows

    def configure(self, rows_local: int) -> None:
        if not self.fits(rows_local):
            raise MemoryError("row count does not fit the workspace it was sized for")
        self.rows = rows_local
        self.heap.reset()
        self.off_a = self.heap.alloc(rows_local * self.k_max * 2)
        self.off_s = self.heap.alloc(self.tp * rows_local * self.n_max * 2)


def fused_all_gather_linear(ws: TPWorkspace, x_local: torch.Tensor, w: torch.Tensor, bias=None, staged: bool = True) -> torch.Tensor:
    """``all_gather(x_local over rows) @ w^T + bias``: every rank's row block is TMA-loaded from its owner while the
    tensor core works; this rank's own rows are scheduled first.  ``x_local [rows, K]``, ``w [N, K]`` (column-parallel shard)."""
    rows, K = x_local.shape
    if rows != ws.rows or K > ws.k_max:
        raise _lib.NativeError("operand does not match the workspace")
    src = ws.heap.tensor(ws.off_a, (rows, K), BF16)
    ws.heap.barrier()
    src.copy_(x_local)
    ws.heap.barrier()
    N = w.shape[0]
    M = rows * ws.tp
    out = torch.empty(M, N, dtype=BF16, device=w.device)
    # remote row blocks are copied once into this local staging buffer by the kernel's copier warps
    stage = ws.stage[: M * K].view(M, K) if staged else None
    ws.epoch += 1
    call("tt_gemm_comm_bf16", ws.heap.ptr_table(ws.off_a), c_int(ws.tp), c_int(2), c_long(rows), c_int(0), c_int(0), None,
         c_long(0), ptr(w), c_int(0), c_long(w.stride(0)), ptr(out), c_long(N), ptr(bias), c_int(M), c_int(N), c_int(K),
         c_int(rows), c_int(ws.rank), c_int(0), None, c_int(0), c_int(0), c_long(0), ptr(stage), ptr(ws.flags), c_int(ws.epoch),
         ptr(status_tensor(w.device)), stream())
    return out


def fused_linear_reduce_scatter(ws: TPWorkspace, x: torch.Tensor, w: torch.Tensor, bias=None, residual=None, gate=None) -> torch.Tensor:
    """``reduce_scatter(x @ w^T over rows) + bias`` (optionally ``residual + gate * (...)``): every rank multiplies its K
    shard for all rows and pushes each row block's partial tile to the block's owner from the GEMM epilogue; the
    owner then sums the ``tp`` partials.  ``x [tp * rows, K_shard]``, ``w [N, K_shard]``; returns ``[rows, N]``."""
    M, K = x.shape
    N = w.shape[0]
    if M != ws.rows * ws.tp or N > ws.n_max:
        raise _lib.NativeError("operand does not match the workspace")
    ws.heap.barrier()              # previous partials have been consumed everywhere
    call("tt_gemm_comm_bf16", _table([x.data_ptr()]), c_int(ws.tp), c_int(0), c_long(M), c_int(0), c_int(0), None, c_long(0),
         ptr(w), c_int(0), c_long(w.stride(0)), None, c_long(0), None, c_int(M), c_int(N), c_int(K), c_int(ws.rows),
         c_int(ws.rank), c_int(2), ws.heap.ptr_table(ws.off_s), c_int(0), c_int(0), c_long(N), None, None, c_int(0),
         ptr(status_tensor(x.device)), stream())
    ws.heap.barrier()              # all partials have landed
    out = torch.empty(ws.rows, N, dtype=BF16, device=x.device)
    stage = ws.heap.tensor(ws.off_s, (ws.tp, ws.rows, N), BF16)
    call("tt_partial_sum", ptr(stage), c_int(ws.tp), c_long(ws.rows), c_int(N), ptr(bias), ptr(residual), ptr(gate),
         c_long(ws.rows), ptr(out), stream())
    return out


# ---- sequence-parallel linears with autograd (the model's MLPs under --sequence-parallel --fused-comm) ----------

_GELU_KIND = {"gelu": 0, "gelu_tanh": 1}


def _ag_gemm(ws: TPWorkspace, x_local: torch.Tensor, w: torch.Tensor, bias, b_mn: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gather(x_local) @ op(w) (+ bias)`` and the gathered operand itself (kept by callers for the weight gradient).
    ``b_mn = 0``: ``w`` is ``[N, K]``; ``b_mn = 1``: ``w`` is ``[K, N]``."""
    rows, K = x_local.shape
    if rows != ws.rows or K > ws.k_max:
        raise _lib.NativeError("operand does not match the workspace")
    src = ws.heap.tensor(ws.off_a, (rows, K), BF16)
    ws.heap.barrier()                       # every rank has finished reading the previous gather source
    src.copy_(x_local)
    ws.heap.barrier()
    N = w.shape[1] if b_mn else w.shape[0]
    M = rows * ws.tp
    out = torch.empty(M, N, dtype=BF16, device=w.device)
    xg = torch.empty(M, K, dtype=BF16, device=w.device)
    ws.epoch += 1
    call("tt_gemm_ag_bf16", ws.heap.ptr_table(ws.off_a), c_int(ws.tp), c_int(ws.rank), c_int(rows), ptr(w), c_int(b_mn),
         c_long(w.stride(0)), ptr(out), c_long(N), ptr(bias), None, c_int(N), c_int(K), c_int(0), ptr(xg), ptr(ws.flags),
         c_int(ws.epoch), ptr(status_tensor(w.device)), stream())
    # the kernel stages only the remote row blocks; this rank's own block completes the gathered operand
    xg[ws.rank * rows:(ws.rank + 1) * rows].copy_(x_local)
    return out, xg


def _gemm_rs(ws: TPWorkspace, x: torch.Tensor, w: torch.Tensor, b_mn: int, bias=None) -> torch.Tensor:
    """``reduce_scatter(x @ op(w)) (+ bias)`` over row blocks: partial tiles are pushed to the block's owner from the
    GEMM epilogue, then the owner sums the ``tp`` partials."""
    M, K = x.shape
    N = w.shape[1] if b_mn else w.shape[0]
    if M != ws.rows * ws.tp or N > ws.n_max:
        raise _lib.NativeError("operand does not match the workspace")
    ws.heap.barrier()                       # previous partials have been consumed everywhere
    call("tt_gemm_comm_bf16", _table([x.data_ptr()]), c_int(ws.tp), c_int(0), c_long(M), c_int(0), c_int(0), None, c_long(0),
         ptr(w), c_int(b_mn), c_long(w.stride(0)), None, c_long(0), None, c_int(M), c_int(N), c_int(K), c_int(ws.rows),
         c_int(ws.rank), c_int(2), ws.heap.ptr_table(ws.off_s), c_int(0), c_int(0), c_long(N), None, None, c_int(0),
         ptr(status_tensor(x.device)), stream())
    ws.heap.barrier()                       # all partials have landed
    out = torch.empty(ws.rows, N, dtype=BF16, device=x.device)
    stage = ws.heap.tensor(ws.off_s, (ws.tp, ws.rows, N), BF16)
    call("tt_partial_sum", ptr(stage), c_int(ws.tp), c_long(ws.rows), c_int(N), ptr(bias), None, None, c_long(ws.rows),
         ptr(out), stream())
    return out


class _SPColumnLinear(torch.autograd.Function):
    """Column-parallel linear on a token-sharded input: all-gather -> GEMM forward; the data gradient is a
    GEMM -> reduce-scatter, the weight gradient uses the gathered operand kept from the forward."""

    @staticmethod
    def forward(ctx, ws, x, w, bias, activation):
        u, xg = _ag_gemm(ws, check(x.contiguous(), BF16, "x"), w, bias, 0)
        ctx.ws, ctx.activation, ctx.has_bias = ws, activation, bias is not None
        if activation is None:
            ctx.save_for_backward(xg, w)
            return u
        y = torch.empty_like(u)
        call("tt_gelu_fwd", ptr(u), ptr(y), c_long(u.numel()), c_int(_GELU_KIND[activation]), stream())
        ctx.save_for_backward(xg, w, u)
        return y

    @staticmethod
    def backward(ctx, dy):
        dy = check(dy.contiguous(), BF16, "dy")
        if ctx.activation is None:
            xg, w = ctx.saved_tensors
            du = dy
        else:
            xg, w, u = ctx.saved_tensors
            du = torch.empty_like(u)
            call("tt_gelu_bwd", ptr(dy), ptr(u), ptr(du), c_long(u.numel()), c_int(_GELU_KIND[ctx.activation]), stream())
        dx = _gemm_rs(ctx.ws, du, w, 1) if ctx.needs_input_grad[1] else None
        dw = gemm.gemm_tn(du, xg) if ctx.needs_input_grad[2] else None
        db = du.sum(dim=0, dtype=torch.float32).to(BF16) if (ctx.has_bias and ctx.needs_input_grad[3]) else None
        return None, dx, dw, db, None


class _SPRowLinear(torch.autograd.Function):
    """Row-parallel linear producing a token-sharded output: GEMM -> reduce-scatter forward (bias added once, by the
    owner of each row block); the data gradient is an all-gather -> GEMM and its gathered operand feeds the weight
    gradient.  The bias gradient is this rank's row block's share (summed over TP with the other partial gradients)."""

    @staticmethod
    def forward(ctx, ws, x, w, bias):
        x = check(x.contiguous(), BF16, "x")
        ctx.ws, ctx.has_bias = ws, bias is not None
        ctx.save_for_backward(x, w)
        return _gemm_rs(ws, x, w, 0, bias)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = check(dy.contiguous(), BF16, "dy")
        dx, dyg = _ag_gemm(ctx.ws, dy, w, None, 1)
        dw = gemm.gemm_tn(dyg, x) if ctx.needs_input_grad[2] else None
        db = dy.sum(dim=0, dtype=torch.float32).to(BF16) if (ctx.has_bias and ctx.needs_input_grad[3]) else None
        return None, dx, dw, db


def sp_column_linear(ws: TPWorkspace, x: torch.Tensor, w: torch.Tensor, bias=None, activation: Optional[str] = None) -> torch.Tensor:
    """``act(all_gather(x) @ w^T + bias)`` for ``x [rows, K]`` token-sharded over the tensor-parallel group."""
    return _SPColumnLinear.apply(ws, x, w, bias, activation)


def sp_row_linear(ws: TPWorkspace, x: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
    """``reduce_scatter(x @ w^T) + bias`` for ``x [tp * rows, K / tp]``; returns this rank's ``[rows, N]`` block."""
    return _SPRowLinear.apply(ws, x, w, bias)


# ---------------------------------------------------------------------------------------------
# F4: data-parallel gradient reduce-scatter (+ scale) and parameter all-gather over peer memory
# ---------------------------------------------------------------------------------------------

def fused_grad_reduce_scatter(heap: SymmetricHeap, grad_off: int, start: int, count: int, out: torch.Tensor, scale: float) -> None:
    """``out[:] = scale * sum_r grad_r[start : start + count]`` reading every rank's bf16 gradient buffer (which lives
    in the heap at ``grad_off``) with peer loads.  The caller brackets it with ``heap.barrier()``."""
    call("tt_reduce_scatter_bf16", heap.ptr_table(grad_off), c_int(heap.world), c_long(start), ptr(out), c_long(count),
         c_float(scale), stream())


def fused_param_all_gather(heap: SymmetricHeap, param_off: int, start: int, src: torch.Tensor) -> None:
    """Write this rank's updated parameter shard into every rank's parameter buffer at ``start``."""
    call("tt_all_gather_push_bf16", heap.ptr_table(param_off), c_int(heap.world), c_long(start), ptr(src),
         c_long(src.numel()), stream())


def fused_reduce_adamw_all_gather(heap: SymmetricHeap, grad_off: int, param_off: int, start: int, count: int,
                                  exp_avg: torch.Tensor, exp_avg_sq: torch.Tensor, master: Optional[torch.Tensor],
                                  master_lo: Optional[torch.Tensor], *, lr: float, beta1: float, beta2: float, eps: float,
                                  weight_decay: float, step: int, grad_scale: float, grads_reduced: bool = False) -> None:
    """One kernel for ``[start, start + count)`` of the flat buffers that live in ``heap``: sum every rank's bf16
    gradients (peer loads) times ``grad_scale``, AdamW on this rank's moments / master weights, and store the new bf16
    weights into every rank's parameter buffer (peer stores).  ``grads_reduced``: the local gradient buffer already
    holds the reduced shard (overlapped reduce-scatter), so only it is read.  The caller brackets the optimizer step
    with ``heap.barrier()``: gradients complete everywhere before, all loads and stores done after."""
    state_bf16 = exp_avg.dtype == BF16
    gt = _table([heap.local_ptr + grad_off]) if grads_reduced else heap.ptr_table(grad_off)
    call("tt_rs_adamw_ag", gt, c_int(1 if grads_reduced else heap.world), heap.ptr_table(param_off), c_int(heap.world),
         c_int(heap.rank), c_long(start), ptr(exp_avg), ptr(exp_avg_sq), ptr(master), ptr(master_lo), c_long(count),
         c_int(1 if state_bf16 else 0), c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(weight_decay),
         c_int(step), c_float(grad_scale), stream())
