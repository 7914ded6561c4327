"""``autograd.Function`` wrappers around the sm_100a kernels in ``libteletron_b200.so``.

Each function mirrors one entry of :mod:`teletron_b200.ops.reference` (same signature, same maths)
and is what :mod:`teletron_b200.ops` dispatches to for CUDA bf16 tensors.  Scratch buffers for the
column reductions are allocated here with ``torch.empty`` and handed to the C side.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib
from ._lib import c_float, c_int, c_long, call, check, ptr, stream

BF16 = torch.bfloat16
_GELU_KIND = {"gelu": 0, "gelu_tanh": 1}
# TELETRON_B200_GELU_EPILOGUE=0 keeps the activation in its own kernel after the GEMM
_FUSE_GELU_EPILOGUE = os.environ.get("TELETRON_B200_GELU_EPILOGUE", "1") != "0"


def _rows_cols(x: torch.Tensor):
    cols = x.shape[-1]
    return x.numel() // cols, cols


def _mod_vec(t: torch.Tensor, batch: int, cols: int, name: str) -> torch.Tensor:
    t = t.reshape(batch, cols)
    if t.dtype != BF16:
        t = t.to(BF16)
    return check(t.contiguous(), BF16, name)


# ---------------------------------------------------------------------------------------------
# LayerNorm + modulation (+ gated residual)
# ---------------------------------------------------------------------------------------------

class _LayerNormModulate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, shift, eps):
        B = x.shape[0]
        rows, cols = _rows_cols(x)
        xc = check(x.contiguous(), BF16, "x")
        sc, sh = _mod_vec(scale, B, cols, "scale"), _mod_vec(shift, B, cols, "shift")
        y = torch.empty_like(xc)
        mean = torch.empty(rows, dtype=torch.float32, device=x.device)
        rstd = torch.empty_like(mean)
        call("tt_ln_mod_fwd", ptr(xc), ptr(None), ptr(None), ptr(sc), ptr(sh), ptr(None), ptr(y), ptr(mean), ptr(rstd),
             c_long(rows), c_int(cols), c_long(rows // B), c_float(eps), stream())
        ctx.save_for_backward(xc, sc, mean, rstd)
        ctx.scale_shape, ctx.shift_shape = scale.shape, shift.shape
        ctx.dtypes = (scale.dtype, shift.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, sc, mean, rstd = ctx.saved_tensors
        B = xc.shape[0]
        rows, cols = _rows_cols(xc)
        dy = check(dy.contiguous(), BF16, "dy")
        dx = torch.empty_like(xc)
        nblk = _lib.lib().tt_norm_partial_blocks(c_long(rows // B), c_int(B))
        partials = torch.empty(B * nblk * 2 * cols, dtype=torch.float32, device=xc.device)
        dscale = torch.empty(B, cols, dtype=BF16, device=xc.device)
        dshift = torch.empty_like(dscale)
        call("tt_ln_mod_bwd", ptr(dy), ptr(None), ptr(xc), ptr(None), ptr(None), ptr(sc), ptr(mean), ptr(rstd), ptr(dx),
             ptr(None), ptr(partials), ptr(dscale), ptr(dshift), ptr(None), c_long(rows), c_int(cols), c_long(rows // B),
             stream())
        return dx, dscale.view(ctx.scale_shape).to(ctx.dtypes[0]), dshift.view(ctx.shift_shape).to(ctx.dtypes[1]), None


def layernorm_modulate(x, scale, shift, eps=1e-6):
    return _LayerNormModulate.apply(x, scale, shift, eps)


class _GateResidualLayerNormModulate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, res, branch, gate, scale, shift, eps):
        B = res.shape[0]
        rows, cols = _rows_cols(res)
        rc = check(res.contiguous(), BF16, "residual")
        bc = check(branch.contiguous(), BF16, "branch")
        g, sc, sh = (_mod_vec(t, B, cols, n) for t, n in ((gate, "gate"), (scale, "scale"), (shift, "shift")))
        new_res = torch.empty_like(rc)
        y = torch.empty_like(rc)
        mean = torch.empty(rows, dtype=torch.float32, device=res.device)
        rstd = torch.empty_like(mean)
        call("tt_ln_mod_fwd", ptr(rc), ptr(bc), ptr(g), ptr(sc), ptr(sh), ptr(new_res), ptr(y), ptr(mean), ptr(rstd),
             c_long(rows), c_int(cols), c_long(rows // B), c_float(eps), stream())
        ctx.save_for_backward(new_res, bc, g, sc, mean, rstd)
        ctx.shapes = (gate.shape, scale.shape, shift.shape)
        return new_res, y

    @staticmethod
    def backward(ctx, dres_out, dy):
        new_res, bc, g, sc, mean, rstd = ctx.saved_tensors
        B = new_res.shape[0]
        rows, cols = _rows_cols(new_res)
        dev = new_res.device
        if dy is None:
            dy = torch.zeros_like(new_res)
        dy = check(dy.contiguous(), BF16, "dy")
        dres_in = None if dres_out is None else check(dres_out.contiguous(), BF16, "dres")
        dx = torch.empty_like(new_res)
        dbranch = torch.empty_like(new_res)
        nblk = _lib.lib().tt_norm_partial_blocks(c_long(rows // B), c_int(B))
        partials = torch.empty(B * nblk * 3 * cols, dtype=torch.float32, device=dev)
        dscale = torch.empty(B, cols, dtype=BF16, device=dev)
        dshift, dgate = torch.empty_like(dscale), torch.empty_like(dscale)
        call("tt_ln_mod_bwd", ptr(dy), ptr(dres_in), ptr(new_res), ptr(bc), ptr(g), ptr(sc), ptr(mean), ptr(rstd), ptr(dx),
             ptr(dbranch), ptr(partials), ptr(dscale), ptr(dshift), ptr(dgate), c_long(rows), c_int(cols),
             c_long(rows // B), stream())
        gs, ss, hs = ctx.shapes
        return dx, dbranch, dgate.view(gs), dscale.view(ss), dshift.view(hs), None


def gate_residual_layernorm_modulate(res, branch, gate, scale, shift, eps=1e-6):
    return _GateResidualLayerNormModulate.apply(res, branch, gate, scale, shift, eps)


class _GateResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, res, branch, gate):
        B = res.shape[0]
        rows, cols = _rows_cols(res)
        rc = check(res.contiguous(), BF16, "residual")
        bc = check(branch.contiguous(), BF16, "branch")
        g = _mod_vec(gate, B, cols, "gate")
        out = torch.empty_like(rc)
        call("tt_gate_residual_fwd", ptr(rc), ptr(bc), ptr(g), ptr(out), c_long(rows), c_int(cols), c_long(rows // B),
             stream())
        ctx.save_for_backward(bc, g)
        ctx.gate_shape = gate.shape
        return out

    @staticmethod
    def backward(ctx, dout):
        bc, g = ctx.saved_tensors
        B = bc.shape[0]
        rows, cols = _rows_cols(bc)
        dout = check(dout.contiguous(), BF16, "dout")
        dbranch = torch.empty_like(bc)
        nblk = _lib.lib().tt_norm_partial_blocks(c_long(rows // B), c_int(B))
        partials = torch.empty(B * nblk * cols, dtype=torch.float32, device=bc.device)
        dgate = torch.empty(B, cols, dtype=BF16, device=bc.device)
        call("tt_gate_residual_bwd", ptr(dout), ptr(bc), ptr(g), ptr(dbranch), ptr(partials), ptr(dgate), c_long(rows),
             c_int(cols), c_long(rows // B), stream())
        return dout, dbranch, dgate.view(ctx.gate_shape)


def gate_residual(res, branch, gate):
    return _GateResidual.apply(res, branch, gate)


# ---------------------------------------------------------------------------------------------
# RMSNorm
# ---------------------------------------------------------------------------------------------

class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        rows, cols = _rows_cols(x)
        xc = check(x.contiguous(), BF16, "x")
        w = check(weight.contiguous(), BF16, "weight")
        y = torch.empty_like(xc)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        call("tt_rmsnorm_fwd", ptr(xc), ptr(w), ptr(y), ptr(rstd), c_long(rows), c_int(cols), c_float(eps), stream())
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, w, rstd = ctx.saved_tensors
        rows, cols = _rows_cols(xc)
        dy = check(dy.contiguous(), BF16, "dy")
        dx = torch.empty_like(xc)
        nblk = _lib.lib().tt_norm_partial_blocks(c_long(rows), c_int(1))
        partials = torch.empty(nblk * cols, dtype=torch.float32, device=xc.device)
        dw = torch.empty(cols, dtype=BF16, device=xc.device)
        call("tt_rmsnorm_bwd", ptr(dy), ptr(xc), ptr(w), ptr(rstd), ptr(dx), ptr(partials), ptr(dw), c_long(rows),
             c_int(cols), stream())
        return dx, dw, None


def rmsnorm(x, weight, eps=1e-6):
    return _RMSNorm.apply(x, weight, eps)


# ---------------------------------------------------------------------------------------------
# GEMMs
# ---------------------------------------------------------------------------------------------

def _gemm_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``a [M, K] @ b [N, K]^T (+ bias)``."""
    from . import gemm
    return gemm.gemm_nt(a, b, bias)


def _gemm_nn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a [M, K] @ b [K, N]``."""
    from . import gemm
    return gemm.gemm_nn(a, b)


def _gemm_tn(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a [K, M]^T @ b [K, N]`` (weight gradients)."""
    from . import gemm
    return gemm.gemm_tn(a, b)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, activation):
        K = x.shape[-1]
        x2 = x.reshape(-1, K)
        ctx.activation = activation
        ctx.has_bias = bias is not None
        if activation is not None and _FUSE_GELU_EPILOGUE:
            # bias + GELU in the GEMM epilogue: the accumulator is activated in fp32 and the kernel writes both the
            # activated output and the bf16 pre-activation that the backward needs
            from . import gemm, gemm_tcgen05
            if gemm.get_backend() != "cublas" and gemm_tcgen05.supported(x2, weight, "nt"):
                gemm.COUNTERS["tcgen05"] += 1
                y, u = gemm_tcgen05.gemm(x2, weight, "nt", bias, epi=1 + _GELU_KIND[activation])
                ctx.save_for_backward(x2, weight, u)
                return y.view(*x.shape[:-1], weight.shape[0])
        u = _gemm_nt(x2, weight, bias)
        if activation is None:
            ctx.save_for_backward(x2, weight)
            return u.view(*x.shape[:-1], weight.shape[0])
        y = torch.empty_like(u)
        call("tt_gelu_fwd", ptr(u), ptr(y), c_long(u.numel()), c_int(_GELU_KIND[activation]), stream())
        ctx.save_for_backward(x2, weight, u)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        if ctx.activation is None:
            x2, weight = ctx.saved_tensors
            du = dy.reshape(-1, weight.shape[0])
            if not du.is_contiguous():
                du = du.contiguous()
        else:
            x2, weight, u = ctx.saved_tensors
            dyc = check(dy.reshape(-1, weight.shape[0]).contiguous(), BF16, "dy")
            du = torch.empty_like(u)
            call("tt_gelu_bwd", ptr(dyc), ptr(u), ptr(du), c_long(u.numel()), c_int(_GELU_KIND[ctx.activation]), stream())
        dx = _gemm_nn(du, weight) if ctx.needs_input_grad[0] else None
        dw = _gemm_tn(du, x2) if ctx.needs_input_grad[1] else None
        db = du.sum(dim=0, dtype=torch.float32).to(du.dtype) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        if dx is not None:
            dx = dx.view(*dy.shape[:-1], weight.shape[1])
        return dx, dw, db, None


class _LinearMerged(torch.autograd.Function):
    """``y = cat([x1, x2], -1) @ weight^T + bias`` for the single-stream block's merged projection (attention output and
    MLP activation side by side).  The forward concatenates once and runs one GEMM; the backward never forms the
    concatenated gradient: each input's gradient comes from its own GEMM against a column slice of the weight (a strided
    B operand), and each half of the weight gradient is written into its column slice of ``dW``, so no strided slice
    of a ``[tokens, k1 + k2]`` gradient has to be copied to make it contiguous."""

    @staticmethod
    def forward(ctx, x1, x2, weight, bias):
        k1, k2 = x1.shape[-1], x2.shape[-1]
        a1, a2 = x1.reshape(-1, k1), x2.reshape(-1, k2)
        y = _gemm_nt(torch.cat([a1, a2], dim=1), weight, bias)
        ctx.save_for_backward(a1, a2, weight)
        ctx.has_bias = bias is not None
        ctx.lead = x1.shape[:-1]
        return y.view(*x1.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import gemm
        a1, a2, weight = ctx.saved_tensors
        k1 = a1.shape[1]
        du = dy.reshape(-1, weight.shape[0])
        if not du.is_contiguous():
            du = du.contiguous()
        d1 = _gemm_nn(du, weight[:, :k1]).view(*ctx.lead, k1) if ctx.needs_input_grad[0] else None
        d2 = _gemm_nn(du, weight[:, k1:]).view(*ctx.lead, a2.shape[1]) if ctx.needs_input_grad[1] else None
        dw = None
        if ctx.needs_input_grad[2]:
            dw = torch.empty_like(weight)
            gemm.gemm_tn_into(du, a1, dw[:, :k1])
            gemm.gemm_tn_into(du, a2, dw[:, k1:])
        db = du.sum(dim=0, dtype=torch.float32).to(du.dtype) if (ctx.has_bias and ctx.needs_input_grad[3]) else None
        return d1, d2, dw, db


def linear_merged(x1, x2, weight, bias=None):
    return _LinearMerged.apply(x1, x2, weight, bias)


def linear(x, weight, bias=None, activation=None):
    if activation not in (None, "gelu", "gelu_tanh"):
        from . import reference
        return reference.linear(x, weight, bias, activation)
    return _Linear.apply(x, weight, bias, activation)


# ---------------------------------------------------------------------------------------------
# QKV projection + QK-RMSNorm + RoPE -> head-major q, k, v
# ---------------------------------------------------------------------------------------------

class _QKVProjection(torch.autograd.Function):
    """One or two token streams (video [+ text]) projected into shared ``[B, h, S_total, 128]`` buffers."""

    @staticmethod
    def forward(ctx, heads, eps, rope_len, cos, sin, x, w, b, qw, kw, x2, w2, b2, qw2, kw2):
        B, S1, K = x.shape
        S2 = 0 if x2 is None else x2.shape[1]
        S = S1 + S2
        dev = x.device
        q = torch.empty(B, heads, S, 128, dtype=BF16, device=dev)
        k, v = torch.empty_like(q), torch.empty_like(q)
        cosf = None if cos is None else check(cos.float().contiguous(), torch.float32, "cos")
        sinf = None if sin is None else check(sin.float().contiguous(), torch.float32, "sin")
        saved = []
        for (xs, ws, bs, qws, kws, off, rl) in ((x, w, b, qw, kw, 0, rope_len), (x2, w2, b2, qw2, kw2, S1, 0)):
            if xs is None:
                saved += [None, None]
                continue
            xs2 = xs.reshape(-1, K)
            qkv = _gemm_nt(xs2, ws, bs)
            if qkv.shape[1] != heads * 384:
                raise _lib.NativeError("QKV weight does not match heads * 3 * 128")
            rows = qkv.shape[0]
            call("tt_qkv_post_fwd", ptr(qkv), ptr(check(qws.contiguous(), BF16, "q_norm")),
                 ptr(check(kws.contiguous(), BF16, "k_norm")), ptr(cosf if rl else None), ptr(sinf if rl else None),
                 ptr(q), ptr(k), ptr(v), c_long(rows), c_int(heads), c_long(rows // B), c_long(S), c_long(off),
                 c_long(rl), c_float(eps), stream())
            saved += [xs2, qkv]
        ctx.save_for_backward(cosf, sinf, w, qw, kw, w2, qw2, kw2, *saved)
        ctx.meta = (heads, eps, rope_len, B, S1, S2, K, b is not None, b2 is not None)
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cosf, sinf, w, qw, kw, w2, qw2, kw2, xa, qkva, xb, qkvb = ctx.saved_tensors
        heads, eps, rope_len, B, S1, S2, K, has_b, has_b2 = ctx.meta
        S = S1 + S2
        dq, dk, dv = (check(t.contiguous(), BF16, "dqkv") for t in (dq, dk, dv))
        outs = []
        for (xs2, qkv, ws, qws, kws, off, rl, hb) in ((xa, qkva, w, qw, kw, 0, rope_len, has_b),
                                                      (xb, qkvb, w2, qw2, kw2, S1, 0, has_b2)):
            if xs2 is None:
                outs.append((None, None, None, None, None))
                continue
            rows = qkv.shape[0]
            dqkv = torch.empty_like(qkv)
            nw = _lib.lib().tt_qkv_partial_warps(c_long(rows), c_int(heads))
            partials = torch.empty(nw * 256, dtype=torch.float32, device=qkv.device)
            dqw = torch.empty(128, dtype=BF16, device=qkv.device)
            dkw = torch.empty_like(dqw)
            call("tt_qkv_post_bwd", ptr(dq), ptr(dk), ptr(dv), ptr(qkv), ptr(qws.contiguous()), ptr(kws.contiguous()),
                 ptr(cosf if rl else None), ptr(sinf if rl else None), ptr(dqkv), ptr(partials), ptr(dqw), ptr(dkw),
                 c_long(rows), c_int(heads), c_long(rows // B), c_long(S), c_long(off), c_long(rl), c_float(eps), stream())
            dx = _gemm_nn(dqkv, ws).view(B, -1, K)
            dw = _gemm_tn(dqkv, xs2)
            db = dqkv.sum(dim=0, dtype=torch.float32).to(BF16) if hb else None
            outs.append((dx, dw, db, dqw, dkw))
        (dx1, dw1, db1, dqw1, dkw1), (dx2, dw2, db2, dqw2, dkw2) = outs
        return None, None, None, None, None, dx1, dw1, db1, dqw1, dkw1, dx2, dw2, db2, dqw2, dkw2


def qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin, num_heads, eps=1e-6, rope_len=None):
    if q_norm_weight.shape[0] != 128:
        from . import reference
        return reference.qkv_projection(x, weight, bias, q_norm_weight, k_norm_weight, cos, sin, num_heads, eps, rope_len)
    rl = 0 if cos is None else (x.shape[1] if rope_len is None else rope_len)
    return _QKVProjection.apply(num_heads, eps, rl, cos, sin, x, weight, bias, q_norm_weight, k_norm_weight,
                                None, None, None, None, None)


def joint_qkv_projection(x, weight, bias, qw, kw, cos, sin, x2, weight2, bias2, qw2, kw2, num_heads, eps=1e-6):
    """Video stream (with RoPE) and text stream (without) into one ``[B, h, S + T, 128]`` q / k / v."""
    return _QKVProjection.apply(num_heads, eps, x.shape[1], cos, sin, x, weight, bias, qw, kw,
                                x2, weight2, bias2, qw2, kw2)


# ---------------------------------------------------------------------------------------------
# attention
# ---------------------------------------------------------------------------------------------

def attention(q, k, v, kv_valid_len=None, scale=None, mask_range=None):
    from . import attention_backend as attn
    return attn.attention(q, k, v, kv_valid_len, scale, mask_range)


# ---------------------------------------------------------------------------------------------
# flow matching: noise mix and weighted MSE loss
# ---------------------------------------------------------------------------------------------

def noise_mix(latents: torch.Tensor, noise: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
    """``(1 - sigma[b]) * latents + sigma[b] * noise`` in one pass (no gradient: the inputs are data)."""
    B = latents.shape[0]
    lat = check(latents.contiguous(), BF16, "latents")
    nz = check(noise.contiguous(), BF16, "noise")
    sg = check(sigma.float().contiguous(), torch.float32, "sigma", align=4)
    out = torch.empty_like(lat)
    call("tt_noise_mix", ptr(lat), ptr(nz), ptr(sg), ptr(out), c_long(lat.numel() // B), c_int(B), stream())
    return out


class _FlowMatchLoss(torch.autograd.Function):
    """``mean(weight[b] * (pred - (noise - latents))^2)``: the forward kernel also writes d loss / d pred, so the backward is
    one scaling by the incoming scalar."""

    @staticmethod
    def forward(ctx, pred, noise, latents, weight):
        B = pred.shape[0]
        p = check(pred.contiguous(), BF16, "pred")
        nz = check(noise.contiguous(), BF16, "noise")
        lat = check(latents.contiguous(), BF16, "latents")
        w = check(weight.float().reshape(B).contiguous(), torch.float32, "weight", align=4)
        partials = torch.empty(_lib.lib().tt_flow_loss_blocks(), dtype=torch.float32, device=p.device)
        loss = torch.empty((), dtype=torch.float32, device=p.device)
        dpred = torch.empty_like(p) if ctx.needs_input_grad[0] else None
        call("tt_flow_loss", ptr(p), ptr(nz), ptr(lat), ptr(w), ptr(partials), ptr(dpred), ptr(loss), c_long(p.numel() // B),
             c_int(B), stream())
        ctx.save_for_backward(dpred)
        ctx.shape = pred.shape
        return loss

    @staticmethod
    def backward(ctx, g):
        (dpred,) = ctx.saved_tensors
        if dpred is None:
            return None, None, None, None
        return (dpred * g.to(dpred.dtype)).view(ctx.shape), None, None, None


def flow_match_loss(pred, noise, latents, weight):
    return _FlowMatchLoss.apply(pred, noise, latents, weight)


# ---------------------------------------------------------------------------------------------
# optimizer
# ---------------------------------------------------------------------------------------------

def adamw_update(param, grad, exp_avg, exp_avg_sq, master, master_lo, *, lr, beta1, beta2, eps, weight_decay, step,
                 grad_scale=1.0):
    n = param.numel()
    state_bf16 = exp_avg.dtype == BF16
    if n % 8 or any(t is not None and t.data_ptr() % 16 for t in (param, grad, exp_avg, exp_avg_sq, master, master_lo)):
        from .optim import adamw_update_reference
        adamw_update_reference(param, grad, exp_avg, exp_avg_sq, master, master_lo, lr=lr, beta1=beta1, beta2=beta2,
                               eps=eps, weight_decay=weight_decay, step=step, grad_scale=grad_scale)
        return
    check(param, BF16, "param")
    check(grad, BF16, "grad")
    sdt = BF16 if state_bf16 else torch.float32
    check(exp_avg, sdt, "exp_avg")
    check(exp_avg_sq, sdt, "exp_avg_sq")
    call("tt_adamw", ptr(param), ptr(grad), ptr(exp_avg), ptr(exp_avg_sq), ptr(master), ptr(master_lo), c_long(n),
         c_int(1 if state_bf16 else 0), c_float(lr), c_float(beta1), c_float(beta2), c_float(eps), c_float(weight_decay),
         c_int(step), c_float(grad_scale), stream())
