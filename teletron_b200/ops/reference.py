"""Pure-PyTorch implementations of every op in :mod:`teletron_b200.ops`.

These run on CPU (fp32) and GPU and are differentiable through ordinary autograd.
They serve three purposes: the numerics oracle for the sm_100a kernels, the CPU /
gloo plumbing path used by the unit tests, and the "library composition" baseline
(cuBLAS GEMM + SDPA + elementwise) that restates what the reference executes
(reference: ``teletron/models/dit/dit_layerspec.py:115-186`` and
``teletron/models/dit/dit_attention.py:240-338``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F


def layernorm_modulate(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor,
                       eps: float = 1e-6) -> torch.Tensor:
    """``LayerNorm(x) * (1 + scale) + shift`` without affine parameters.

    ``x`` is ``[B, S, H]``; ``scale`` / ``shift`` are ``[B, H]``.  Statistics are
    taken in fp32 regardless of the input dtype (the reference's fused kernel does
    the modulation in bf16, ``teletron_op/fused_adaln/adaln_forward.cu:188-189``).
    """
    xf = x.float()
    mean = xf.mean(dim=-1, keepdim=True)
    var = xf.var(dim=-1, unbiased=False, keepdim=True)
    xn = (xf - mean) * torch.rsqrt(var + eps)
    y = xn * (1.0 + scale.float().unsqueeze(1)) + shift.float().unsqueeze(1)
    return y.to(x.dtype)


def gate_residual(residual: torch.Tensor, branch: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``residual + gate[:, None, :] * branch`` (``dit_layerspec.py:152-156``)."""
    return (residual.float() + gate.float().unsqueeze(1) * branch.float()).to(residual.dtype)


def gate_residual_layernorm_modulate(residual, branch, gate, scale, shift, eps: float = 1e-6):
    """Fusion of :func:`gate_residual` and :func:`layernorm_modulate`.

    Returns ``(new_residual, modulated)``.
    """
    new_res = gate_residual(residual, branch, gate)
    return new_res, layernorm_modulate(new_res, scale, shift, eps)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """RMSNorm over the last dimension with fp32 statistics."""
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + eps)
    return (xf * rstd * weight.float()).to(x.dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding on adjacent element pairs (``(2i, 2i+1)``).

    ``x`` is ``[B, h, S, D]``; ``cos`` / ``sin`` are ``[S, D]`` with each frequency
    repeated twice, the layout produced by the rotary table of
    ``teletron/models/hunyuanvideo/layers.py:224-252``.
    """
    xf = x.float()
    x_even = xf[..., 0::2]
    x_odd = xf[..., 1::2]
    rot = torch.stack((-x_odd, x_even), dim=-1).flatten(-2)
    out = xf * cos.float() + rot * sin.float()
    return out.to(x.dtype)


def _act(x: torch.Tensor, activation: Optional[str]) -> torch.Tensor:
    if activation is None:
        return x
    if activation == "gelu":
        return F.gelu(x)
    if activation == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    if activation == "silu":
        return F.silu(x)
    raise ValueError(f"unknown activation {activation!r}")


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           activation: Optional[str] = None) -> torch.Tensor:
    """``act(x @ weight.T + bias)``; ``weight`` is ``[out, in]``."""
    return _act(F.linear(x, weight, bias), activation)


def linear_merged(x1: torch.Tensor, x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``cat([x1, x2], -1) @ weight.T + bias``: the single-stream block's projection of ``[attention | MLP]``."""
    return F.linear(torch.cat([x1, x2], dim=-1), weight, bias)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
              kv_valid_len: Optional[int] = None, scale: Optional[float] = None, mask_range=None) -> torch.Tensor:
    """Non-causal softmax attention.

    ``q, k, v`` are ``[B, h, S, D]``; the result is ``[B, S, h * D]`` (token-major,
    the layout the output projection consumes).  ``kv_valid_len`` masks keys at
    positions ``>= kv_valid_len`` (padded text tokens sit at the sequence tail) and
    ``mask_range = (lo, hi)`` masks keys in ``[lo, hi)`` (padded text tokens when the text
    comes first); the reference never applies its mask (``dit_attention.py:313``), so
    ``None`` is the parity setting.
    """
    B, h, S, D = q.shape
    n = k.shape[2]
    tail = kv_valid_len is not None and kv_valid_len < n
    mid = mask_range is not None and mask_range[0] < mask_range[1]
    if tail or mid:
        mask = torch.ones(1, 1, 1, n, dtype=torch.bool, device=q.device)
        if tail:
            mask[..., kv_valid_len:] = False
        if mid:
            mask[..., mask_range[0]:mask_range[1]] = False
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale)
    else:
        o = F.scaled_dot_product_attention(q, k, v, scale=scale)
    return o.transpose(1, 2).reshape(B, S, h * D)


def qkv_projection(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                   q_norm_weight: torch.Tensor, k_norm_weight: torch.Tensor,
                   cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                   num_heads: int, eps: float = 1e-6,
                   rope_len: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """QKV GEMM + per-head split + QK-RMSNorm + RoPE.

    ``weight`` rows are ordered ``[head][q | k | v][head_dim]`` (the Megatron packing
    kept by the converted checkpoints, ``convert_hunyuanvideo.py:379-387``).  Returns
    ``q, k, v`` each ``[B, heads, S, D]``.  RoPE is applied to the first ``rope_len``
    tokens (all tokens when ``None``); tokens beyond it (text) are left un-rotated,
    matching ``dit_attention.py:435-447``.
    """
    B, S, _ = x.shape
    qkv = F.linear(x, weight, bias)
    D = qkv.shape[-1] // (3 * num_heads)
    qkv = qkv.view(B, S, num_heads, 3, D)
    q = qkv[:, :, :, 0].transpose(1, 2)
    k = qkv[:, :, :, 1].transpose(1, 2)
    v = qkv[:, :, :, 2].transpose(1, 2).contiguous()
    q = rmsnorm(q, q_norm_weight, eps)
    k = rmsnorm(k, k_norm_weight, eps)
    if cos is not None:
        n = S if rope_len is None else rope_len
        if n == S:
            q = apply_rope(q, cos, sin)
            k = apply_rope(k, cos, sin)
        else:
            q = torch.cat([apply_rope(q[:, :, :n], cos, sin), q[:, :, n:]], dim=2)
            k = torch.cat([apply_rope(k[:, :, :n], cos, sin), k[:, :, n:]], dim=2)
    return q.contiguous(), k.contiguous(), v


def joint_qkv_projection(x, weight, bias, qw, kw, cos, sin, x2, weight2, bias2, qw2, kw2, num_heads, eps=1e-6):
    """Two streams with separate weights into one concatenated ``[B, h, S + T, D]`` q / k / v."""
    q, k, v = qkv_projection(x, weight, bias, qw, kw, cos, sin, num_heads, eps)
    q2, k2, v2 = qkv_projection(x2, weight2, bias2, qw2, kw2, None, None, num_heads, eps)
    return torch.cat([q, q2], dim=2), torch.cat([k, k2], dim=2), torch.cat([v, v2], dim=2)


def noise_mix(latents: torch.Tensor, noise: torch.Tensor, sigma: torch.Tensor) -> torch.Tensor:
    """``(1 - sigma[b]) * latents + sigma[b] * noise`` in the dtype of ``latents`` (``pipeline.py:118-129``)."""
    sig = sigma.view(-1, *([1] * (latents.dim() - 1))).to(latents.dtype)
    return (1.0 - sig) * latents + sig * noise


def flow_match_loss(pred: torch.Tensor, noise: torch.Tensor, latents: torch.Tensor,
                    weight: torch.Tensor) -> torch.Tensor:
    """Mean of ``weight * (pred - (noise - latents))^2`` in fp32 (``pipeline.py:215-224``)."""
    target = noise.float() - latents.float()
    w = weight.float().view(-1, *([1] * (pred.dim() - 1)))
    return (w * (pred.float() - target) ** 2).mean()
