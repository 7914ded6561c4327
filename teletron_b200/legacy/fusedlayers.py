"""Module-level names of the reference's fused-layer wrappers (``teletron/models/dit/dit_fusedlayers.py``), on top of
:mod:`teletron_b200.ops`, for code that imported them directly.

* :class:`FP32LayerNorm` (``:48-57``), :class:`AdaLNCustom` (``:139-153``), :func:`AdaLNModelFunction.apply`
  (``:59-137``): ``LN(x) * (1 + scale) + shift`` with per-sample ``scale`` / ``shift``.
* :class:`FusedAdaLayerNormZero` (``:155-224``, six modulation vectors) and :class:`FusedAdaLayerNormZeroSingle`
  (``:226-272``, three): ``Linear(SiLU(emb))`` column-parallel over the tensor-parallel group with the output
  all-gathered, followed by the modulated LayerNorm.
* :func:`RMSNormModelFunction.apply` (``:274-348``) and :func:`Get_RMSNorm` (``:350-375``).

The op layer picks the sm_100a kernels for bf16 CUDA tensors and the PyTorch formulation otherwise, for any hidden
size that is a multiple of 8: the reference switches to its kernel only for ``embedding_dim == 3072`` and with
``FUSED_KERNELS=1``; here the environment variable still selects the implementation (``0`` forces the PyTorch one), but
there is a single code path and a single set of numerics checks.
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..models.hunyuanvideo.blocks import AdaLNModulation


def _impl():
    """``FUSED_KERNELS=0`` pins the PyTorch implementation, as the reference's environment switch does."""
    return ops.impl("torch") if os.environ.get("FUSED_KERNELS", "1") == "0" else ops.impl(ops.get_impl())


class FP32LayerNorm(nn.LayerNorm):
    """LayerNorm evaluated in fp32 whatever the input dtype."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = None if self.weight is None else self.weight.float()
        b = None if self.bias is None else self.bias.float()
        return F.layer_norm(x.float(), self.normalized_shape, w, b, self.eps).to(x.dtype)


class AdaLNModelFunction:
    """``apply(x, scale, shift, eps, cols)``: ``x [B, S, cols]``, ``scale`` / ``shift`` ``[B, cols]``."""

    @staticmethod
    def apply(x: torch.Tensor, scale: torch.Tensor, shift: torch.Tensor, eps: float = 1e-6, cols: Optional[int] = None) -> torch.Tensor:
        if cols is not None and x.shape[-1] != cols:
            raise ValueError(f"last dim of x must be {cols}, got {x.shape[-1]}")
        with _impl():
            return ops.layernorm_modulate(x, scale, shift, eps)


class AdaLNCustom(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6):
        super().__init__()
        self.hidden_size, self.eps = hidden_size, eps

    def forward(self, x, scale, shift):
        for name, t in (("x", x), ("scale", scale), ("shift", shift)):
            if t.shape[-1] != self.hidden_size:
                raise ValueError(f"last dim of {name} must be hidden_size {self.hidden_size}, got {t.shape[-1]}")
        return AdaLNModelFunction.apply(x, scale, shift, self.eps, self.hidden_size)


class _FusedAdaLNBase(nn.Module):
    def __init__(self, embedding_dim: int, n_chunks: int, norm_type: str, bias: bool, linear_parallel: bool, tp: int,
                 device=None, dtype=None):
        super().__init__()
        if norm_type not in ("layer_norm", "fp32_layer_norm"):
            raise ValueError(f"Unsupported `norm_type` ({norm_type}) provided. Supported ones are: 'layer_norm', 'fp32_layer_norm'.")
        self.n_chunks = n_chunks
        if linear_parallel:
            self.mod = AdaLNModulation(embedding_dim, n_chunks, tp=tp, device=device, dtype=dtype)
        else:
            self.mod = None
            self.linear = nn.Linear(embedding_dim, n_chunks * embedding_dim, bias=bias, device=device, dtype=dtype)
        self.adaLN = AdaLNCustom(embedding_dim, eps=1e-6)

    def _vectors(self, emb: torch.Tensor):
        if self.mod is not None:
            return self.mod(emb)
        return self.linear(F.silu(emb)).chunk(self.n_chunks, dim=1)


class FusedAdaLayerNormZero(_FusedAdaLNBase):
    """adaLN-Zero of a dual-stream block: returns ``(x_modulated, gate_msa, shift_mlp, scale_mlp, gate_mlp)``."""

    def __init__(self, embedding_dim: int, num_embeddings: Optional[int] = None, norm_type: str = "layer_norm", bias: bool = True,
                 fused_kernels: bool = True, linear_parallel: bool = False, tp: int = 1, device=None, dtype=None):
        if num_embeddings is not None:
            raise NotImplementedError("class-label embeddings are not part of the HunyuanVideo model")
        super().__init__(embedding_dim, 6, norm_type, bias, linear_parallel, tp, device, dtype)

    def forward(self, x: torch.Tensor, emb: torch.Tensor) -> Tuple[torch.Tensor, ...]:
        shift_msa, scale_msa, gate_msa, shift_mlp, scale_mlp, gate_mlp = self._vectors(emb)
        return self.adaLN(x, scale_msa, shift_msa), gate_msa, shift_mlp, scale_mlp, gate_mlp


class FusedAdaLayerNormZeroSingle(_FusedAdaLNBase):
    """adaLN-Zero of a single-stream block: returns ``(x_modulated, gate_msa)``."""

    def __init__(self, embedding_dim: int, norm_type: str = "layer_norm", bias: bool = True, fused_kernels: bool = True,
                 linear_parallel: bool = False, tp: int = 1, device=None, dtype=None):
        super().__init__(embedding_dim, 3, norm_type, bias, linear_parallel, tp, device, dtype)

    def forward(self, x: torch.Tensor, emb: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        shift_msa, scale_msa, gate_msa = self._vectors(emb)
        return self.adaLN(x, scale_msa, shift_msa), gate_msa


class RMSNormModelFunction:
    """``apply(x, weight, eps)``: RMSNorm over the last dim."""

    @staticmethod
    def apply(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
        with _impl():
            return ops.rmsnorm(x, weight, eps)


class _RMSNorm(nn.Module):
    def __init__(self, hidden_size: int, eps: float = 1e-6, device=None, dtype=None, **_unused):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return RMSNormModelFunction.apply(x, self.weight, self.eps)


def Get_RMSNorm():
    """The RMSNorm module class to use (the reference returns its fused class or an fp32 fallback depending on
    ``FUSED_KERNELS``; here one class covers both, the switch is read at call time)."""
    return _RMSNorm
