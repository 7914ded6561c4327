"""Architecture and runtime configuration of the HunyuanVideo-style MMDiT.

Architecture constants follow ``teletron/models/hunyuanvideo/model.py:39-59``; the
``NUM_LAYERS`` / ``NUM_SINGLE_LAYERS`` / ``FUSED_KERNELS`` environment overrides follow
``model.py:69-88``.  Unlike the reference the defaults here are the real 13B depths
(20 dual-stream + 40 single-stream blocks); the reference's class defaults (3 + 6) are
its sanity-check size and are available as :func:`sanity_config`.
"""

from __future__ import annotations

import dataclasses
import os
from typing import Optional, Tuple


@dataclasses.dataclass
class HunyuanParams:
    hidden_size: int = 3072
    num_attention_heads: int = 24
    attention_head_dim: int = 128
    in_channels: int = 33            # I2V: 16 latent + 16 first-frame latent + 1 mask
    out_channels: int = 16
    num_layers: int = 20             # dual-stream blocks
    num_single_layers: int = 40      # single-stream blocks
    num_refiner_layers: int = 2
    mlp_ratio: float = 4.0
    patch_size: int = 2
    patch_size_t: int = 1
    qk_norm: str = "rms_norm"
    guidance_embeds: bool = True
    text_embed_dim: int = 4096
    pooled_projection_dim: int = 768
    rope_theta: float = 256.0
    rope_axes_dim: Tuple[int, int, int] = (16, 56, 56)
    add_qkv_bias: bool = True
    # dual-block MLP activation: the reference uses exact-erf GELU for the dual blocks
    # (model.py:42) and tanh GELU in the single blocks (dit_layerspec.py:276)
    dual_mlp_activation: str = "gelu"
    single_mlp_activation: str = "gelu_tanh"
    layernorm_epsilon: float = 1e-6
    # runtime
    recompute_granularity: Optional[str] = None      # None | "full" | "selective"
    recompute_method: str = "block"                  # "block" | "uniform"
    recompute_num_layers: Optional[int] = None       # None = every block (reference behaviour)
    sequence_parallel: bool = False                  # shard the residual stream's tokens over tensor-parallel ranks
    sequence_pad_multiple: int = 8                   # local video tokens are padded to a multiple of this (GEMM K / TMA alignment of the weight gradients)
    sequence_parallel_row_multiple: int = 1          # token blocks are padded to a multiple of this (128 for the fused TP kernels)
    recompute_save_attention: bool = False           # keep attention (out, lse) so the recompute pass skips that kernel
    fused_kernels: bool = True
    init_method_std: float = 0.006
    apply_text_mask: bool = False                    # reference never applies it (dit_attention.py:313)
    seed: int = 1234

    def __post_init__(self):
        if self.hidden_size != self.num_attention_heads * self.attention_head_dim:
            raise ValueError("hidden_size must equal heads * head_dim")
        if sum(self.rope_axes_dim) != self.attention_head_dim:
            raise ValueError("rope axes must sum to the head dim")

    def apply_env_overrides(self) -> "HunyuanParams":
        """Depth / fused-kernel overrides exported by the launch scripts."""
        for env, field in (("NUM_LAYERS", "num_layers"), ("NUM_SINGLE_LAYERS", "num_single_layers")):
            v = os.environ.get(env)
            if v:
                try:
                    setattr(self, field, int(v))
                except ValueError as e:
                    raise ValueError(f"Invalid integer value for {env}: {v}") from e
        v = os.environ.get("FUSED_KERNELS")
        if v:
            self.fused_kernels = bool(int(v))
        return self

    @property
    def mlp_hidden(self) -> int:
        return int(self.hidden_size * self.mlp_ratio)

    def num_parameters(self) -> int:
        """Parameters in the dual + single blocks (the '13B' figure counts these)."""
        h = self.hidden_size
        dual = 2 * (6 * h * h + 6 * h) + 2 * (3 * h * h + 3 * h) + 2 * (h * h + h) \
            + 2 * (2 * h * self.mlp_hidden + h + self.mlp_hidden) + 4 * self.attention_head_dim
        single = (3 * h * h + 3 * h) + (3 * h * h + 3 * h) + (h * self.mlp_hidden + self.mlp_hidden) \
            + ((h + self.mlp_hidden) * h + h) + 2 * self.attention_head_dim
        return self.num_layers * dual + self.num_single_layers * single


def hunyuan_13b(**kw) -> HunyuanParams:
    return HunyuanParams(**kw)


def sanity_config(**kw) -> HunyuanParams:
    """3 dual + 6 single blocks at full width (``run_unified_sanity_check.sh:32-33``)."""
    return HunyuanParams(num_layers=3, num_single_layers=6, **kw)


def tiny_config(**kw) -> HunyuanParams:
    """CPU plumbing model: hidden 128 = 2 heads x 64, 2 + 2 blocks, RoPE axes (16, 24, 24)."""
    base = dict(hidden_size=128, num_attention_heads=2, attention_head_dim=64, in_channels=16,
                out_channels=16, num_layers=2, num_single_layers=2, num_refiner_layers=2,
                text_embed_dim=64, pooled_projection_dim=32, rope_axes_dim=(16, 24, 24),
                init_method_std=0.02)
    base.update(kw)
    return HunyuanParams(**base)
