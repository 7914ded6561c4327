"""Per-GPU memory model of a HunyuanVideo training step and the frame count it allows.

Terms (bf16 weights and gradients, ZeRO-1 optimizer state sharded over DP x CP, full activation recompute):

* weights + gradients: ``4 B x P / tp``;
* optimizer: ``(master + 2 moments) x P / tp / (dp * cp)`` - 12 B per parameter with an fp32 master and fp32 moments,
  6 B with the bf16 + int16 split master and bf16 moments;
* block-boundary activations kept for recompute: ``layers x local tokens x hidden x 2 B`` (video tokens are split over
  CP, and over TP as well with sequence parallelism; text tokens are replicated);
* attention outputs kept so that the recompute pass skips attention (``--recompute-save-attention``):
  ``layers x heads / (tp * cp) x all tokens x (128 x 2 B + 4 B)``;
* the working set of the one block that is being recomputed and differentiated:
  ``WORKING_SET_WIDTHS x local tokens x hidden x 2 B`` (its TP-sharded part shrinks with tp);
* Ulysses workspaces of the in-kernel collectives (q, k, v, o and their gradients in head-major layout).

``WORKING_SET_WIDTHS`` is the one fitted constant.  Measured peaks the model reproduces (GiB, 13B model, 720P): 147.2
on 1 GPU at 33 frames with the compact optimizer state; 23.9 (allocator) on 8 GPUs at tp2 x cp4, 33 frames; 79.9
(allocator 32.0 + symmetric heaps) on 8 GPUs at cp8, 129 frames.
"""

from __future__ import annotations

import dataclasses
from typing import Optional, Tuple

GIB = float(2 ** 30)
WORKING_SET_WIDTHS = 46.0        # hidden-widths of bf16 activations alive per local token inside one block's recompute + backward
EMBEDDER_PARAMS = 0.20e9         # patch / text / time embedders, token refiner, output head of the 13B model (not in the block count)


@dataclasses.dataclass
class MemoryEstimate:
    weights_grads: float
    optimizer: float
    boundaries: float
    saved_attention: float
    working_set: float
    workspaces: float

    @property
    def total(self) -> float:
        return self.weights_grads + self.optimizer + self.boundaries + self.saved_attention + self.working_set + self.workspaces

    def as_gib(self) -> dict:
        d = {k: v / GIB for k, v in dataclasses.asdict(self).items()}
        d["total"] = self.total / GIB
        return d


def video_tokens(frames: int, resolution: Tuple[int, int] = (1280, 720), patch: int = 2, patch_t: int = 1) -> int:
    """Latent frames ``(F - 1) / 4 + 1``, latent pixels ``/ 8``, patches ``1 x 2 x 2``."""
    w, h = resolution
    return ((frames - 1) // 4 + 1) // patch_t * (h // 8 // patch) * (w // 8 // patch)


def estimate(cfg, frames: int, resolution: Tuple[int, int] = (1280, 720), text_len: int = 256, tp: int = 1, cp: int = 1,
             dp: int = 1, sequence_parallel: bool = False, save_attention: bool = True, fused_comm: bool = True,
             optimizer_bytes_per_param: float = 12.0, extra_params: Optional[float] = None) -> MemoryEstimate:
    """Peak bytes per GPU.  ``cfg``: a :class:`HunyuanParams`; ``optimizer_bytes_per_param``: 12 (fp32 master + fp32
    moments) or 6 (split master + bf16 moments)."""
    params = cfg.num_parameters() + (EMBEDDER_PARAMS if extra_params is None else extra_params)
    layers = cfg.num_layers + cfg.num_single_layers
    hidden = cfg.hidden_size
    s = video_tokens(frames, resolution, cfg.patch_size, cfg.patch_size_t)
    s_cp = -(-s // cp)                                       # video tokens of one context-parallel rank
    local = (s_cp + text_len) / (tp if sequence_parallel else 1)
    heads_local = cfg.num_attention_heads / (tp * cp)
    all_tokens = s_cp * cp + text_len
    weights_grads = 4.0 * params / tp
    optimizer = optimizer_bytes_per_param * params / tp / (dp * cp)
    boundaries = layers * local * hidden * 2.0
    saved = layers * heads_local * all_tokens * (cfg.attention_head_dim * 2.0 + 4.0) if save_attention else 0.0
    # roughly a third of the block's live activations (LayerNorm outputs, residuals) is not TP-sharded
    working = WORKING_SET_WIDTHS * (s_cp + text_len) * hidden * 2.0 * (1.0 / 3.0 + 2.0 / 3.0 / tp)
    workspaces = 0.0
    if fused_comm and cp > 1:
        workspaces = 8.0 * heads_local * all_tokens * cfg.attention_head_dim * 2.0 + (s_cp + text_len) * hidden / tp * 2.0
    return MemoryEstimate(weights_grads, optimizer, boundaries, saved, working, workspaces)


def max_frames(cfg, limit_gib: float = 165.0, **kw) -> int:
    """Largest ``4k + 1`` frame count whose estimated peak stays under ``limit_gib`` (0 if even one frame does not fit)."""
    def fits(latent: int) -> bool:
        return estimate(cfg, 4 * (latent - 1) + 1, **kw).total / GIB <= limit_gib
    if not fits(1):
        return 0
    lo, hi = 1, 2
    while fits(hi) and hi < 1 << 16:
        lo, hi = hi, hi * 2
    while hi - lo > 1:
        mid = (lo + hi) // 2
        if fits(mid):
            lo = mid
        else:
            hi = mid
    return 4 * (lo - 1) + 1
