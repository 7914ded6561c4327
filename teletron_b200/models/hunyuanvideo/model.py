"""HunyuanVideo-style MMDiT (``teletron/models/hunyuanvideo/model.py:61-434``).

``forward(hidden_states, timestep, encoder_hidden_states, encoder_attention_mask,
pooled_projections, guidance)`` keeps the reference signature.  Differences made on
purpose:

* no dense ``[B, N, N]`` boolean mask is materialised (the reference builds one and never
  uses it, ``model.py:295-319``); an optional key-length mask is passed to attention when
  ``cfg.apply_text_mask`` is set;
* context-parallel padding is an explicit value threaded through the blocks instead of
  module globals, and is handled identically with and without recompute (the reference's
  non-recompute path strips the pad from local shards, ``model.py:386-389``);
* ``recompute_method="block"`` honours ``recompute_num_layers`` (``None`` = every block, which
  is what the reference's loop does in effect, ``model.py:225-238``).
"""

from __future__ import annotations

import hashlib
from typing import Optional

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from ... import ops
from ...parallel import mappings as M
from ...parallel import state as ps
from ...parallel.pad import SeqPad
from .blocks import AdaLNContinuous, HunyuanDiTLayer, HunyuanSingleDiTLayer
from .config import HunyuanParams
from .embeddings import (CombinedTimestepGuidanceTextProjEmbeddings, HunyuanVideoPatchEmbed,
                         HunyuanVideoRotaryPosEmbed)
from .refiner import HunyuanVideoTokenRefiner


def _param_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


class HunyuanVideoTransformer3DModel(nn.Module):
    def __init__(self, cfg: HunyuanParams, tp: Optional[int] = None, device=None, dtype=None):
        super().__init__()
        self.cfg = cfg
        tp = ps.get_tensor_model_parallel_world_size() if tp is None else tp
        self.tp = tp
        kw = dict(device=device, dtype=dtype)
        H = cfg.hidden_size
        if cfg.num_attention_heads % tp:
            raise ValueError(f"{cfg.num_attention_heads} heads not divisible by tp={tp}")
        self.x_embedder = HunyuanVideoPatchEmbed((cfg.patch_size_t, cfg.patch_size, cfg.patch_size),
                                                 cfg.in_channels, H).to(**kw)
        self.context_embedder = HunyuanVideoTokenRefiner(cfg.text_embed_dim, cfg.num_attention_heads,
                                                         cfg.attention_head_dim, cfg.num_refiner_layers).to(**kw)
        self.time_text_embed = CombinedTimestepGuidanceTextProjEmbeddings(
            H, cfg.pooled_projection_dim, guidance=cfg.guidance_embeds).to(**kw)
        self.rope = HunyuanVideoRotaryPosEmbed(cfg.patch_size, cfg.patch_size_t, cfg.rope_axes_dim, cfg.rope_theta)
        self.transformer_blocks = nn.ModuleList([HunyuanDiTLayer(cfg, tp, **kw) for _ in range(cfg.num_layers)])
        self.single_transformer_blocks = nn.ModuleList(
            [HunyuanSingleDiTLayer(cfg, tp, **kw) for _ in range(cfg.num_single_layers)])
        self.norm_out = AdaLNContinuous(H, H, cfg.layernorm_epsilon, **kw)
        self.proj_out = nn.Linear(H, cfg.patch_size_t * cfg.patch_size * cfg.patch_size * cfg.out_channels, **kw)
        self.reset_parameters(cfg.seed)

    # ------------------------------------------------------------------ init
    @torch.no_grad()
    def reset_parameters(self, seed: int) -> None:
        """Deterministic, tensor-parallel-consistent initialisation.

        Every parameter is drawn from a generator seeded by ``(seed, parameter name)`` at
        its *full* (unsharded) shape on the parameter's device and then sliced, so any TP
        layout holds exactly the shards of the TP=1 model (Megatron gets the same effect
        with ``use_cpu_initialization``, ``model.py:103``).
        """
        n_blocks = max(1, self.cfg.num_layers + self.cfg.num_single_layers)
        std = self.cfg.init_method_std
        tp_rank = ps.get_tensor_model_parallel_rank() if self.tp > 1 else 0
        for name, p in self.named_parameters():
            kind = getattr(p, "init_kind", None)
            gen = torch.Generator(device=p.device)
            gen.manual_seed(_param_seed(seed, name))
            if kind is None:
                # embedders / head: fan-in uniform for matrices, zeros for vectors
                if p.dim() >= 2:
                    fan_in = p[0].numel()
                    bound = (1.0 / fan_in) ** 0.5
                    p.copy_(torch.empty(p.shape, device=p.device, dtype=torch.float32).uniform_(-bound, bound, generator=gen))
                elif name.endswith("weight"):
                    p.fill_(1.0)        # LayerNorm weights in the refiner
                else:
                    p.zero_()
                continue
            if kind == "zeros":
                p.zero_()
                continue
            if kind == "ones":
                p.fill_(1.0)
                continue
            s = std if kind == "normal" else std / (2.0 * n_blocks) ** 0.5
            full = torch.empty(p.full_shape, device=p.device, dtype=torch.float32).normal_(0.0, s, generator=gen)
            p.copy_(shard_tensor(full, p.partition_dim, self.tp, tp_rank, p.partitions))

    # ------------------------------------------------------------------ forward
    def _run_blocks(self, blocks, x, ctx, temb, cos, sin, pad, kv_valid_len):
        cfg = self.cfg
        n = len(blocks)
        if cfg.recompute_granularity == "full":
            if cfg.recompute_method == "uniform":
                chunk = cfg.recompute_num_layers or 1

                def run(start, end):
                    def fn(x, ctx, temb, cos, sin):
                        for b in blocks[start:end]:
                            x, ctx = b(x, ctx, temb, cos, sin, pad, kv_valid_len)
                        return x, ctx
                    return fn
                if chunk > 1:
                    # several blocks per checkpoint: tensors that the fused collective ops save are private copies here,
                    # since a later block's replay would overwrite the shared workspace before an earlier block's backward
                    for start in range(0, n, chunk):
                        x, ctx = checkpoint(run(start, min(n, start + chunk)), x, ctx, temb, cos, sin,
                                            use_reentrant=False, preserve_rng_state=False)
                    return x, ctx
                limit = n
            else:
                limit = n if cfg.recompute_num_layers is None else min(n, cfg.recompute_num_layers)
            from ...training.recompute import checkpoint_block
            for i, b in enumerate(blocks):
                if i < limit:
                    # one block per checkpoint: its replay is followed at once by its backward
                    x, ctx = checkpoint_block(b, (x, ctx, temb, cos, sin), (pad, kv_valid_len),
                                              save_attention=bool(cfg.recompute_save_attention))
                else:
                    x, ctx = b(x, ctx, temb, cos, sin, pad, kv_valid_len)
            return x, ctx
        for b in blocks:
            x, ctx = b(x, ctx, temb, cos, sin, pad, kv_valid_len)
        return x, ctx

    def forward(self, hidden_states: torch.Tensor, timestep: torch.Tensor, encoder_hidden_states: torch.Tensor,
                encoder_attention_mask: Optional[torch.Tensor], pooled_projections: torch.Tensor,
                guidance: Optional[torch.Tensor] = None, return_dict: bool = False):
        cfg = self.cfg
        B, _, Fr, Hh, Ww = hidden_states.shape
        p, pt = cfg.patch_size, cfg.patch_size_t
        f, h, w = Fr // pt, Hh // p, Ww // p

        cos, sin = self.rope(hidden_states)
        temb = self.time_text_embed(timestep, guidance, pooled_projections)
        x = self.x_embedder(hidden_states)
        ctx = self.context_embedder(encoder_hidden_states, timestep, encoder_attention_mask)

        kv_valid_len = None
        if cfg.apply_text_mask and encoder_attention_mask is not None:
            kv_valid_len = int(encoder_attention_mask.sum(dim=1).max().item())

        cp = ps.get_context_parallel_world_size()
        cp_group = ps.get_context_parallel_group()
        pad = None
        sp = bool(cfg.sequence_parallel) and self.tp > 1
        tp_group = ps.get_tensor_model_parallel_group()
        if sp and ctx.shape[1] % self.tp:
            raise ValueError(f"sequence parallelism needs the text length {ctx.shape[1]} divisible by tp = {self.tp}")
        if sp and cp == 1 and x.shape[1] % self.tp:
            raise ValueError(f"sequence parallelism needs the video token count {x.shape[1]} divisible by tp = {self.tp}")
        if cp > 1:
            # with sequence parallelism each context-parallel chunk is cut once more into tp token blocks
            # every rank's chunk is a multiple of sequence_pad_multiple tokens: the token count is the K dim of the weight-
            # gradient GEMMs, which the tensor-core kernel takes in multiples of 8
            per_rank = cfg.sequence_pad_multiple * (self.tp * cfg.sequence_parallel_row_multiple if sp else 1)
            pad = SeqPad.for_length(x.shape[1], cp * max(1, per_rank))
            x = M.split_forward_gather_backward(pad.add(x, 1), cp_group, dim=1, grad_scale="down")
            cos = M.split_forward_gather_backward(pad.add(cos, 0), cp_group, dim=0, grad_scale="down")
            sin = M.split_forward_gather_backward(pad.add(sin, 0), cp_group, dim=0, grad_scale="down")

        if sp:
            x = M.scatter_to_sequence_parallel_region(x, tp_group, dim=1)
            ctx = M.scatter_to_sequence_parallel_region(ctx, tp_group, dim=1)

        with ops.nvtx_range("dual_blocks"):
            x, ctx = self._run_blocks(self.transformer_blocks, x, ctx, temb, cos, sin, pad, kv_valid_len)
        with ops.nvtx_range("single_blocks"):
            x, ctx = self._run_blocks(self.single_transformer_blocks, x, ctx, temb, cos, sin, pad, kv_valid_len)

        if sp:
            # everything after the blocks is replicated over TP: every rank holds the full gradient of the gathered rows
            x = M.gather_forward_split_backward(x, tp_group, dim=1, grad_scale=None)
        if cp > 1:
            x = M.gather_forward_split_backward(x, cp_group, dim=1, grad_scale="up")
            x = pad.remove(x, 1)

        x = self.proj_out(self.norm_out(x, temb))
        x = x.reshape(B, f, h, w, -1, pt, p, p).permute(0, 4, 1, 5, 2, 6, 3, 7)
        x = x.flatten(6, 7).flatten(4, 5).flatten(2, 3)
        if return_dict:
            return {"sample": x}
        return (x,)

    def state_dict_for_save_checkpoint(self, prefix: str = "", keep_vars: bool = False):
        return self.state_dict(prefix=prefix, keep_vars=keep_vars)


def shard_tensor(full: torch.Tensor, dim: Optional[int], tp: int, rank: int, partitions=None) -> torch.Tensor:
    """This rank's tensor-parallel shard of a full weight.

    ``partitions`` (sizes along ``dim``) marks a dimension made of concatenated groups that
    are each sharded separately (single-block ``proj_out`` input ``[attn | mlp]``).
    """
    if dim is None or tp == 1:
        return full
    if partitions:
        parts, off = [], 0
        for n in partitions:
            step = n // tp
            parts.append(full.narrow(dim, off + rank * step, step))
            off += n
        return torch.cat(parts, dim=dim)
    step = full.size(dim) // tp
    return full.narrow(dim, rank * step, step)


def unshard_tensors(shards, dim: Optional[int], partitions=None) -> torch.Tensor:
    """Inverse of :func:`shard_tensor` given all ranks' shards in rank order."""
    tp = len(shards)
    if dim is None or tp == 1:
        return shards[0]
    if partitions:
        out, off = [], 0
        for n in partitions:
            step = n // tp
            out.extend(s.narrow(dim, off, step) for s in shards)
            off += step
        return torch.cat(out, dim=dim)
    return torch.cat(list(shards), dim=dim)
