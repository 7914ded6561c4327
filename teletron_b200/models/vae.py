"""3-D causal-convolution video VAE (4x temporal, 8x spatial compression, 16 latent channels).

The reference takes ``AutoencoderKLHunyuanVideo`` from ``diffusers`` (``teletron/models/hunyuanvideo/pipeline.py:49-55,
228-233``; ``producer.py:45-58``; decode at ``examples/hunyuanvideo/pipelines.py:1001-1006``), which is not installed
here, so the architecture is restated with the same sub-module names (``encoder.down_blocks.N.resnets.M.conv1.conv``,
``mid_block.attentions.0.to_q`` ...) so that a diffusers checkpoint's ``vae.*`` keys load by name.  It runs on the
encoder-service ranks (or on DiT ranks with ``--with-vae``) through cuDNN convolutions; it is not a hand-kernel
target.  Slicing (one sample at a time) and spatial tiling with blended overlaps bound the activation memory at 720P.
"""

from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn


class CausalConv3d(nn.Module):
    """Conv3d that pads ``k_t - 1`` frames at the front (replicate) and nothing at the back."""

    def __init__(self, cin: int, cout: int, kernel: int = 3, stride=1, bias: bool = True):
        super().__init__()
        k = (kernel,) * 3 if isinstance(kernel, int) else tuple(kernel)
        self.pad = (k[2] // 2, k[2] // 2, k[1] // 2, k[1] // 2, k[0] - 1, 0)
        self.conv = nn.Conv3d(cin, cout, k, stride=stride, bias=bias)

    def forward(self, x):
        return self.conv(F.pad(x, self.pad, mode="replicate"))


class ResnetBlockCausal3D(nn.Module):
    def __init__(self, cin: int, cout: Optional[int] = None, groups: int = 32, eps: float = 1e-6):
        super().__init__()
        cout = cout or cin
        self.norm1 = nn.GroupNorm(groups, cin, eps=eps)
        self.conv1 = CausalConv3d(cin, cout, 3)
        self.norm2 = nn.GroupNorm(groups, cout, eps=eps)
        self.conv2 = CausalConv3d(cout, cout, 3)
        self.conv_shortcut = CausalConv3d(cin, cout, 1) if cin != cout else None

    def forward(self, x):
        h = self.conv1(F.silu(self.norm1(x)))
        h = self.conv2(F.silu(self.norm2(h)))
        return h + (x if self.conv_shortcut is None else self.conv_shortcut(x))


class _MidAttention(nn.Module):
    """Single-head attention over all (t, h, w) positions with a frame-causal mask."""

    def __init__(self, ch: int, groups: int = 32, eps: float = 1e-6):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, ch, eps=eps)
        self.to_q, self.to_k, self.to_v = nn.Linear(ch, ch), nn.Linear(ch, ch), nn.Linear(ch, ch)
        self.to_out = nn.ModuleList([nn.Linear(ch, ch), nn.Identity()])

    def forward(self, x):
        B, C, T, H, W = x.shape
        h = self.group_norm(x).permute(0, 2, 3, 4, 1).reshape(B, T * H * W, C)
        frame = torch.arange(T, device=x.device).repeat_interleave(H * W)
        mask = frame[:, None] >= frame[None, :]
        q, k, v = self.to_q(h)[:, None], self.to_k(h)[:, None], self.to_v(h)[:, None]
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)[:, 0]
        o = self.to_out[0](o).reshape(B, T, H, W, C).permute(0, 4, 1, 2, 3)
        return x + o


class _MidBlock(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlockCausal3D(ch), ResnetBlockCausal3D(ch)])
        self.attentions = nn.ModuleList([_MidAttention(ch)])

    def forward(self, x):
        return self.resnets[1](self.attentions[0](self.resnets[0](x)))


class _Downsample(nn.Module):
    def __init__(self, ch: int, stride: Tuple[int, int, int]):
        super().__init__()
        self.conv = CausalConv3d(ch, ch, 3, stride=stride)

    def forward(self, x):
        return self.conv(x)


class _Upsample(nn.Module):
    def __init__(self, ch: int, factor: Tuple[int, int, int]):
        super().__init__()
        self.factor = factor
        self.conv = CausalConv3d(ch, ch, 3)

    def forward(self, x):
        ft, fh, fw = self.factor
        if ft > 1 and x.shape[2] > 1:
            # the first latent frame stands for one video frame, every later one for `ft`
            first = F.interpolate(x[:, :, :1], scale_factor=(1, fh, fw), mode="nearest")
            rest = F.interpolate(x[:, :, 1:], scale_factor=(ft, fh, fw), mode="nearest")
            x = torch.cat([first, rest], dim=2)
        else:
            x = F.interpolate(x, scale_factor=(1, fh, fw), mode="nearest")
        return self.conv(x)


class _DownBlock(nn.Module):
    def __init__(self, cin: int, cout: int, layers: int, stride: Optional[Tuple[int, int, int]]):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlockCausal3D(cin if i == 0 else cout, cout) for i in range(layers)])
        self.downsamplers = nn.ModuleList([_Downsample(cout, stride)]) if stride else None

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        if self.downsamplers is not None:
            x = self.downsamplers[0](x)
        return x


class _UpBlock(nn.Module):
    def __init__(self, cin: int, cout: int, layers: int, factor: Optional[Tuple[int, int, int]]):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlockCausal3D(cin if i == 0 else cout, cout) for i in range(layers)])
        self.upsamplers = nn.ModuleList([_Upsample(cout, factor)]) if factor else None

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        if self.upsamplers is not None:
            x = self.upsamplers[0](x)
        return x


class Encoder3D(nn.Module):
    def __init__(self, in_ch: int, latent_ch: int, chans: Sequence[int], layers: int, spatial_log2: int, temporal_log2: int):
        super().__init__()
        self.conv_in = CausalConv3d(in_ch, chans[0], 3)
        blocks = []
        c = chans[0]
        n = len(chans)
        for i, co in enumerate(chans):
            stride = None
            if i < n - 1:
                sp = 2 if i < spatial_log2 else 1
                tm = 2 if i >= n - 1 - temporal_log2 else 1
                stride = (tm, sp, sp)
            blocks.append(_DownBlock(c, co, layers, stride))
            c = co
        self.down_blocks = nn.ModuleList(blocks)
        self.mid_block = _MidBlock(c)
        self.conv_norm_out = nn.GroupNorm(32, c, eps=1e-6)
        self.conv_out = CausalConv3d(c, 2 * latent_ch, 3)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        x = self.mid_block(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class Decoder3D(nn.Module):
    def __init__(self, out_ch: int, latent_ch: int, chans: Sequence[int], layers: int, spatial_log2: int, temporal_log2: int):
        super().__init__()
        rev = list(reversed(chans))
        self.conv_in = CausalConv3d(latent_ch, rev[0], 3)
        self.mid_block = _MidBlock(rev[0])
        blocks = []
        c = rev[0]
        n = len(rev)
        for i, co in enumerate(rev):
            factor = None
            if i < n - 1:
                sp = 2 if i < spatial_log2 else 1
                tm = 2 if i >= n - 1 - temporal_log2 else 1
                factor = (tm, sp, sp)
            blocks.append(_UpBlock(c, co, layers + 1, factor))
            c = co
        self.up_blocks = nn.ModuleList(blocks)
        self.conv_norm_out = nn.GroupNorm(32, c, eps=1e-6)
        self.conv_out = CausalConv3d(c, out_ch, 3)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class AutoencoderKLHunyuanVideo(nn.Module):
    scaling_factor = 0.476986

    def __init__(self, in_channels: int = 3, latent_channels: int = 16, block_out_channels: Sequence[int] = (128, 256, 512, 512),
                 layers_per_block: int = 2, spatial_compression_ratio: int = 8, temporal_compression_ratio: int = 4):
        super().__init__()
        sl, tl = spatial_compression_ratio.bit_length() - 1, temporal_compression_ratio.bit_length() - 1
        self.encoder = Encoder3D(in_channels, latent_channels, block_out_channels, layers_per_block, sl, tl)
        self.decoder = Decoder3D(in_channels, latent_channels, block_out_channels, layers_per_block, sl, tl)
        self.quant_conv = nn.Conv3d(2 * latent_channels, 2 * latent_channels, 1)
        self.post_quant_conv = nn.Conv3d(latent_channels, latent_channels, 1)
        self.spatial_ratio, self.temporal_ratio = spatial_compression_ratio, temporal_compression_ratio
        self.use_slicing, self.use_tiling = True, False
        self.tile_sample_min = 256
        self.tile_overlap = 0.25

    def enable_tiling(self, on: bool = True):
        self.use_tiling = bool(on)

    def enable_slicing(self, on: bool = True):
        self.use_slicing = bool(on)

    # ---- encode -------------------------------------------------------------------------
    def _moments(self, x):
        return self.quant_conv(self.encoder(x))

    def _blend(self, a, b, extent, dim):
        extent = min(a.shape[dim], b.shape[dim], extent)
        if extent <= 0:
            return b
        w = torch.linspace(0, 1, extent, device=b.device, dtype=b.dtype)
        shape = [1] * b.dim()
        shape[dim] = extent
        w = w.view(shape)
        head = a.narrow(dim, a.shape[dim] - extent, extent) * (1 - w) + b.narrow(dim, 0, extent) * w
        return torch.cat([head, b.narrow(dim, extent, b.shape[dim] - extent)], dim=dim)

    def _tiled(self, x, fn, tile: int, ratio_in_out: float):
        """Apply ``fn`` on overlapping spatial tiles of ``x`` and blend the seams (sizes in ``x`` pixels)."""
        B, C, T, H, W = x.shape
        align = max(1, int(round(1.0 / ratio_in_out)))                 # keep tile strides on latent-pixel boundaries
        stride = max(align, int(tile * (1 - self.tile_overlap)) // align * align)
        blend = int(round((tile - stride) * ratio_in_out))
        keep = int(round(stride * ratio_in_out))
        rows = []
        for i in range(0, H, stride):
            row = []
            for j in range(0, W, stride):
                row.append(fn(x[:, :, :, i:i + tile, j:j + tile]))
            rows.append(row)
        out_rows = []
        for i, row in enumerate(rows):
            res = []
            for j, t in enumerate(row):
                if i > 0:
                    t = self._blend(rows[i - 1][j], t, blend, 3)
                if j > 0:
                    t = self._blend(row[j - 1], t, blend, 4)
                res.append(t[:, :, :, :keep if i < len(rows) - 1 else t.shape[3], :keep if j < len(row) - 1 else t.shape[4]])
            out_rows.append(torch.cat(res, dim=4))
        return torch.cat(out_rows, dim=3)

    def encode(self, x: torch.Tensor, sample: bool = True, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """``[B, 3, F, H, W]`` pixels in [-1, 1] -> latents ``[B, 16, (F-1)/4+1, H/8, W/8]`` (unscaled)."""
        def one(xx):
            if self.use_tiling and max(xx.shape[-2:]) > self.tile_sample_min:
                m = self._tiled(xx, self._moments, self.tile_sample_min, 1.0 / self.spatial_ratio)
            else:
                m = self._moments(xx)
            mean, logvar = m.chunk(2, dim=1)
            if not sample:
                return mean
            std = torch.exp(0.5 * logvar.clamp(-30.0, 20.0))
            return mean + std * torch.randn(mean.shape, device=mean.device, dtype=mean.dtype, generator=generator)
        if self.use_slicing and x.shape[0] > 1:
            return torch.cat([one(s) for s in x.split(1)], dim=0)
        return one(x)

    # ---- decode -------------------------------------------------------------------------
    def decode(self, z: torch.Tensor) -> torch.Tensor:
        def one(zz):
            f = lambda t: self.decoder(self.post_quant_conv(t))  # noqa: E731
            tile = self.tile_sample_min // self.spatial_ratio
            if self.use_tiling and max(zz.shape[-2:]) > tile:
                return self._tiled(zz, f, tile, float(self.spatial_ratio))
            return f(zz)
        if self.use_slicing and z.shape[0] > 1:
            return torch.cat([one(s) for s in z.split(1)], dim=0)
        return one(z)

    def forward(self, x):
        return self.decode(self.encode(x))
