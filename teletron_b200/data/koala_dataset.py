"""Video-clip dataset driven by a YAML option file and a ``;``-separated annotation file.

Behavioural parity with ``teletron/datasets/koala_dataset.py:607-707``: the option file has
``data.test-data.args`` with ``anno_file``, ``data_prefix``, ``phase`` and ``sample_types``; frame count
and resolution of every sample type are overridden from ``--num-frames`` / ``--video-resolution``;
annotation lines are ``path;prompt;prompt_embeds;clip_text_embed;latents`` with Python-literal
tensors; frames are temporally sampled by fragment samplers (``:416-547``), spatially sampled as
grid "fragments" (``:122-226``), normalised with ImageNet mean / std and returned as
``images [F, 3, H, W]`` plus the text / latent fields.

Decoding uses ``decord`` when it is installed; otherwise clips stored as ``.pt`` / ``.npy`` uint8 arrays
``[T, H, W, 3]`` are read, which is also what the unit tests use.  The reference's quirks are not kept:
length is the number of annotation entries times ``repeat`` (the reference indexes ``% 9`` with a
fixed length of 100000, ``:682, 706-707``).
"""

from __future__ import annotations

import ast
import os
import random
from typing import Dict, List, Optional

import numpy as np
import torch
import torch.nn.functional as F
import yaml
from torch.utils.data import Dataset

from .registry import DATASETS

IMAGENET_MEAN = torch.tensor([123.675, 116.28, 103.53])
IMAGENET_STD = torch.tensor([58.395, 57.12, 57.375])


class SampleFrames:
    """``num_clips`` clips of ``clip_len`` frames at ``frame_interval`` (train: random offsets;
    test: evenly spaced), wrapping around short videos."""

    def __init__(self, clip_len: int, frame_interval: int = 1, num_clips: int = 1):
        self.clip_len, self.frame_interval, self.num_clips = clip_len, frame_interval, num_clips

    def _offsets(self, num_frames: int, train: bool) -> np.ndarray:
        ori = self.clip_len * self.frame_interval
        avg = (num_frames - ori + 1) // self.num_clips
        if train:
            if avg > 0:
                return np.arange(self.num_clips) * avg + np.random.randint(avg, size=self.num_clips)
            if num_frames > max(self.num_clips, ori):
                return np.sort(np.random.randint(num_frames - ori + 1, size=self.num_clips))
            return np.zeros(self.num_clips, dtype=np.int64)
        if num_frames > ori - 1:
            step = (num_frames - ori + 1) / float(self.num_clips)
            return (np.arange(self.num_clips) * step + step / 2.0).astype(np.int64)
        return np.zeros(self.num_clips, dtype=np.int64)

    def __call__(self, total_frames: int, train: bool = False, start_index: int = 0) -> np.ndarray:
        off = self._offsets(total_frames, train)
        idx = off[:, None] + np.arange(self.clip_len)[None, :] * self.frame_interval
        idx = np.mod(idx.reshape(-1), max(total_frames, 1))
        return idx.astype(np.int64) + start_index


class FragmentSampleFrames:
    """Temporal fragments: the video is cut into ``fragments_t`` equal spans and ``fsize_t`` consecutive
    (strided) frames are taken from each, at a random (train) or centred (test) offset."""

    def __init__(self, fsize_t: int, fragments_t: int, frame_interval: int = 1, num_clips: int = 1,
                 drop_rate: float = 0.0):
        self.fsize_t, self.fragments_t = fsize_t, fragments_t
        self.size_t = fsize_t * fragments_t
        self.frame_interval, self.num_clips, self.drop_rate = frame_interval, num_clips, drop_rate

    def get_frame_indices(self, num_frames: int, train: bool = False) -> np.ndarray:
        tgrids = np.array([num_frames // self.fragments_t * i for i in range(self.fragments_t)], dtype=np.int64)
        tlength = num_frames // self.fragments_t
        span = self.fsize_t * self.frame_interval
        if tlength > span:
            if train:
                rnd = np.random.randint(0, tlength - span, size=len(tgrids))
            else:
                rnd = np.full(len(tgrids), (tlength - span) // 2, dtype=np.int64)
        else:
            rnd = np.zeros(len(tgrids), dtype=np.int64)
        ranges = np.arange(self.fsize_t)[None, :] * self.frame_interval + rnd[:, None] + tgrids[:, None]
        if self.drop_rate > 0 and train:
            keep = np.random.rand(self.fragments_t) >= self.drop_rate
            if keep.any():
                ranges = ranges[keep]
        return ranges.reshape(-1)

    def __call__(self, total_frames: int, train: bool = False, start_index: int = 0) -> np.ndarray:
        idx = np.concatenate([self.get_frame_indices(total_frames, train) for _ in range(self.num_clips)])
        return np.mod(idx, max(total_frames, 1)).astype(np.int64) + start_index


def get_spatial_fragments(video: torch.Tensor, fragments_h: int = 1, fragments_w: int = 1, fsize_h: int = 720,
                          fsize_w: int = 1280, aligned: int = 1, random: bool = False, **_unused) -> torch.Tensor:
    """Grid mini-patch sampling on ``[C, T, H, W]``: one ``fsize`` patch from each cell of a
    ``fragments_h x fragments_w`` grid, stitched together; patch offsets are shared by groups of
    ``aligned`` frames.  Videos smaller than the target are up-scaled first."""
    C, T, H, W = video.shape
    size_h, size_w = fragments_h * fsize_h, fragments_w * fsize_w
    ratio = min(H / size_h, W / size_w)
    if ratio < 1:
        video = F.interpolate(video.float(), scale_factor=(1 / ratio, 1 / ratio), mode="bilinear").to(video.dtype) \
            if video.dim() == 4 else video
        C, T, H, W = video.shape
    hgrids = torch.tensor([min(H // fragments_h * i, H - fsize_h) for i in range(fragments_h)])
    wgrids = torch.tensor([min(W // fragments_w * i, W - fsize_w) for i in range(fragments_w)])
    hlen, wlen = H // fragments_h, W // fragments_w
    groups = max(T // aligned, 1)
    if random and hlen > fsize_h:
        rnd_h = torch.randint(hlen - fsize_h, (fragments_h, fragments_w, groups))
    else:
        rnd_h = torch.full((fragments_h, fragments_w, groups), max((hlen - fsize_h) // 2, 0))
    if random and wlen > fsize_w:
        rnd_w = torch.randint(wlen - fsize_w, (fragments_h, fragments_w, groups))
    else:
        rnd_w = torch.full((fragments_h, fragments_w, groups), max((wlen - fsize_w) // 2, 0))
    out = torch.zeros(C, T, size_h, size_w, dtype=video.dtype)
    for i, hs in enumerate(hgrids.tolist()):
        for j, ws in enumerate(wgrids.tolist()):
            for t in range(groups):
                t0, t1 = t * aligned, (min((t + 1) * aligned, T) if t < groups - 1 else T)
                h0 = min(hs + int(rnd_h[i, j, t]), H - fsize_h)
                w0 = min(ws + int(rnd_w[i, j, t]), W - fsize_w)
                out[:, t0:t1, i * fsize_h:(i + 1) * fsize_h, j * fsize_w:(j + 1) * fsize_w] = \
                    video[:, t0:t1, h0:h0 + fsize_h, w0:w0 + fsize_w]
    return out


def get_resized_video(video: torch.Tensor, size_h: int = 224, size_w: int = 224, **_unused) -> torch.Tensor:
    """Bilinear resize of ``[C, T, H, W]`` to ``size_h x size_w``."""
    v = video.permute(1, 0, 2, 3).float()
    return F.interpolate(v, size=(size_h, size_w), mode="bilinear", align_corners=False).permute(1, 0, 2, 3)


def get_single_sample(video: torch.Tensor, sample_type: str, random: bool = False, **kwargs) -> torch.Tensor:
    if sample_type.startswith("resize"):
        return get_resized_video(video, **kwargs)
    if sample_type.startswith("fragments"):
        return get_spatial_fragments(video, random=random, **kwargs)
    if sample_type.startswith("original"):
        return video
    raise ValueError(f"unknown sample type {sample_type}")


def read_video(path: str, frame_indices: Optional[np.ndarray] = None) -> torch.Tensor:
    """``[T, H, W, 3]`` uint8 frames (all, or the requested indices)."""
    ext = os.path.splitext(path)[1].lower()
    if ext == ".pt":
        v = torch.load(path)
    elif ext == ".npy":
        v = torch.from_numpy(np.load(path))
    else:
        try:
            import decord  # type: ignore
        except ImportError as e:
            raise RuntimeError(f"decoding {path} needs the `decord` package, which is not installed; "
                               "store clips as .pt / .npy uint8 [T,H,W,3] or install decord") from e
        vr = decord.VideoReader(path)
        idx = list(range(len(vr))) if frame_indices is None else np.mod(frame_indices, len(vr)).tolist()
        return torch.from_numpy(vr.get_batch(idx).asnumpy())
    if frame_indices is not None:
        v = v[torch.from_numpy(np.mod(frame_indices, v.shape[0]))]
    return v


def video_num_frames(path: str) -> int:
    ext = os.path.splitext(path)[1].lower()
    if ext in (".pt", ".npy"):
        return int(read_video(path).shape[0])
    import decord  # type: ignore
    return len(decord.VideoReader(path))


def get_spatial_and_temporal_samples(path: str, sample_types: Dict[str, dict], samplers: Dict[str, object],
                                     is_train: bool = False, augment: bool = False) -> Dict[str, torch.Tensor]:
    total = video_num_frames(path)
    out = {}
    for stype, sopt in sample_types.items():
        idx = samplers[stype](total, is_train)
        frames = read_video(path, idx)                        # [T, H, W, 3]
        video = frames.permute(3, 0, 1, 2).float()           # [C, T, H, W]
        out[stype] = get_single_sample(video, stype, random=is_train and augment, **sopt)
    return out


def parse_annotation_line(line: str) -> dict:
    path, prompt, pe, ce, lat = line.rstrip("\n").split(";")
    return {"file_path": path, "prompt": prompt,
            "prompt_embeds": torch.tensor(ast.literal_eval(pe)).float(),
            "clip_text_embed": torch.tensor(ast.literal_eval(ce)).float(),
            "latents": torch.tensor(ast.literal_eval(lat)).to(torch.bfloat16).squeeze(0)}


@DATASETS.register_module()
class KoalaDataset(Dataset):
    def __init__(self, koala_opt: Optional[str] = None, num_frames: Optional[int] = None,
                 video_resolution=None, opt: Optional[dict] = None, repeat: int = 1, **_unused):
        if opt is None:
            if koala_opt is None:
                raise ValueError("KoalaDataset needs --koala-opt <yaml> (or an `opt` dict)")
            with open(koala_opt) as f:
                opt = yaml.safe_load(f)["data"]["test-data"]["args"]
        self.opt = opt
        for sopt in opt["sample_types"].values():
            if num_frames is not None:
                sopt["clip_len"] = int(num_frames)
            if video_resolution is not None:
                sopt["fsize_w"], sopt["fsize_h"] = int(video_resolution[0]), int(video_resolution[1])
        self.sample_types = opt["sample_types"]
        self.data_prefix = opt.get("data_prefix", "")
        self.phase = opt.get("phase", "test")
        self.augment = bool(opt.get("augment", False))
        self.repeat = repeat
        self.samplers = {}
        self._spatial = {}
        for stype, sopt in self.sample_types.items():
            t_frag = sopt.get("t_frag", 1)
            self.samplers[stype] = FragmentSampleFrames(sopt["clip_len"] // t_frag, t_frag,
                                                        sopt.get("frame_interval", 1), sopt.get("num_clips", 1))
            self._spatial[stype] = {k: v for k, v in sopt.items()
                                    if k not in ("clip_len", "frame_interval", "num_clips", "t_frag")}
        ann = opt["anno_file"]
        if isinstance(ann, list):
            self.video_infos: List[dict] = ann
        else:
            with open(ann) as f:
                self.video_infos = [parse_annotation_line(l) for l in f if l.strip()]
        if not self.video_infos:
            raise ValueError("empty annotation file")

    def __len__(self):
        return len(self.video_infos) * self.repeat

    def __getitem__(self, index: int):
        info = self.video_infos[index % len(self.video_infos)]
        path = info["file_path"]
        if not os.path.isabs(path):
            path = os.path.join(self.data_prefix, path)
        data = get_spatial_and_temporal_samples(path, self._spatial, self.samplers, self.phase == "train",
                                                self.augment and self.phase == "train")
        frames = data[next(iter(data))]                                       # [C, T, H, W]
        frames = ((frames.permute(1, 2, 3, 0) - IMAGENET_MEAN) / IMAGENET_STD).permute(0, 3, 1, 2)   # [T, C, H, W]
        return {"images": frames, "first_ref_image": frames[0], "prompt": info["prompt"],
                "prompt_embeds": info["prompt_embeds"], "clip_text_embed": info["clip_text_embed"],
                "latents": info["latents"]}


def seed_worker(worker_id: int) -> None:
    s = torch.initial_seed() % 2 ** 32
    np.random.seed(s)
    random.seed(s)
