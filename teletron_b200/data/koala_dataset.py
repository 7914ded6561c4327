"""Video-clip dataset driven by a YAML option file and a ``;``-separated annotation file.

Behavioural parity with ``teletron/datasets/koala_dataset.py:607-707``: the option file has
``data.test-data.args`` with ``anno_file``, ``data_prefix``, ``phase`` and ``sample_types``; frame count
and resolution of every sample type are overridden from ``--num-frames`` / ``--video-resolution``;
annotation lines are ``path;prompt;prompt_embeds;clip_text_embed;latents`` with Python-literal
tensors; frames are temporally sampled by fragment samplers (``:416-547``), spatially sampled as
grid "fragments" (``:122-226``), normalised with ImageNet mean / std and returned as
``images [F, 3, H, W]`` plus the text / latent fields.

Decoding uses ``decord`` when it is installed, else OpenCV; clips may also be stored as ``.pt`` / ``.npy`` uint8 arrays
``[T, H, W, 3]``, which is what most unit tests use.  The reference's quirks are not kept:
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


class UnifiedFrameSampler:
    """``fragments_t`` temporal cells, ``fsize_t`` frames (``frame_interval`` apart) from a random offset inside each
    cell, optionally dropping a share of the cells; indices wrap around the clip (``koala_dataset.py:45-94``)."""

    def __init__(self, fsize_t: int, fragments_t: int, frame_interval: int = 1, num_clips: int = 1, drop_rate: float = 0.0):
        self.fsize_t, self.fragments_t = fsize_t, fragments_t
        self.size_t = fragments_t * fsize_t
        self.frame_interval, self.num_clips, self.drop_rate = frame_interval, num_clips, drop_rate

    def get_frame_indices(self, num_frames: int, train: bool = False) -> np.ndarray:
        cell = num_frames // self.fragments_t
        starts = np.arange(self.fragments_t, dtype=np.int64) * cell
        span = self.fsize_t * self.frame_interval
        offs = np.random.randint(0, cell - span, size=self.fragments_t) if cell > span else np.zeros(self.fragments_t, dtype=np.int64)
        ranges = np.arange(self.fsize_t)[None, :] * self.frame_interval + offs[:, None] + starts[:, None]
        dropped = set(random.sample(range(self.fragments_t), int(self.fragments_t * self.drop_rate)))
        return np.concatenate([r for i, r in enumerate(ranges) if i not in dropped])

    def __call__(self, total_frames: int, train: bool = False, start_index: int = 0) -> np.ndarray:
        inds = np.concatenate([self.get_frame_indices(total_frames, train) for _ in range(self.num_clips)])
        return np.mod(inds + start_index, total_frames).astype(np.int32)


class SimpleFrameSampler:
    """Evenly spread frames including the first and the last one (one frame: the middle; two: first and middle),
    ``koala_dataset.py:97-119``."""

    def __init__(self, fsize_t: int):
        self.fsize_t = fsize_t

    def __call__(self, total_frames: int, train: bool = False, start_index: int = 0) -> np.ndarray:
        n = self.fsize_t
        if n == 1:
            inds = [total_frames // 2]
        elif n == 2:
            inds = [0, total_frames // 2]
        else:
            step = total_frames // (n - 1)
            inds = [0] + [step * (i + 1) for i in range(n - 2)] + [total_frames - 1]
        return np.asarray(inds, dtype=np.int32)


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


def _random_square_crop(video: torch.Tensor) -> torch.Tensor:
    """Random crop of ``[..., H, W]`` to a square of the short edge (training-time augmentation of the aspect-ratio
    preserving sample types; the reference's version indexes the wrong axis for wide clips, ``koala_dataset.py:266-268``)."""
    H, W = video.shape[-2:]
    e = min(H, W)
    if H > e:
        o = random.randrange(H - e)
        return video[..., o:o + e, :]
    if W > e:
        o = random.randrange(W - e)
        return video[..., :, o:o + e]
    return video


def get_arp_resized_video(video: torch.Tensor, short_edge: int = 224, train: bool = False, **_unused) -> torch.Tensor:
    """Resize ``[C, T, H, W]`` so that the short edge becomes ``short_edge``, keeping the aspect ratio (training: after a
    random square crop)."""
    if train:
        video = _random_square_crop(video)
    scale = short_edge / min(video.shape[-2:])
    out = F.interpolate(video.permute(1, 0, 2, 3).float(), scale_factor=scale, mode="bilinear", align_corners=False)
    return out.permute(1, 0, 2, 3).to(video.dtype) if video.dtype.is_floating_point else out.permute(1, 0, 2, 3)


def get_arp_fragment_video(video: torch.Tensor, short_fragments: int = 7, fsize: int = 32, train: bool = False,
                           **kwargs) -> torch.Tensor:
    """Grid fragments with ``short_fragments`` cells along the short edge and proportionally more along the long one."""
    if train:
        video = _random_square_crop(video)
    H, W = video.shape[-2:]
    if H > W:
        fh, fw = int(short_fragments * H / W), short_fragments
    else:
        fh, fw = short_fragments, int(short_fragments * W / H)
    kwargs.pop("fragments_h", None)
    kwargs.pop("fragments_w", None)
    return get_spatial_fragments(video, fragments_h=fh, fragments_w=fw, fsize_h=fsize, fsize_w=fsize, **kwargs)


def get_cropped_video(video: torch.Tensor, size_h: int = 224, size_w: int = 224, **kwargs) -> torch.Tensor:
    """One ``size_h x size_w`` window (centre, or random with ``random=True``): a 1 x 1 fragment grid."""
    for k in ("fragments_h", "fragments_w", "fsize_h", "fsize_w"):
        kwargs.pop(k, None)
    return get_spatial_fragments(video, fragments_h=1, fragments_w=1, fsize_h=size_h, fsize_w=size_w, **kwargs)


def get_single_sample(video: torch.Tensor, sample_type: str, random: bool = False, **kwargs) -> torch.Tensor:
    """Dispatch on the sample-type prefix (``koala_dataset.py:315-337``).  ``arp_*`` must be tested before their
    un-prefixed namesakes; the reference tests ``resize`` first, so its ``arp_resize`` branch is dead."""
    if sample_type.startswith("arp_resize"):
        return get_arp_resized_video(video, **kwargs)
    if sample_type.startswith("arp_fragments"):
        return get_arp_fragment_video(video, random=random, **kwargs)
    if sample_type.startswith(("resize", "image", "semantic")):
        return get_resized_video(video, **kwargs)
    if sample_type.startswith("fragments"):
        return get_spatial_fragments(video, random=random, **kwargs)
    if sample_type.startswith("crop"):
        return get_cropped_video(video, random=random, **kwargs)
    if sample_type.startswith("original"):
        return video
    raise ValueError(f"unknown sample type {sample_type}")


def get_spatial_samples(video: torch.Tensor, random_crop: int = 0, sample_types: Optional[Dict[str, dict]] = None) -> Dict[str, torch.Tensor]:
    """All spatial views of one decoded clip ``[C, T, H, W]``.  ``random_crop`` 1: random window of 80-100 % keeping the
    aspect ratio, then up-scaled by 1.0-1.3; 2: random near-square window of 80-100 % of the short edge
    (``koala_dataset.py:339-371``, whose mode 1 references an undefined name)."""
    H, W = video.shape[-2:]
    if random_crop == 1:
        r = random.random() * 0.2 + 0.8
        nh, nw = int(r * H), int(r * W)
        oh, ow = random.randrange(max(H - nh, 1)), random.randrange(max(W - nw, 1))
        video = video[..., oh:oh + nh, ow:ow + nw]
        up = random.random() * 0.3 + 1.0
        scaled = F.interpolate(video.permute(1, 0, 2, 3).float(), scale_factor=up, mode="bilinear", align_corners=False)
        video = scaled.permute(1, 0, 2, 3).to(video.dtype) if video.dtype.is_floating_point else scaled.permute(1, 0, 2, 3)
    elif random_crop == 2:
        r = random.random() * 0.2 + 0.8
        n = int(r * min(H, W))
        oh, ow = random.randrange(max(H - n, 1)), random.randrange(max(W - n, 1))
        video = video[..., oh:oh + n, ow:ow + n]
    sample_types = sample_types if sample_types is not None else {"resize": {}, "fragments": {}}
    return {name: get_single_sample(video, name, **(opt or {})) for name, opt in sample_types.items()}


def _decord():
    try:
        import decord  # type: ignore
        return decord
    except ImportError:
        return None


def _cv2_read(path: str, frame_indices: Optional[np.ndarray]) -> torch.Tensor:
    """Decode with OpenCV: the requested frames in one forward pass over the file (seeking per frame is slow and, with
    some codecs, inexact)."""
    import cv2
    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise RuntimeError(f"cannot open {path}")
    try:
        total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        frames = []
        if frame_indices is None:
            while True:
                ok, f = cap.read()
                if not ok:
                    break
                frames.append(f[:, :, ::-1])
            return torch.from_numpy(np.ascontiguousarray(np.stack(frames)))
        if total <= 0:
            raise RuntimeError(f"{path}: the container does not report a frame count")
        want = np.mod(np.asarray(frame_indices), total)
        last, pos, cache = int(want.max()), 0, {}
        needed = set(int(i) for i in want)
        while pos <= last:
            ok, f = cap.read()
            if not ok:
                break
            if pos in needed:
                cache[pos] = f[:, :, ::-1]
            pos += 1
        if len(cache) < len(needed):       # a container that reports more frames than it holds: repeat the last one
            tail = cache[max(cache)] if cache else None
            if tail is None:
                raise RuntimeError(f"{path}: no frame could be decoded")
            for i in needed - set(cache):
                cache[i] = tail
        return torch.from_numpy(np.ascontiguousarray(np.stack([cache[int(i)] for i in want])))
    finally:
        cap.release()


def read_video(path: str, frame_indices: Optional[np.ndarray] = None) -> torch.Tensor:
    """``[T, H, W, 3]`` uint8 RGB frames (all, or the requested indices).  ``.pt`` / ``.npy`` hold the array itself;
    container files (``.mp4``, ``.avi``, ...) are decoded with ``decord`` as the reference does
    (``koala_dataset.py``), or with OpenCV when ``decord`` is not installed."""
    ext = os.path.splitext(path)[1].lower()
    if ext == ".pt":
        v = torch.load(path)
    elif ext == ".npy":
        v = torch.from_numpy(np.load(path))
    else:
        decord = _decord()
        if decord is not None:
            vr = decord.VideoReader(path)
            idx = list(range(len(vr))) if frame_indices is None else np.mod(frame_indices, len(vr)).tolist()
            return torch.from_numpy(vr.get_batch(idx).asnumpy())
        try:
            import cv2  # noqa: F401
        except ImportError as e:
            raise RuntimeError(f"decoding {path} needs `decord` or OpenCV, neither is installed; "
                               "store clips as .pt / .npy uint8 [T,H,W,3]") from e
        return _cv2_read(path, frame_indices)
    if frame_indices is not None:
        v = v[torch.from_numpy(np.mod(frame_indices, v.shape[0]))]
    return v


def video_num_frames(path: str) -> int:
    ext = os.path.splitext(path)[1].lower()
    if ext in (".pt", ".npy"):
        return int(read_video(path).shape[0])
    decord = _decord()
    if decord is not None:
        return len(decord.VideoReader(path))
    import cv2
    cap = cv2.VideoCapture(path)
    try:
        n = int(cap.get(cv2.CAP_PROP_FRAME_COUNT)) if cap.isOpened() else 0
    finally:
        cap.release()
    if n <= 0:
        raise RuntimeError(f"cannot read the frame count of {path}")
    return n


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


@DATASETS.register_module()
class SimpleDataset(Dataset):
    """Labelled clips with one sample type (``koala_dataset.py:549-604``): ``opt`` carries ``anno_file`` (a path whose
    lines are ``filename,_,_,label``, or a ready list of ``{"filename", "label"}``), ``data_prefix``, ``sample_type``,
    ``sampling_args``, ``phase``, ``clip_len``, ``frame_interval`` and ``num_clips``."""

    def __init__(self, opt: dict):
        self.opt = opt
        self.sample_type, self.phase = opt["sample_type"], opt["phase"]
        self.sampler = SampleFrames(opt["clip_len"], opt["frame_interval"], opt["num_clips"])
        ann = opt["anno_file"]
        if isinstance(ann, list):
            self.video_infos = list(ann)
        else:
            self.video_infos = []
            with open(ann) as f:
                for line in f:
                    if not line.strip():
                        continue
                    name, _, _, label = line.strip().split(",")
                    self.video_infos.append({"filename": os.path.join(opt["data_prefix"], name), "label": float(label)})

    def __len__(self):
        return len(self.video_infos)

    def __getitem__(self, index: int):
        info = self.video_infos[index]
        inds = self.sampler(video_num_frames(info["filename"]), self.phase == "train")
        video = read_video(info["filename"], inds).permute(3, 0, 1, 2).float()            # [C, T, H, W]
        video = get_single_sample(video, self.sample_type, **self.opt.get("sampling_args", {}))
        video = ((video.permute(1, 2, 3, 0) - IMAGENET_MEAN) / IMAGENET_STD).permute(3, 0, 1, 2)
        return {"video": video, "num_clips": self.opt["num_clips"], "frame_inds": inds, "gt_label": info["label"],
                "name": os.path.basename(info["filename"])}


def seed_worker(worker_id: int) -> None:
    s = torch.initial_seed() % 2 ** 32
    np.random.seed(s)
    random.seed(s)
