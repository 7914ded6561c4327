"""Writing generated frames as video files without depending on a media stack.

The reference ends its sampling script with diffusers' ``export_to_video(video, args.output_file, fps=15)``
(``examples/hunyuanvideo/video_generation.py:66``), which needs imageio / ffmpeg.  :func:`export_to_video` here picks
the container from the file name:

* ``.avi`` - written by this module itself as a RIFF / AVI 1.0 file: Motion-JPEG frames when Pillow is importable
  (any player opens these), otherwise uncompressed 24-bit frames; no other dependency.
* ``.mp4`` / ``.mov`` / ``.mkv`` - through OpenCV's ``VideoWriter`` when ``cv2`` is importable and its build can open the
  container; if not, the same frames are written next to the requested name as ``.avi`` and that path is returned.
* ``.gif`` - through Pillow.
* ``.npy`` / ``.pt`` - the raw ``uint8`` array / the float tensor.

Frames are ``[F, 3, H, W]`` or ``[F, H, W, 3]``, float in ``[0, 1]`` or ``uint8``.
"""

from __future__ import annotations

import io
import os
import struct
from typing import List, Optional

import numpy as np
import torch


def to_uint8_frames(frames) -> np.ndarray:
    """``[F, H, W, 3]`` uint8 RGB from a tensor / array in either channel order."""
    if isinstance(frames, (list, tuple)):
        frames = np.stack([np.asarray(f) for f in frames])
    if torch.is_tensor(frames):
        t = frames.detach()
        if t.is_floating_point():
            t = (t.float().clamp(0, 1) * 255).round().to(torch.uint8)
        frames = t.cpu().numpy()
    a = np.asarray(frames)
    if a.ndim != 4:
        raise ValueError(f"expected 4-D frames, got shape {a.shape}")
    if a.shape[1] == 3 and a.shape[-1] != 3:
        a = a.transpose(0, 2, 3, 1)
    if a.shape[-1] != 3:
        raise ValueError(f"frames must have 3 colour channels, got shape {a.shape}")
    if a.dtype != np.uint8:
        a = (np.clip(a.astype(np.float32), 0, 1) * 255).round().astype(np.uint8)
    return np.ascontiguousarray(a)


def _chunk(tag: bytes, payload: bytes) -> bytes:
    pad = b"\x00" if len(payload) & 1 else b""
    return tag + struct.pack("<I", len(payload)) + payload + pad


def _list(kind: bytes, payload: bytes) -> bytes:
    return b"LIST" + struct.pack("<I", len(payload) + 4) + kind + payload


def write_avi(path: str, frames: np.ndarray, fps: float = 15.0, mjpeg: Optional[bool] = None, quality: int = 92) -> str:
    """RIFF / AVI 1.0 with one video stream and an ``idx1`` index.  ``mjpeg=None`` uses JPEG frames when Pillow is
    there and raw BGR frames (bottom-up rows padded to 4 bytes, as a DIB wants them) otherwise."""
    n, h, w, _ = frames.shape
    if mjpeg is None:
        try:
            import PIL.Image  # noqa: F401
            mjpeg = True
        except Exception:
            mjpeg = False
    payloads: List[bytes] = []
    if mjpeg:
        from PIL import Image
        for f in frames:
            buf = io.BytesIO()
            Image.fromarray(f, "RGB").save(buf, format="JPEG", quality=quality)
            payloads.append(buf.getvalue())
        handler, compression, bits = b"MJPG", b"MJPG", 24
    else:
        stride = (w * 3 + 3) & ~3
        for f in frames:
            rows = np.zeros((h, stride), dtype=np.uint8)
            rows[:, :w * 3] = f[::-1, :, ::-1].reshape(h, w * 3)       # bottom-up, BGR
            payloads.append(rows.tobytes())
        handler, compression, bits = b"DIB ", struct.pack("<I", 0), 24
    largest = max(len(p) for p in payloads) if payloads else 0
    usec = int(round(1e6 / fps))
    rate, scale = int(round(fps * 1000)), 1000
    avih = struct.pack("<IIIIIIIIII4I", usec, int(largest * fps), 0, 0x10, n, 0, 1, largest, w, h, 0, 0, 0, 0)
    strh = b"vids" + handler + struct.pack("<IHHIIIIIIII4h", 0, 0, 0, 0, scale, rate, 0, n, largest, 0xFFFFFFFF, 0, 0, 0, w, h)
    strf = struct.pack("<IiiHH4sIiiII", 40, w, h, 1, bits, compression, largest, 0, 0, 0, 0)
    hdrl = _list(b"hdrl", _chunk(b"avih", avih) + _list(b"strl", _chunk(b"strh", strh) + _chunk(b"strf", strf)))
    movi_body, index, off = b"", b"", 4
    parts = []
    for p in payloads:
        c = _chunk(b"00dc", p)
        parts.append(c)
        index += b"00dc" + struct.pack("<III", 0x10, off, len(p))
        off += len(c)
    movi_body = b"".join(parts)
    body = b"AVI " + hdrl + _list(b"movi", movi_body) + _chunk(b"idx1", index)
    with open(path, "wb") as fh:
        fh.write(b"RIFF" + struct.pack("<I", len(body)) + body)
    return path


def read_avi_info(path: str) -> dict:
    """Header fields and frame payloads of a file written by :func:`write_avi` (enough to check or decode it)."""
    data = open(path, "rb").read()
    if data[:4] != b"RIFF" or data[8:12] != b"AVI ":
        raise ValueError("not an AVI file")
    info = {"frames": []}

    def walk(lo: int, hi: int):
        pos = lo
        while pos + 8 <= hi:
            tag, size = data[pos:pos + 4], struct.unpack("<I", data[pos + 4:pos + 8])[0]
            body = pos + 8
            if tag == b"LIST":
                walk(body + 4, body + size)
            elif tag == b"avih":
                usec, _, _, _, total, _, _, _, w, h = struct.unpack("<10I", data[body:body + 40])
                info.update(usec_per_frame=usec, total_frames=total, width=w, height=h)
            elif tag == b"strh":
                info["handler"] = data[body + 4:body + 8]
                info["scale"], info["rate"] = struct.unpack("<II", data[body + 20:body + 28])
            elif tag == b"strf":
                info["bits"] = struct.unpack("<H", data[body + 14:body + 16])[0]
                info["compression"] = data[body + 16:body + 20]
            elif tag == b"00dc":
                info["frames"].append(data[body:body + size])
            elif tag == b"idx1":
                info["index_entries"] = size // 16
            pos = body + size + (size & 1)
    walk(12, len(data))
    return info


def export_to_video(frames, output_video_path: str, fps: float = 15.0) -> str:
    """Write the frames; returns the path actually written (it differs from the requested one only when an ``.mp4``
    was asked for and no installed library can produce one)."""
    ext = os.path.splitext(output_video_path)[1].lower()
    if ext == ".pt":
        torch.save(frames.cpu() if torch.is_tensor(frames) else torch.as_tensor(np.asarray(frames)), output_video_path)
        return output_video_path
    a = to_uint8_frames(frames)
    if ext == ".npy":
        np.save(output_video_path, a)
        return output_video_path
    if ext == ".gif":
        from PIL import Image
        imgs = [Image.fromarray(f, "RGB") for f in a]
        imgs[0].save(output_video_path, save_all=True, append_images=imgs[1:], duration=int(round(1000 / fps)), loop=0)
        return output_video_path
    if ext == ".avi":
        return write_avi(output_video_path, a, fps)
    try:
        import cv2
        writer = cv2.VideoWriter(output_video_path, cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (a.shape[2], a.shape[1]))
        if writer.isOpened():
            for f in a:
                writer.write(np.ascontiguousarray(f[:, :, ::-1]))
            writer.release()
            if os.path.isfile(output_video_path) and os.path.getsize(output_video_path) > 0:
                return output_video_path
    except Exception:
        pass
    alt = os.path.splitext(output_video_path)[0] + ".avi"
    print(f"no library here can write {ext}; writing {alt} instead")
    return write_avi(alt, a, fps)
