"""Video generation entry point (counterpart of the reference's ``examples/hunyuanvideo/video_generation.py``):
same flags; the reference frame is read from an image tensor file (``.pt`` / ``.npy`` ``[3, H, W]`` in [0, 1]) and the
result is written as a tensor file, since no image / video codecs are bundled."""

import argparse
import os
import sys

sys.path.insert(0, os.path.abspath(os.path.join(os.path.dirname(__file__), "..", "..")))

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

from teletron_b200.inference import HunyuanVideoPipeline, save_video_tensor  # noqa: E402


def prepare_reference_images(width: int, height: int, num_frames: int, ref_image_path: str) -> torch.Tensor:
    """``[num_frames, 3, H, W]`` in [-1, 1] with only the first frame set from the input image."""
    ref = torch.full((num_frames, 3, height, width), -1.0)
    if ref_image_path:
        if ref_image_path.endswith(".npy"):
            import numpy as np
            img = torch.from_numpy(np.load(ref_image_path)).float()
        else:
            img = torch.load(ref_image_path).float()
        img = F.interpolate(img[None], size=(height, width), mode="bilinear", align_corners=False)[0]
        ref[0] = img * 2 - 1
    return ref


def main():
    p = argparse.ArgumentParser(description="Hunyuan Video Generation Script")
    p.add_argument("--width", type=int, default=1280)
    p.add_argument("--height", type=int, default=720)
    p.add_argument("--num_frames", type=int, default=49)
    p.add_argument("--num_inference_steps", type=int, default=50)
    p.add_argument("--base_model_path", type=str, default=None)
    p.add_argument("--transformer_model_path", type=str, default=None)
    p.add_argument("--ref_frame", type=str, default="")
    p.add_argument("--prompt", type=str, required=True)
    p.add_argument("--device", type=str, default="cuda:0")
    p.add_argument("--output_file", type=str, default="output.mp4")
    p.add_argument("--fps", type=float, default=15.0)
    p.add_argument("--seed", type=int, default=42)
    p.add_argument("--guidance_scale", type=float, default=4.0)
    p.add_argument("--embedded_guidance_scale", type=float, default=1.0)
    p.add_argument("--model_type", type=str, default="i2v", choices=["t2v", "i2v", "token_replace"])
    p.add_argument("--cfg_zero_star", action="store_true")
    a = p.parse_args()
    pipe = HunyuanVideoPipeline.from_pretrained(a.base_model_path, transformer_model_path=a.transformer_model_path,
                                                torch_dtype=torch.bfloat16, device=torch.device(a.device),
                                                in_channels=33 if a.model_type == "i2v" else 16)
    pipe.vae.enable_tiling()
    ref = prepare_reference_images(a.width, a.height, a.num_frames, a.ref_frame) if a.model_type != "t2v" else None
    out = pipe(prompt=a.prompt, height=a.height, width=a.width, num_frames=a.num_frames,
               num_inference_steps=a.num_inference_steps, seed=a.seed, model_type=a.model_type, ref_images=ref,
               guidance_scale=a.guidance_scale, embedded_guidance_scale=a.embedded_guidance_scale,
               cfg_zero_star=a.cfg_zero_star)
    written = save_video_tensor(out.frames[0], a.output_file, fps=a.fps)
    print(f"wrote {tuple(out.frames[0].shape)} frames to {written}")


if __name__ == "__main__":
    main()
