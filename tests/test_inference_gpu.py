"""The sampling pipeline on a B200 with the sm_100a kernels (bf16 transformer with 128-wide heads): text -> video and
image -> video at a tiny size, written out as a video file; the library fallbacks are forbidden while it runs."""

import os

import pytest
import torch

pytestmark = pytest.mark.gpu


def _pipeline(in_channels: int, dev):
    from teletron_b200.inference.pipeline import HunyuanVideoPipeline
    from teletron_b200.models.hunyuanvideo import HunyuanVideoTransformer3DModel, tiny_config
    from teletron_b200.models.text_encoders import ClipTextEncoder, LlamaTextEncoder, clip_text_config, llama_config
    from teletron_b200.models.vae import AutoencoderKLHunyuanVideo
    torch.manual_seed(0)
    # two heads of 128 (the kernels' head size); RoPE axes sum to the head size
    cfg = tiny_config(in_channels=in_channels, hidden_size=256, num_attention_heads=2, attention_head_dim=128,
                      rope_axes_dim=(16, 56, 56), num_layers=1, num_single_layers=1)
    tr = HunyuanVideoTransformer3DModel(cfg, tp=1, device=dev, dtype=torch.bfloat16).eval()
    vae = AutoencoderKLHunyuanVideo(block_out_channels=(32, 32, 32, 32)).to(dev, torch.bfloat16).eval()
    llama = LlamaTextEncoder(max_length=24, device=dev, dtype=torch.float32, config=llama_config(2, 64, 4, 2, 128, 1000))
    clip = ClipTextEncoder(max_length=16, device=dev, dtype=torch.float32, config=clip_text_config(2, 32, 4, 500, 16))
    return HunyuanVideoPipeline(tr, vae, llama, clip)


def test_sampling_runs_on_the_native_kernels_and_writes_a_video(tmp_path):
    from teletron_b200.inference.video_io import export_to_video, read_avi_info
    from teletron_b200.ops import attention_backend, fallback, gemm
    dev = torch.device("cuda", 0)
    was = fallback.strict()
    fallback.set_strict(True)
    try:
        before = (gemm.COUNTERS["tcgen05"], attention_backend.COUNTERS["tcgen05"], attention_backend.COUNTERS["sdpa"])
        kw = dict(height=64, width=64, num_frames=5, num_inference_steps=2, max_sequence_length=16, guidance_scale=1.0)
        out = _pipeline(16, dev)("a red cube turns slowly", seed=3, **kw).frames
        assert out.shape == (1, 5, 3, 64, 64) and torch.isfinite(out.float()).all()
        assert float(out.min()) >= 0.0 and float(out.max()) <= 1.0
        again = _pipeline(16, dev)("a red cube turns slowly", seed=3, **kw).frames
        assert torch.equal(out, again)                    # deterministic kernels, seeded noise
        ref = torch.rand(1, 3, 64, 64, device=dev) * 2 - 1
        i2v = _pipeline(33, dev)("a boat", model_type="i2v", ref_images=ref, seed=5, **kw).frames
        assert i2v.shape == (1, 5, 3, 64, 64) and torch.isfinite(i2v.float()).all()
        after = (gemm.COUNTERS["tcgen05"], attention_backend.COUNTERS["tcgen05"], attention_backend.COUNTERS["sdpa"])
        assert after[0] > before[0] and after[1] > before[1], "the tcgen05 GEMM / attention kernels did not run"
        assert after[2] == before[2], "attention fell back to SDPA"
    finally:
        fallback.set_strict(was)
    path = export_to_video(out[0], str(tmp_path / "sample.avi"), fps=15)
    info = read_avi_info(path)
    assert (info["width"], info["height"], info["total_frames"]) == (64, 64, 5) and os.path.getsize(path) > 0
