"""Sampling pipeline (text / image -> video), I2V training input and batch distribution on CPU with tiny components."""

import os

import pytest
import torch

from dist_utils import run_distributed


def _pipeline(in_channels: int):
    from teletron_b200.inference.pipeline import HunyuanVideoPipeline
    from teletron_b200.models.hunyuanvideo import HunyuanVideoTransformer3DModel, tiny_config
    from teletron_b200.models.text_encoders import ClipTextEncoder, LlamaTextEncoder, clip_text_config, llama_config
    from teletron_b200.models.vae import AutoencoderKLHunyuanVideo
    torch.manual_seed(0)
    cfg = tiny_config(in_channels=in_channels)
    tr = HunyuanVideoTransformer3DModel(cfg, tp=1, dtype=torch.float32).eval()
    vae = AutoencoderKLHunyuanVideo(block_out_channels=(32, 32, 32, 32)).eval()
    llama = LlamaTextEncoder(max_length=24, dtype=torch.float32, config=llama_config(2, 64, 4, 2, 128, 1000))
    clip = ClipTextEncoder(max_length=16, dtype=torch.float32, config=clip_text_config(2, 32, 4, 500, 16))
    return HunyuanVideoPipeline(tr, vae, llama, clip)


def test_t2v_sampling_shapes_seed_and_guidance():
    pipe = _pipeline(16)
    kw = dict(height=32, width=32, num_frames=5, num_inference_steps=2, max_sequence_length=16)
    a = pipe("a red cube turns slowly", guidance_scale=1.0, seed=3, **kw).frames
    assert a.shape == (1, 5, 3, 32, 32) and float(a.min()) >= 0.0 and float(a.max()) <= 1.0
    b = pipe("a red cube turns slowly", guidance_scale=1.0, seed=3, **kw).frames
    assert torch.equal(a, b)                                   # same seed, same video
    c = pipe("a red cube turns slowly", guidance_scale=1.0, seed=4, **kw).frames
    assert not torch.equal(a, c)
    lat = pipe("a red cube turns slowly", guidance_scale=1.0, seed=3, output_type="latent", **kw).frames
    assert lat.shape == (1, 16, 2, 4, 4)
    # true classifier-free guidance runs the transformer twice per step; with the zero-star rule the first two steps
    # contribute nothing, so two steps return the initial noise
    noise = torch.randn(1, 16, 2, 4, 4, generator=torch.Generator().manual_seed(9))
    cfg = pipe("a red cube", negative_prompt="blurry", guidance_scale=6.0, cfg_zero_star=True, latents=noise.clone(),
               output_type="latent", **kw).frames
    torch.testing.assert_close(cfg, noise)
    plain = pipe("a red cube", negative_prompt="blurry", guidance_scale=6.0, latents=noise.clone(), output_type="latent", **kw).frames
    assert not torch.allclose(plain, noise)
    seen = []
    pipe("a red cube", guidance_scale=1.0, seed=1, output_type="latent",
         callback_on_step_end=lambda p, i, t, d: seen.append((i, float(t[0]))), **kw)
    assert [i for i, _ in seen] == [0, 1] and seen[0][1] == pytest.approx(1000.0) and seen[1][1] < 1000.0


def test_i2v_and_token_replace_conditioning():
    kw = dict(height=32, width=32, num_frames=9, num_inference_steps=2, max_sequence_length=16, guidance_scale=1.0,
              output_type="latent", seed=5)
    ref = torch.rand(2, 3, 32, 32) * 2 - 1
    # image-to-video: the first-frame latent and a mask channel are concatenated to the noisy latent (33 channels in)
    i2v = _pipeline(33)
    out = i2v("a boat", model_type="i2v", ref_images=ref, **kw).frames
    assert out.shape == (1, 16, 3, 4, 4) and torch.isfinite(out).all()
    with pytest.raises(ValueError):
        i2v("a boat", model_type="i2v", **kw)
    # token replace: the first (and optionally last) latent frame is pinned to the encoded reference after every step
    t2v = _pipeline(16)
    steps = []
    out = t2v("a boat", model_type="token_replace", ref_images=ref, first_last=True,
              callback_on_step_end=lambda p, i, t, d: steps.append(d["latents"].clone()), **kw).frames
    assert len(steps) == 2
    torch.testing.assert_close(steps[0][:, :, :1], out[:, :, :1], rtol=0, atol=0)
    torch.testing.assert_close(steps[0][:, :, -1:], out[:, :, -1:], rtol=0, atol=0)
    assert not torch.equal(steps[0][:, :, 1:-1], out[:, :, 1:-1])          # the frames in between keep denoising
    again = t2v("a boat", model_type="token_replace", ref_images=ref, first_last=True, **kw).frames
    assert torch.equal(again, out)                                          # the reference frames' posterior sample is seeded too
    only_first = t2v("a boat", model_type="token_replace", ref_images=ref, **kw).frames
    torch.testing.assert_close(only_first[:, :, :1], out[:, :, :1], rtol=0, atol=0)
    with pytest.raises(ValueError):
        t2v("a boat", model_type="nonsense", **kw)


def test_flow_sigmas_and_zero_star_scale():
    from teletron_b200.inference.pipeline import flow_sigmas, optimized_scale
    s = flow_sigmas(4, shift=7.0)
    assert s.shape == (5,) and float(s[0]) == 1.0 and float(s[-1]) == 0.0 and bool((s[:-1] > s[1:]).all())
    # shift k maps s -> k s / (1 + (k - 1) s): the midpoint 0.5 goes to 7 / 8
    assert float(s[2]) == pytest.approx(0.875)
    pos, neg = torch.tensor([[2.0, 0.0, 2.0]]), torch.tensor([[1.0, 1.0, 0.0]])
    assert float(optimized_scale(pos, neg)) == pytest.approx(1.0, abs=1e-6)      # <pos, neg> / |neg|^2 = 2 / 2


def _i2v_loss(rank, world, cp):
    from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, tiny_config
    from teletron_b200.parallel import state as ps
    if world > 1:
        ps.initialize_model_parallel(1, cp)
    else:
        ps.destroy_model_parallel()
    torch.manual_seed(0)
    pipe = HunyuanPipeline(tiny_config(in_channels=33), FlowConfig(model_type="i2v"))
    g = torch.Generator().manual_seed(11)
    batch = dict(latents=torch.randn(1, 16, 3, 8, 8, generator=g), prompt_embeds=torch.randn(1, 16, 64, generator=g),
                 clip_text_embed=torch.randn(1, 32, generator=g), first_frame_latents=torch.randn(1, 16, 1, 8, 8, generator=g))
    loss = pipe(batch)[0]
    loss.backward()
    w = pipe.transformer.x_embedder.proj.weight
    return float(loss.detach()), tuple(w.shape), float(w.grad.abs().sum())


def test_i2v_training_input_has_33_channels_and_cp2_matches_single():
    """First-frame latent (zero-padded in time) + one mask channel are concatenated to the noisy latent."""
    single = _i2v_loss(0, 1, 1)
    assert single[1][1] == 33 and single[2] > 0
    for loss, shape, _ in run_distributed(_i2v_loss, 2, 2):
        assert shape[1] == 33 and abs(loss - single[0]) < 1e-5 * max(1.0, abs(single[0]))


def _bcast(rank, world):
    from teletron_b200.parallel import state as ps
    from teletron_b200.training.batch import get_batch_on_this_tp_cp_rank
    ps.initialize_model_parallel(1, 2)              # one TP x CP block of two ranks, rank 0 is its source
    g = torch.Generator().manual_seed(2)
    sample = dict(latents=torch.randn(1, 16, 3, 4, 4, generator=g).bfloat16(), prompt_embeds=torch.randn(1, 7, 64, generator=g),
                  clip_text_embed=torch.randn(1, 32, generator=g), prompt_attention_mask=torch.tensor([[True] * 5 + [False] * 2]),
                  prompt=["not a tensor: stays on the source rank"])
    out = get_batch_on_this_tp_cp_rank(iter([sample]) if rank == 0 else None, torch.device("cpu"))
    assert "prompt" not in out
    return {k: (str(v.dtype), tuple(v.shape), float(v.float().sum())) for k, v in out.items()}


def test_batch_is_broadcast_with_a_fixed_size_header():
    a, b = run_distributed(_bcast, 2)
    assert a == b and a["latents"][0] == "torch.bfloat16" and a["prompt_attention_mask"][0] == "torch.bool"
    assert a["prompt_embeds"][1] == (1, 7, 64) and a["prompt_attention_mask"][2] == 5.0


def test_video_writer_avi_round_trip_and_other_containers(tmp_path):
    """The dependency-free AVI writer: header fields, index and frame payloads read back; raw frames decode to the input
    exactly, Motion-JPEG frames approximately; .gif / .npy / .mp4 (or its .avi stand-in) are produced."""
    import numpy as np
    from teletron_b200.inference import video_io as V
    g = torch.Generator().manual_seed(0)
    frames = torch.rand(5, 3, 18, 30, generator=g)                       # width 30: raw rows need padding to 4 bytes
    u8 = V.to_uint8_frames(frames)
    assert u8.shape == (5, 18, 30, 3) and u8.dtype == np.uint8
    raw = V.write_avi(str(tmp_path / "raw.avi"), u8, fps=12.5, mjpeg=False)
    info = V.read_avi_info(raw)
    assert (info["width"], info["height"], info["total_frames"], info["index_entries"]) == (30, 18, 5, 5)
    assert info["usec_per_frame"] == 80000 and info["rate"] / info["scale"] == 12.5 and info["bits"] == 24
    stride = (30 * 3 + 3) & ~3
    for f, payload in zip(u8, info["frames"]):
        rows = np.frombuffer(payload, dtype=np.uint8).reshape(18, stride)[:, :90].reshape(18, 30, 3)
        assert np.array_equal(rows[::-1, :, ::-1], f)
    smooth = torch.linspace(0, 1, 64).view(1, 1, 1, 64).expand(4, 3, 48, 64).contiguous()
    mj = V.export_to_video(smooth, str(tmp_path / "clip.avi"), fps=15)
    info = V.read_avi_info(mj)
    assert info["handler"] == b"MJPG" and len(info["frames"]) == 4 and info["frames"][0][:2] == b"\xff\xd8"
    from PIL import Image
    import io
    dec = np.asarray(Image.open(io.BytesIO(info["frames"][0])).convert("RGB")).astype(np.float32)
    assert np.abs(dec - V.to_uint8_frames(smooth)[0].astype(np.float32)).mean() < 3.0
    assert os.path.getsize(V.export_to_video(smooth, str(tmp_path / "clip.gif"))) > 0
    assert np.load(V.export_to_video(frames, str(tmp_path / "clip.npy"))).shape == (5, 18, 30, 3)
    written = V.export_to_video(smooth, str(tmp_path / "clip.mp4"))
    assert os.path.getsize(written) > 0 and os.path.splitext(written)[1] in (".mp4", ".avi")
