"""CPU tests of the framework components around the model: ops oracle identities, parallel-state layout, optimizer
(ZeRO-1 sharding, split16 master weights), data pipeline, VAE, text encoders, watchdog / heartbeat."""

import math
import os
import time

import pytest
import torch

from dist_utils import run_distributed


# ---------------------------------------------------------------- ops oracle
def test_rope_matches_complex_rotation():
    from teletron_b200.ops import reference as R
    x = torch.randn(2, 3, 10, 16)
    ang = torch.rand(10, 8) * 6.28
    cos, sin = ang.cos().repeat_interleave(2, 1), ang.sin().repeat_interleave(2, 1)
    y = R.apply_rope(x, cos, sin)
    xc = torch.view_as_complex(x.reshape(2, 3, 10, 8, 2))
    ref = torch.view_as_real(xc * torch.polar(torch.ones_like(ang), ang)).reshape(2, 3, 10, 16)
    torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-5)


def test_layernorm_modulate_and_fused_variant():
    from teletron_b200.ops import reference as R
    x, br = torch.randn(2, 7, 32), torch.randn(2, 7, 32)
    g, sc, sh = torch.randn(2, 32), torch.randn(2, 32), torch.randn(2, 32)
    y = R.layernorm_modulate(x, sc, sh)
    ref = torch.nn.functional.layer_norm(x, (32,), eps=1e-6) * (1 + sc[:, None]) + sh[:, None]
    torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-5)
    nr, y2 = R.gate_residual_layernorm_modulate(x, br, g, sc, sh)
    torch.testing.assert_close(nr, x + g[:, None] * br)
    torch.testing.assert_close(y2, R.layernorm_modulate(nr, sc, sh))


def test_qkv_projection_layout_and_joint():
    from teletron_b200.ops import reference as R
    H, D, heads = 64, 16, 4
    x, xt = torch.randn(1, 6, H), torch.randn(1, 3, H)
    w, b = torch.randn(3 * H, H) * 0.1, torch.randn(3 * H)
    qw, kw = torch.rand(D) + 0.5, torch.rand(D) + 0.5
    ang = torch.rand(6, D // 2)
    cos, sin = ang.cos().repeat_interleave(2, 1), ang.sin().repeat_interleave(2, 1)
    q, k, v = R.qkv_projection(x, w, b, qw, kw, cos, sin, heads)
    raw = (x @ w.t() + b).view(1, 6, heads, 3, D)
    torch.testing.assert_close(v, raw[:, :, :, 2].transpose(1, 2))
    torch.testing.assert_close(q, R.apply_rope(R.rmsnorm(raw[:, :, :, 0].transpose(1, 2), qw), cos, sin))
    jq, jk, jv = R.joint_qkv_projection(x, w, b, qw, kw, cos, sin, xt, w, b, qw, kw, heads)
    assert jq.shape == (1, heads, 9, D)
    torch.testing.assert_close(jq[:, :, :6], q)


def test_flow_scheduler_and_weighting():
    from teletron_b200.models.hunyuanvideo.pipeline import FlowMatchScheduler, compute_loss_weighting
    s = FlowMatchScheduler(1000, 1.0)
    assert abs(float(s.sigmas[0]) - 1.0) < 1e-6 and abs(float(s.sigmas[-1]) - 0.001) < 1e-6
    s7 = FlowMatchScheduler(1000, 7.0)
    x = s.sigmas
    torch.testing.assert_close(s7.sigmas, 7 * x / (1 + 6 * x))
    w = compute_loss_weighting("cosmap", torch.tensor([0.5]))
    assert abs(float(w) - 2 / (math.pi * 0.5)) < 1e-6


# ---------------------------------------------------------------- parallel state
def test_rank_lists_follow_tp_cp_dp_order():
    from teletron_b200.parallel.state import build_comm_pairs, build_rank_lists, rank_coords
    L = build_rank_lists(8, 2, 2)
    assert L["tp"] == [[0, 1], [2, 3], [4, 5], [6, 7]]
    assert L["cp"] == [[0, 2], [1, 3], [4, 6], [5, 7]]
    assert L["dp"] == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert L["dp_cp"] == [[0, 2, 4, 6], [1, 3, 5, 7]]
    assert L["tp_cp"] == [[0, 1, 2, 3], [4, 5, 6, 7]]
    assert rank_coords(6, 2, 2) == {"tp": 0, "cp": 1, "dp": 1, "pp": 0}
    pairs = build_comm_pairs(6, 2, 2, 3)            # 6 DiT ranks (tp2 cp3 -> dp1) + 2 encoder ranks
    # more encoder ranks than DiT groups: both feed the one consumer in turn (the reference would leave rank 7 idle)
    assert [(p.producer, p.consumer, p.lane, p.lanes) for p in pairs] == [(6, 0, 0, 2), (7, 0, 1, 2)]
    pairs = build_comm_pairs(8, 2, 1, 2)            # dp 4, two producers
    assert [(p.producer, p.consumer, p.dp_rank) for p in pairs] == [(8, 0, 0), (9, 2, 1), (8, 4, 2), (9, 6, 3)]
    with pytest.raises(ValueError):
        build_rank_lists(6, 4, 1)


def _groups(rank, world):
    import torch.distributed as dist
    from teletron_b200.parallel import state as ps
    ps.initialize_model_parallel(2, 1, encoder_world_size=1)      # 3 ranks: tp group [0,1] + encoder rank 2
    info = (ps.is_dit_rank(), ps.get_tensor_model_parallel_world_size(), ps.get_tensor_model_parallel_rank(),
            ps.get_tensor_context_parallel_src_rank(), [(p.producer, p.consumer) for p in ps.get_comm_pairs()])
    if ps.is_dit_rank():
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, group=ps.get_tensor_model_parallel_group())
        assert float(t) == 3.0
    return info


def test_every_rank_walks_the_same_group_list_with_encoder_ranks():
    res = run_distributed(_groups, 3)
    assert res[0][0] and res[1][0] and not res[2][0]
    assert res[0][4] == [(2, 0)]


# ---------------------------------------------------------------- optimizer
def test_split16_pack_is_exact():
    from teletron_b200.ops.optim import _pack16, _unpack16
    w = torch.randn(10000) * torch.logspace(-6, 3, 10000)
    hi, lo = _pack16(w)
    assert torch.equal(_unpack16(hi, lo).view(torch.int32), w.view(torch.int32))
    assert (hi.float() - w).abs().max() <= (w.abs().max() * 2 ** -8)


def _zero1(rank, world, master_mode):
    import torch.distributed as dist
    from teletron_b200.parallel.grad_buffer import DistributedDataParallel
    from teletron_b200.training.optimizer import DistributedOptimizer
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.GELU(), torch.nn.Linear(40, 8))
    ref = torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.GELU(), torch.nn.Linear(40, 8))
    ref.load_state_dict(net.state_dict())
    ddp = DistributedDataParallel(net, dist.group.WORLD, use_distributed_optimizer=True, bucket_bytes=1024)
    opt = DistributedOptimizer(ddp, lr=1e-2, weight_decay=0.1, clip_grad=1.0, master_mode=master_mode)
    decay = [p for n, p in ref.named_parameters() if not n.endswith("bias")]
    nodecay = [p for n, p in ref.named_parameters() if n.endswith("bias")]
    ropt = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": nodecay, "weight_decay": 0.0}], lr=1e-2)
    for step in range(4):
        g = torch.Generator().manual_seed(step)
        xs = torch.randn(world, 5, 24, generator=g)
        opt.zero_grad()
        net(xs[rank]).pow(2).mean().backward()
        ddp.finish_grad_sync()
        opt.step()
        ropt.zero_grad()
        sum(ref(xs[r]).pow(2).mean() for r in range(world)).div(world).backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        ropt.step()
    return [(a.detach() - b.detach()).abs().max().item() for a, b in zip(net.parameters(), ref.parameters())]


@pytest.mark.parametrize("master_mode", ["fp32", "none"])
def test_zero1_adamw_matches_torch_adamw(master_mode):
    for diffs in run_distributed(_zero1, 2, master_mode):
        assert max(diffs) < 2e-5, diffs


def test_lr_schedule():
    from teletron_b200.training.optimizer import OptimizerParamScheduler

    class O:
        lr = 0.0
    o = O()
    s = OptimizerParamScheduler(o, max_lr=1.0, min_lr=0.1, lr_warmup_steps=10, lr_decay_steps=110, lr_decay_style="cosine")
    s.step(5)
    assert abs(o.lr - 0.5) < 1e-9
    s.step(5)
    assert abs(o.lr - 1.0) < 1e-9
    s.step(50)
    assert abs(o.lr - 0.55) < 1e-6
    s.step(100)
    assert abs(o.lr - 0.1) < 1e-9
    r = OptimizerParamScheduler(o, max_lr=1.0, min_lr=0.05, lr_warmup_steps=16, lr_decay_style="inverse-square-root")
    r.step(16)
    assert abs(o.lr - 1.0) < 1e-9
    r.step(48)                                   # step 64: sqrt(16 / 64) = 0.5
    assert abs(o.lr - 0.5) < 1e-9
    r.step(100000)
    assert abs(o.lr - 0.05) < 1e-9               # floored at min_lr


# ---------------------------------------------------------------- data
def test_fake_dataset_shapes_and_determinism():
    from teletron_b200.data import build_dataset
    ds = build_dataset("FakeDataset", num_frames=9, video_resolution=(64, 32), text_len=120)
    a, b = ds[3], ds[3]
    assert a["images"].shape == (9, 3, 32, 64) and a["latents"].shape == (16, 3, 4, 8)
    assert a["prompt_embeds"].shape == (120, 4096) and a["clip_text_embed"].shape == (768,) and len(a["prompt"]) == 880
    assert torch.equal(a["latents"], b["latents"]) and a["prompt"] == b["prompt"]
    assert not torch.equal(ds[4]["latents"], a["latents"])


def test_samplers_partition_global_batches():
    from teletron_b200.data.samplers import PretrainingRandomSampler, PretrainingSampler
    got = [list(PretrainingSampler(20, 4, 2, r, 2)) for r in range(2)]
    assert got[0][0] == [4, 5] and got[1][0] == [6, 7] and got[0][1] == [8, 9]
    seen = set()
    for r in range(2):
        for b in PretrainingRandomSampler(16, 0, 2, r, 2, seed=1):
            seen.update(b)
    assert seen == set(range(16))


def test_koala_dataset_reads_tensor_clips(tmp_path):
    from teletron_b200.data import build_dataset
    clip = torch.randint(0, 255, (20, 40, 48, 3), dtype=torch.uint8)
    torch.save(clip, tmp_path / "a.pt")
    pe = str(torch.zeros(2, 4).tolist())
    ce = str(torch.zeros(4).tolist())
    lat = str(torch.zeros(1, 2, 3, 2, 2).tolist())
    (tmp_path / "list.txt").write_text(f"a.pt;a prompt;{pe};{ce};{lat}\n")
    opt = {"phase": "test", "anno_file": str(tmp_path / "list.txt"), "data_prefix": str(tmp_path),
           "sample_types": {"fragments": {"fragments_h": 1, "fragments_w": 1, "fsize_h": 32, "fsize_w": 32, "aligned": 1,
                                          "clip_len": 5, "frame_interval": 1, "num_clips": 1}}}
    ds = build_dataset("KoalaDataset", opt=opt, num_frames=9, video_resolution=(32, 16))
    item = ds[0]
    assert item["images"].shape == (9, 3, 16, 32) and item["first_ref_image"].shape == (3, 16, 32)
    assert item["prompt"] == "a prompt" and item["latents"].shape == (2, 3, 2, 2)


def test_koala_samplers_and_spatial_sample_types(tmp_path):
    import numpy as np
    from teletron_b200.data import koala_dataset as K
    np.random.seed(0)
    u = K.UnifiedFrameSampler(fsize_t=4, fragments_t=3, frame_interval=2)
    inds = u(60)
    assert inds.shape == (12,) and inds.min() >= 0 and inds.max() < 60
    for c in range(3):                                   # four frames, two apart, inside each third of the clip
        cell = inds[4 * c:4 * c + 4]
        assert (np.diff(cell) == 2).all() and 20 * c <= cell[0] and cell[-1] < 20 * (c + 1)
    assert len(K.UnifiedFrameSampler(4, 4, drop_rate=0.5)(64)) == 8
    s = K.SimpleFrameSampler
    assert s(1)(31).tolist() == [15] and s(2)(31).tolist() == [0, 15] and s(4)(31).tolist() == [0, 10, 20, 30]
    video = torch.arange(3 * 2 * 48 * 64, dtype=torch.float32).reshape(3, 2, 48, 64)     # wide clip
    assert K.get_arp_resized_video(video, short_edge=24).shape == (3, 2, 24, 32)          # aspect ratio kept
    assert K.get_arp_resized_video(video, short_edge=24, train=True).shape == (3, 2, 24, 24)   # square crop first
    assert K.get_arp_fragment_video(video, short_fragments=3, fsize=8).shape == (3, 2, 24, 32)  # 3 x 4 cells of 8
    crop = K.get_cropped_video(video, size_h=16, size_w=16)
    assert crop.shape == (3, 2, 16, 16) and torch.equal(crop, video[:, :, 16:32, 24:40])  # centre window
    assert K.get_single_sample(video, "arp_resize_sem", short_edge=12).shape == (3, 2, 12, 16)
    assert K.get_single_sample(video, "semantic", size_h=8, size_w=8).shape == (3, 2, 8, 8)
    both = K.get_spatial_samples(video, random_crop=2, sample_types={"resize": {"size_h": 8, "size_w": 8},
                                                                      "crop": {"size_h": 8, "size_w": 8}})
    assert both["resize"].shape == both["crop"].shape == (3, 2, 8, 8)
    assert K.get_spatial_samples(video, random_crop=1, sample_types={"original": {}})["original"].shape[0] == 3
    with pytest.raises(ValueError):
        K.get_single_sample(video, "nonsense")
    # labelled-clip dataset
    torch.save(torch.randint(0, 255, (12, 20, 24, 3), dtype=torch.uint8), tmp_path / "c.pt")
    (tmp_path / "labels.txt").write_text("c.pt,0,0,3.5\n")
    ds = K.SimpleDataset({"anno_file": str(tmp_path / "labels.txt"), "data_prefix": str(tmp_path), "sample_type": "resize",
                          "sampling_args": {"size_h": 16, "size_w": 16}, "phase": "test", "clip_len": 4, "frame_interval": 2,
                          "num_clips": 1})
    item = ds[0]
    assert len(ds) == 1 and item["video"].shape == (3, 4, 16, 16) and item["gt_label"] == 3.5 and item["name"] == "c.pt"


# ---------------------------------------------------------------- models around the DiT
def test_vae_shapes_tiling_and_roundtrip_geometry():
    from teletron_b200.models.vae import AutoencoderKLHunyuanVideo
    torch.manual_seed(0)
    vae = AutoencoderKLHunyuanVideo(block_out_channels=(32, 32, 64, 64)).eval()
    x = torch.rand(1, 3, 9, 64, 96) * 2 - 1
    with torch.no_grad():
        z = vae.encode(x, sample=False)
        assert z.shape == (1, 16, 3, 8, 12)
        y = vae.decode(z)
        assert y.shape == x.shape
        # the convolutions are causal in time: output frame t sees input frames <= t only
        from teletron_b200.models.vae import CausalConv3d
        conv = CausalConv3d(3, 4, 3)
        x2 = x.clone()
        x2[:, :, 4:] = 0
        torch.testing.assert_close(conv(x2)[:, :, :4], conv(x)[:, :, :4])
        vae.tile_sample_min = 48
        vae.enable_tiling(True)
        zt = vae.encode(x, sample=False)
        assert zt.shape == z.shape


def test_text_encoders_from_config():
    from teletron_b200.models.text_encoders import (ClipTextEncoder, LlamaTextEncoder, clip_text_config, llama_config,
                                                    pad_prompt, truncate_prompt)
    llama = LlamaTextEncoder(max_length=16, dtype=torch.float32, config=llama_config(2, 64, 4, 2, 128, 1000))
    emb, mask = llama(["a short prompt", "another slightly longer prompt here"])
    assert emb.shape == (2, 16, 64) and mask.sum(1).tolist() == [4, 6]
    clip = ClipTextEncoder(max_length=12, dtype=torch.float32, config=clip_text_config(2, 32, 4, 500, 12))
    assert clip(["x y z"]).shape == (1, 32)
    t = truncate_prompt(emb[:1], mask[:1])
    assert t.shape == (4, 64)
    p, m = pad_prompt(t, 10)
    assert p.shape == (10, 64) and m.sum() == 4


def test_prompt_encoder_modes():
    from teletron_b200.models.text_encoders import PromptEncoder, clip_text_config, llama_config, t5_config
    clip_cfg = clip_text_config(2, 32, 4, 500, 12)
    prompts = ["a cat", "two dogs run"]
    emb, mask = PromptEncoder("llama", max_length=10, dtype=torch.float32, configs=[llama_config(2, 64, 4, 2, 128, 1000)])(
        prompts, with_attention_mask=True)
    assert emb.shape == (2, 10, 64) and mask.shape == (2, 10)
    emb, mask = PromptEncoder("clip_text", max_length=12, dtype=torch.float32, configs=[clip_cfg])(prompts)
    assert emb.shape == (2, 12, 32) and mask is None
    emb, _ = PromptEncoder("clip_text_proj", max_length=12, dtype=torch.float32, configs=[clip_cfg])(prompts)
    assert emb.shape == (2, 1, 32)                        # projected pooled embedding with a length-1 token axis
    (emb, pooled), masks = PromptEncoder("clip_text_and_proj", max_length=12, dtype=torch.float32,
                                         configs=[clip_cfg, clip_text_config(2, 48, 4, 500, 12)])(prompts, with_attention_mask=True)
    assert emb.shape == (2, 12, 32 + 48) and pooled.shape == (2, 48) and len(masks) == 2   # penultimate states of both towers
    emb, _ = PromptEncoder("t5", max_length=9, dtype=torch.float32, configs=[t5_config(2, 32, 4, 64, 300)])(prompts[0])
    assert emb.shape == (1, 9, 32)
    with pytest.raises(ValueError):
        PromptEncoder("bert")


def test_clip_transforms():
    from transformers import CLIPConfig, CLIPVisionConfig
    from teletron_b200.models.clip_transform import (CLIPTextTransform, CLIPTextWithProjectionTransform, CLIPTransform,
                                                     preprocess_images)
    from teletron_b200.models.text_encoders import clip_text_config
    torch.manual_seed(0)
    tcfg = clip_text_config(2, 32, 4, 300, 12)
    vcfg = CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, image_size=32,
                            patch_size=8, projection_dim=24)
    cfg = CLIPConfig(text_config=tcfg.to_dict(), vision_config=vcfg.to_dict(), projection_dim=24)
    images = torch.rand(2, 3, 40, 56)
    assert preprocess_images(images, 32).shape == (2, 3, 32, 32)
    clip = CLIPTransform(None, dtype=torch.float32, config=cfg)
    text_f, image_f = clip(text=["a cat", "a dog on grass"], image=images)
    assert text_f.shape == (2, 24) and image_f.shape == (2, 24)
    assert abs(float((text_f[0] ** 2).sum()) - 1.0) < 1e-4 and abs(float((image_f[1] ** 2).sum()) - 1.0) < 1e-4   # L2-normalised
    pooled = clip(text="a cat", text_w_proj=False, to_numpy=False)
    assert tuple(pooled.shape) == (1, 32) and clip() is None
    tt = CLIPTextTransform(None, dtype=torch.float32, config=tcfg)
    assert tt(["a cat"], "after_pool").shape == (1, 32) and tt(["a cat"], "before_pool").shape == (1, 12, 32)
    with pytest.raises(ValueError):
        tt("a cat", "middle")
    two = CLIPTextWithProjectionTransform(None, dtype=torch.float32, config=(tcfg, clip_text_config(2, 48, 4, 300, 12)))
    feats, pooled = two(["a cat", "a dog"], "after_pool")
    assert feats.shape == (2, 32 + 48) and pooled.shape == (2, 48)
    feats, pooled = two(["a cat", "a dog"], "before_pool")
    assert feats.shape == (2, 12, 32 + 48) and pooled.shape == (2, 48)


def test_legacy_fused_layer_names():
    """The reference's module-level wrapper names, checked against plain PyTorch formulas (and their gradients)."""
    import torch.nn.functional as F
    from teletron_b200.legacy.fusedlayers import (AdaLNCustom, FP32LayerNorm, FusedAdaLayerNormZero,
                                                  FusedAdaLayerNormZeroSingle, Get_RMSNorm, RMSNormModelFunction)
    torch.manual_seed(0)
    x = torch.randn(2, 5, 16, requires_grad=True)
    emb = torch.randn(2, 16)
    ln = lambda t: F.layer_norm(t, (16,), eps=1e-6)  # noqa: E731
    zero = FusedAdaLayerNormZero(16)
    out, gate_msa, shift_mlp, scale_mlp, gate_mlp = zero(x, emb)
    sh, sc, g, sh2, sc2, g2 = zero.linear(F.silu(emb)).chunk(6, dim=1)
    torch.testing.assert_close(out, ln(x) * (1 + sc[:, None]) + sh[:, None], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(gate_msa, g)
    torch.testing.assert_close(scale_mlp, sc2)
    out.sum().backward()
    assert x.grad is not None and zero.linear.weight.grad is not None
    single = FusedAdaLayerNormZeroSingle(16)
    out, gate = single(x.detach(), emb)
    sh, sc, g = single.linear(F.silu(emb)).chunk(3, dim=1)
    torch.testing.assert_close(out, ln(x.detach()) * (1 + sc[:, None]) + sh[:, None], rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError):
        AdaLNCustom(8)(x, sc, sh)
    with pytest.raises(ValueError):
        FusedAdaLayerNormZero(16, norm_type="batch_norm")
    y = FP32LayerNorm(16, elementwise_affine=False)(x.detach().bfloat16())
    assert y.dtype == torch.bfloat16 and torch.allclose(y.float(), ln(x.detach().bfloat16().float()), atol=2e-2)
    norm = Get_RMSNorm()(16)
    w = torch.rand(16)
    with torch.no_grad():
        norm.weight.copy_(w)
    xd = x.detach()
    ref = xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + 1e-6) * w
    torch.testing.assert_close(norm(xd), ref, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(RMSNormModelFunction.apply(xd, w, 1e-6), ref, rtol=1e-5, atol=1e-5)


# ---------------------------------------------------------------- failure detection (host side only)
def test_step_watchdog_fires_without_heartbeat():
    from teletron_b200.training.watchdog import StepWatchdog
    fired = []
    w = StepWatchdog(0.2, on_timeout=lambda step, idle: fired.append((step, idle)), poll=0.05)
    w.beat(7)
    time.sleep(0.6)
    w.stop()
    assert fired and fired[0][0] == 7
    ok = StepWatchdog(0.5, on_timeout=lambda s, i: fired.append("bad"), poll=0.05)
    for i in range(5):
        ok.beat(i)
        time.sleep(0.05)
    ok.stop()
    assert "bad" not in fired


def test_heartbeat_reports_departed_and_silent_ranks():
    import torch.distributed as dist
    from teletron_b200.training.watchdog import Heartbeat
    store = dist.HashStore()
    hb = [Heartbeat(store, r, 3, timeout=0.2) for r in range(3)]
    assert hb[0].dead_ranks() == []
    hb[1].leave()
    assert hb[0].dead_ranks() == [1]
    time.sleep(0.3)
    hb[0].dead_ranks()
    time.sleep(0.3)
    assert hb[0].dead_ranks() == [1, 2]        # rank 2 stopped beating
    hb[2].beat()
    assert hb[0].dead_ranks() == [1]


def test_max_frames_proposal_stays_under_the_limit():
    import importlib.util
    import os
    spec = importlib.util.spec_from_file_location("max_frames", os.path.join(os.path.dirname(__file__), "..", "benchmarks", "max_frames.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    # 1 GB per latent frame on top of 75 GB fixed: 90 latent frames (357 frames) fit under 165 GB, 91 do not
    f = m.propose(33, 84.0, 65, 92.0, 165.0)
    assert f == 357 and m.latent_frames(f) == 90
    with pytest.raises(ValueError):
        m.propose(33, 84.0, 35, 84.0, 165.0)


def test_memory_model_reproduces_measured_peaks_and_bounds_frames():
    from teletron_b200.models.hunyuanvideo import hunyuan_13b
    from teletron_b200.utils import estimate, max_frames, roofline_ms, video_tokens
    assert video_tokens(33) == 32400 and video_tokens(129) == 118800
    t2v, i2v = hunyuan_13b(in_channels=16), hunyuan_13b(in_channels=33)
    one = estimate(t2v, 33, optimizer_bytes_per_param=6.0, fused_comm=False).as_gib()
    assert abs(one["total"] - 147.2) / 147.2 < 0.03                       # 1 GPU, compact optimizer state
    e = estimate(t2v, 33, tp=2, cp=4).as_gib()
    assert abs(e["total"] - e["weights_grads"] - e["workspaces"] - 23.9) < 1.5   # allocator part at tp2 x cp4
    assert abs(estimate(i2v, 129, cp=8).as_gib()["total"] - 79.9) / 79.9 < 0.03  # allocator + symmetric heaps at cp8
    f = max_frames(i2v, 165.0, tp=1, cp=8)
    assert f % 4 == 1 and f > 245                                         # well past the reference's 8 x H800 figure
    assert estimate(i2v, f, cp=8).total / 2 ** 30 <= 165.0 < estimate(i2v, f + 4, cp=8).total / 2 ** 30
    assert max_frames(t2v, 1.0) == 0
    # a GEMM of 1e15 FLOPs is compute bound, 1 GB over NVLink takes 1.3 ms
    assert roofline_ms(flops=1e15) > 500 and abs(roofline_ms(nvlink_bytes=1e9) - 1e3 / 770.0) < 1e-6


def test_restart_wrapper_relaunches_only_on_watchdog_exit(tmp_path):
    import os
    import subprocess
    script = os.path.join(os.path.dirname(__file__), "..", "examples", "hunyuanvideo", "run_with_restart.sh")
    counter = tmp_path / "n"
    # exits 75 (the step watchdog's code) twice, then succeeds
    prog = f"n=$(cat {counter} 2>/dev/null || echo 0); echo $((n+1)) > {counter}; [ $n -ge 2 ] && exit 0; exit 75"
    env = dict(os.environ, MAX_RESTARTS="5", RESTART_DELAY="0")
    r = subprocess.run(["bash", script, "bash", "-c", prog], env=env, capture_output=True, text=True)
    assert r.returncode == 0 and counter.read_text().strip() == "3" and r.stderr.count("restart") >= 2
    # an ordinary failure is final
    r = subprocess.run(["bash", script, "bash", "-c", "exit 3"], env=env, capture_output=True, text=True)
    assert r.returncode == 3 and "not restarting" in r.stderr
    # the restart budget is respected
    r = subprocess.run(["bash", script, "bash", "-c", "exit 75"], env=dict(env, MAX_RESTARTS="1"), capture_output=True, text=True)
    assert r.returncode == 75 and "giving up" in r.stderr


def test_split_tokens_backward_is_one_concatenation():
    """``split_tokens`` returns the two slices; its gradient equals that of plain slicing, also when one half is unused."""
    from teletron_b200.parallel.mappings import split_tokens
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 9, 5, generator=g, requires_grad=True)
    y = x.detach().clone().requires_grad_()
    a, b = split_tokens(x * 1.0, 6)
    ra, rb = (y * 1.0)[:, :6], (y * 1.0)[:, 6:]
    assert a.shape == (2, 6, 5) and b.shape == (2, 3, 5) and torch.equal(a, ra) and torch.equal(b, rb)
    wa, wb = torch.randn(2, 6, 5, generator=g), torch.randn(2, 3, 5, generator=g)
    ((a * wa).sum() + (b * wb).sum()).backward()
    ((ra * wa).sum() + (rb * wb).sum()).backward()
    torch.testing.assert_close(x.grad, y.grad)
    x.grad = None
    a, _ = split_tokens(x * 1.0, 6)
    (a * wa).sum().backward()
    assert float(x.grad[:, 6:].abs().max()) == 0.0 and torch.allclose(x.grad[:, :6], wa)
    # without autograd it is plain slicing
    with torch.no_grad():
        p, q = split_tokens(x, 4)
    assert p.shape[1] == 4 and q.shape[1] == 5


def test_linear_merged_matches_linear_of_the_concatenation():
    from teletron_b200 import ops
    g = torch.Generator().manual_seed(1)
    x1, x2 = torch.randn(1, 7, 6, generator=g, requires_grad=True), torch.randn(1, 7, 10, generator=g, requires_grad=True)
    w, b = torch.randn(4, 16, generator=g, requires_grad=True), torch.randn(4, generator=g, requires_grad=True)
    y = ops.linear_merged(x1, x2, w, b)
    ref = torch.nn.functional.linear(torch.cat([x1, x2], -1), w, b)
    torch.testing.assert_close(y, ref)
    y.square().sum().backward()
    assert x1.grad.shape == x1.shape and x2.grad.shape == x2.shape and w.grad.shape == w.shape


def test_read_video_decodes_a_container_file_with_opencv(tmp_path):
    """Without ``decord`` the dataset decodes ``.mp4`` / ``.avi`` clips through OpenCV: frame count, requested indices
    (wrapping past the end) and RGB channel order."""
    cv2 = pytest.importorskip("cv2")
    import numpy as np
    from teletron_b200.data.koala_dataset import read_video, video_num_frames
    path = str(tmp_path / "clip.avi")
    w = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"MJPG"), 10.0, (64, 48))
    if not w.isOpened():
        pytest.skip("this OpenCV build cannot write MJPG")
    for i in range(6):
        frame = np.zeros((48, 64, 3), dtype=np.uint8)
        frame[..., 2] = 40 * i + 20            # OpenCV frames are BGR: this is the red channel
        w.write(frame)
    w.release()
    assert video_num_frames(path) == 6
    v = read_video(path)
    assert v.shape == (6, 48, 64, 3) and v.dtype == torch.uint8
    red = v[..., 0].float().mean(dim=(1, 2))
    assert torch.all(red[1:] > red[:-1]) and float(v[..., 2].float().mean()) < 12        # red grows, blue stays dark
    sel = read_video(path, np.array([4, 1, 7]))                                           # 7 wraps to 1
    assert sel.shape[0] == 3 and torch.equal(sel[1], sel[2]) and torch.equal(sel[0], v[4])
