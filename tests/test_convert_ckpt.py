"""HF <-> TeleTron converter: layout rules, round trip through TP-sharded files, and loading into the model."""

import os

import torch

from teletron_b200.convert_ckpt.hunyuan import convert_hunyuanvideo as C
from teletron_b200.models.hunyuanvideo import HunyuanVideoTransformer3DModel, tiny_config
from teletron_b200.parallel import state as ps


def _fake_hf_state(cfg):
    """An HF-named state dict with the tiny model's shapes, built from our own model through the inverse mapping."""
    ps.destroy_model_parallel()
    model = HunyuanVideoTransformer3DModel(cfg)
    g = torch.Generator().manual_seed(3)
    tel = {k: torch.randn(v.shape, generator=g) for k, v in model.state_dict().items()}
    return C.tel_to_hf_state(tel, cfg.num_attention_heads), tel, model


def test_qkv_interleave_is_per_head():
    heads, d = 3, 4
    q, k, v = (torch.arange(heads * d * 2).float().reshape(heads * d, 2) + 100 * i for i in range(3))
    w = C.interleave_qkv(q, k, v, heads)
    assert w.shape == (heads * 3 * d, 2)
    torch.testing.assert_close(w[:d], q[:d])
    torch.testing.assert_close(w[d:2 * d], k[:d])
    torch.testing.assert_close(w[3 * d:4 * d], q[d:2 * d])
    for a, b in zip(C.deinterleave_qkv(w, heads), (q, k, v)):
        torch.testing.assert_close(a, b)


def test_round_trip_through_tp2_files_and_model_load(tmp_path):
    cfg = tiny_config()
    hf, tel_ref, model = _fake_hf_state(cfg)
    assert any(k.endswith("attn.to_q.weight") for k in hf) and "norm_out.linear.weight" in hf
    src = tmp_path / "hf.pt"
    torch.save(hf, src)
    out = tmp_path / "tel"
    C.convert_hf_to_tel(str(src), str(out), tp=2, dtype=torch.float32, heads=cfg.num_attention_heads,
                        hidden=cfg.hidden_size, mlp_hidden=cfg.mlp_hidden)
    assert open(out / "latest_checkpointed_iteration.txt").read() == "release"
    f0 = torch.load(out / "release" / "mp_rank_00" / "model_optim_rng.pt", weights_only=False)
    assert f0["checkpoint_version"] == 3.0 and all(k.startswith("transformer.") for k in f0["model"])
    # column-parallel: rows halved; row-parallel: columns halved, bias whole; single proj_out: both input groups halved
    H, F = cfg.hidden_size, cfg.mlp_hidden
    m = f0["model"]
    assert m["transformer.transformer_blocks.0.self_attention.linear_qkv.weight"].shape == (3 * H // 2, H)
    assert m["transformer.transformer_blocks.0.mlp.linear_fc2.weight"].shape == (H, F // 2)
    assert m["transformer.transformer_blocks.0.mlp.linear_fc2.bias"].shape == (H,)
    po = m["transformer.single_transformer_blocks.0.proj_out.weight"]
    assert po.shape == (H, (H + F) // 2)
    full_po = tel_ref["single_transformer_blocks.0.proj_out.weight"]
    torch.testing.assert_close(po, torch.cat([full_po[:, :H // 2], full_po[:, H:H + F // 2]], dim=1))
    # back to HF names: identical to the source
    back = tmp_path / "hf_back"
    C.convert_tel_to_hf(str(out), str(back), torch.float32, cfg.num_attention_heads, cfg.hidden_size, cfg.mlp_hidden,
                        max_shard_size="300KB")
    # a diffusers-style folder: numbered safetensors shards, the index that maps every tensor to its shard, config.json
    import json
    from safetensors.torch import load_file
    index = json.load(open(back / "diffusion_pytorch_model.safetensors.index.json"))
    shard_names = sorted(set(index["weight_map"].values()))
    assert len(shard_names) > 1 and all(n.startswith("diffusion_pytorch_model-000") and n.endswith(f"-of-{len(shard_names):05d}.safetensors")
                                        for n in shard_names)
    assert set(index["weight_map"]) == set(hf)
    assert index["metadata"]["total_size"] == sum(v.numel() * v.element_size() for v in hf.values())
    hf2 = {}
    for n in shard_names:
        part = load_file(str(back / n))
        assert all(index["weight_map"][k] == n for k in part)
        hf2.update(part)
    assert set(hf2) == set(hf)
    for k in hf:
        torch.testing.assert_close(hf2[k], hf[k], rtol=0, atol=0)
    conf = json.load(open(back / "config.json"))
    assert conf["num_layers"] == cfg.num_layers and conf["num_single_layers"] == cfg.num_single_layers
    assert conf["num_attention_heads"] == cfg.num_attention_heads and conf["_class_name"] == "HunyuanVideoTransformer3DModel"
    # the converter reads its own output back (HF folder -> TeleTron), and one shard when everything fits
    again = tmp_path / "tel_again"
    C.convert_hf_to_tel(str(back), str(again), tp=1, dtype=torch.float32, heads=cfg.num_attention_heads,
                        hidden=cfg.hidden_size, mlp_hidden=cfg.mlp_hidden)
    single = tmp_path / "hf_single"
    C.convert_tel_to_hf(str(again), str(single), torch.float32, cfg.num_attention_heads, cfg.hidden_size, cfg.mlp_hidden)
    assert (single / "diffusion_pytorch_model.safetensors").is_file() and not (single / "diffusion_pytorch_model.safetensors.index.json").exists()
    one_file = load_file(str(single / "diffusion_pytorch_model.safetensors"))
    for k in hf:
        torch.testing.assert_close(one_file[k], hf[k], rtol=0, atol=0)
    # a TP=1 conversion loads into the model by name (training's loader strips the prefix)
    one = tmp_path / "tel1"
    C.convert_hf_to_tel(str(src), str(one), tp=1, dtype=torch.float32, heads=cfg.num_attention_heads,
                        hidden=cfg.hidden_size, mlp_hidden=cfg.mlp_hidden)
    from teletron_b200.training.checkpoint import normalize_model_keys
    sd = normalize_model_keys(torch.load(one / "release" / "mp_rank_00" / "model_optim_rng.pt", weights_only=False)["model"])
    missing, unexpected = model.load_state_dict(sd, strict=True)
    assert not missing and not unexpected
    torch.testing.assert_close(model.state_dict()["transformer_blocks.1.self_attention.linear_qkv.weight"],
                               tel_ref["transformer_blocks.1.self_attention.linear_qkv.weight"])
