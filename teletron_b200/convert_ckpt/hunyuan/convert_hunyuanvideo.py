"""HuggingFace (diffusers) <-> TeleTron checkpoint conversion for the HunyuanVideo transformer.

Same command line and on-disk result as the reference converter
(``teletron/convert_ckpt/hunyuan/convert_hunyuanvideo.py:52-106, 325-622, 635-1008``):

* ``--load-path`` (diffusers ``transformer`` directory or a ``.pt`` / ``.safetensors`` state dict), ``--save-path``,
  ``--target-tensor-model-parallel-size``, ``--target-params-dtype``; writes
  ``<save>/release/mp_rank_{tp:02d}/model_optim_rng.pt`` (keys prefixed ``transformer.``; ``vae.*`` appended when a VAE
  state dict is given) and ``latest_checkpointed_iteration.txt`` containing ``release``.
* ``--convert-checkpoint-from-megatron-to-transformers`` reverses it (all TP shards merged into one HF state dict).

Layout rules: q / k / v (and the added text q / k / v) are interleaved per head into one ``linear_qkv`` weight with rows
``[head][q | k | v][head_dim]`` (``:379-398``); column-parallel weights shard dim 0, row-parallel weights dim 1 with the
bias kept whole (``:491-551``); the single block's ``proj_out`` input is sharded separately over its attention part
(first ``hidden`` columns) and its MLP part (``:578-589``); ``norm_out.linear`` becomes ``norm_out.adaLN_modulation.1``
(``:593-594``).  Unlike the reference, the reverse direction reads the tensor-parallel size from the checkpoint
directory instead of a flag, accepts prefixed and un-prefixed keys alike, and writes a real ``.pt`` state dict.
"""

from __future__ import annotations

import argparse
import glob
import json
import os
import re
import shutil
from types import SimpleNamespace
from typing import Dict, List, Optional

import torch

from ...models.hunyuanvideo.model import shard_tensor, unshard_tensors

# HF name fragment -> TeleTron name fragment for tensors that are copied as they are
DUAL_RENAMES = {
    "norm1.linear": "norm1.linear",
    "norm1_context.linear": "norm1_context.linear",
    "attn.to_out.0": "self_attention.linear_proj",
    "attn.to_add_out": "self_attention.added_linear_proj",
    "attn.norm_q": "self_attention.q_layernorm",
    "attn.norm_k": "self_attention.k_layernorm",
    "attn.norm_added_q": "self_attention.added_q_layernorm",
    "attn.norm_added_k": "self_attention.added_k_layernorm",
    "ff.net.0.proj": "mlp.linear_fc1",
    "ff.net.2": "mlp.linear_fc2",
    "ff_context.net.0.proj": "ff_context.linear_fc1",
    "ff_context.net.2": "ff_context.linear_fc2",
}
SINGLE_RENAMES = {
    "norm.linear": "norm.linear",
    "attn.norm_q": "self_attention.q_layernorm",
    "attn.norm_k": "self_attention.k_layernorm",
    "proj_mlp": "proj_mlp",
    "proj_out": "proj_out",
}
COLUMN_PARALLEL = ("norm1.linear", "norm1_context.linear", "norm.linear", "linear_qkv", "added_linear_qkv", "linear_fc1", "proj_mlp")
ROW_PARALLEL = ("linear_proj", "added_linear_proj", "linear_fc2")


def interleave_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, heads: int) -> torch.Tensor:
    """``[heads*d, ...] x 3 -> [heads*3*d, ...]`` with rows ordered ``[head][q|k|v][d]``."""
    d = q.shape[0] // heads
    parts = [t.reshape(heads, 1, d, *t.shape[1:]) for t in (q, k, v)]
    return torch.cat(parts, dim=1).reshape(heads * 3 * d, *q.shape[1:])


def deinterleave_qkv(qkv: torch.Tensor, heads: int):
    d = qkv.shape[0] // (3 * heads)
    t = qkv.reshape(heads, 3, d, *qkv.shape[1:])
    return tuple(t[:, i].reshape(heads * d, *qkv.shape[1:]) for i in range(3))


def _partition(name: str, hidden: int, mlp_hidden: int):
    """(partition_dim, partitions) of a TeleTron tensor name."""
    is_block = name.startswith(("transformer_blocks.", "single_transformer_blocks."))
    if not is_block:
        return None, None
    body = name.split(".", 2)[2]
    stem = body.rsplit(".", 1)[0]
    leaf = body.rsplit(".", 1)[1]
    last = stem.split(".")[-1] if "." in stem else stem
    if stem.endswith(COLUMN_PARALLEL) or last in COLUMN_PARALLEL:
        return 0, None
    if name.startswith("single_transformer_blocks.") and stem == "proj_out":
        return (1, (hidden, mlp_hidden)) if leaf == "weight" else (None, None)
    if last in ROW_PARALLEL:
        return (1, None) if leaf == "weight" else (None, None)
    return None, None


def hf_to_tel_state(hf: Dict[str, torch.Tensor], heads: int = 24) -> Dict[str, torch.Tensor]:
    """Full (unsharded) TeleTron-named state dict from a diffusers state dict."""
    out: Dict[str, torch.Tensor] = {}
    done = set()
    for key, val in hf.items():
        m = re.match(r"^(transformer_blocks|single_transformer_blocks)\.(\d+)\.(.+)\.(weight|bias)$", key)
        if m is None:
            if key.startswith("norm_out.linear."):
                out[key.replace("norm_out.linear.", "norm_out.adaLN_modulation.1.")] = val
            else:
                out[key] = val
            continue
        kind, idx, stem, leaf = m.groups()
        prefix = f"{kind}.{idx}."
        if stem in ("attn.to_q", "attn.to_k", "attn.to_v"):
            tag = prefix + "self_attention.linear_qkv." + leaf
            if tag not in done:
                out[tag] = interleave_qkv(*(hf[f"{prefix}attn.to_{c}.{leaf}"] for c in "qkv"), heads)
                done.add(tag)
        elif stem in ("attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj"):
            tag = prefix + "self_attention.added_linear_qkv." + leaf
            if tag not in done:
                out[tag] = interleave_qkv(*(hf[f"{prefix}attn.add_{c}_proj.{leaf}"] for c in "qkv"), heads)
                done.add(tag)
        else:
            table = DUAL_RENAMES if kind == "transformer_blocks" else SINGLE_RENAMES
            if stem not in table:
                raise KeyError(f"unexpected tensor in a transformer block: {key}")
            out[prefix + table[stem] + "." + leaf] = val
    return out


def tel_to_hf_state(tel: Dict[str, torch.Tensor], heads: int = 24) -> Dict[str, torch.Tensor]:
    out: Dict[str, torch.Tensor] = {}
    inv_dual = {v: k for k, v in DUAL_RENAMES.items()}
    inv_single = {v: k for k, v in SINGLE_RENAMES.items()}
    for key, val in tel.items():
        if key.endswith("_extra_state"):
            continue
        m = re.match(r"^(transformer_blocks|single_transformer_blocks)\.(\d+)\.(.+)\.(weight|bias)$", key)
        if m is None:
            out[key.replace("norm_out.adaLN_modulation.1.", "norm_out.linear.")] = val
            continue
        kind, idx, stem, leaf = m.groups()
        prefix = f"{kind}.{idx}."
        if stem == "self_attention.linear_qkv":
            for c, t in zip("qkv", deinterleave_qkv(val, heads)):
                out[f"{prefix}attn.to_{c}.{leaf}"] = t
        elif stem == "self_attention.added_linear_qkv":
            for c, t in zip("qkv", deinterleave_qkv(val, heads)):
                out[f"{prefix}attn.add_{c}_proj.{leaf}"] = t
        else:
            table = inv_dual if kind == "transformer_blocks" else inv_single
            out[prefix + table[stem] + "." + leaf] = val
    return out


def shard_state(full: Dict[str, torch.Tensor], tp: int, hidden: int, mlp_hidden: int) -> List[Dict[str, torch.Tensor]]:
    ranks = [dict() for _ in range(tp)]
    for name, t in full.items():
        dim, parts = _partition(name, hidden, mlp_hidden)
        for r in range(tp):
            ranks[r][name] = shard_tensor(t, dim, tp, r, parts).clone() if dim is not None else t
    return ranks


def merge_shards(shards: List[Dict[str, torch.Tensor]], hidden: int, mlp_hidden: int) -> Dict[str, torch.Tensor]:
    tp = len(shards)
    out = {}
    for name in shards[0]:
        dim, parts = _partition(name, hidden, mlp_hidden)
        if dim is None or tp == 1:
            out[name] = shards[0][name]
        else:
            local = None
            if parts is not None:
                local = tuple(p for p in parts)
            out[name] = unshard_tensors([s[name] for s in shards], dim, local)
    return out


def _strip_prefix(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {(k[len("transformer."):] if k.startswith("transformer.") else k): v for k, v in sd.items() if not k.startswith("vae.")}


def _load_any(path: str) -> Dict[str, torch.Tensor]:
    if os.path.isdir(path):
        files = sorted(glob.glob(os.path.join(path, "*.safetensors"))) or sorted(glob.glob(os.path.join(path, "*.bin"))) \
            or sorted(glob.glob(os.path.join(path, "*.pt")))
        if not files:
            raise FileNotFoundError(f"no weight files under {path}")
        sd = {}
        for f in files:
            sd.update(_load_any(f))
        return sd
    if path.endswith(".safetensors"):
        from safetensors.torch import load_file
        return load_file(path)
    obj = torch.load(path, map_location="cpu", weights_only=False)
    return obj.get("state_dict", obj) if isinstance(obj, dict) else obj


def save_tel_checkpoint(save_path: str, rank_states: List[Dict[str, torch.Tensor]], dtype: torch.dtype,
                        vae_state: Optional[Dict[str, torch.Tensor]] = None, extra_args: Optional[dict] = None) -> None:
    os.makedirs(save_path, exist_ok=True)
    with open(os.path.join(save_path, "latest_checkpointed_iteration.txt"), "w") as f:
        f.write("release")
    tp = len(rank_states)
    for r, sd in enumerate(rank_states):
        d = os.path.join(save_path, "release", f"mp_rank_{r:02d}")
        os.makedirs(d, exist_ok=True)
        model = {"transformer." + k: (v.to(dtype) if v.is_floating_point() else v) for k, v in sd.items()}
        if vae_state:
            model.update({"vae." + k: v for k, v in vae_state.items()})
        args = SimpleNamespace(tensor_model_parallel_size=tp, pipeline_model_parallel_size=1, **(extra_args or {}))
        torch.save({"model": model, "checkpoint_version": 3.0, "args": args, "iteration": 0}, os.path.join(d, "model_optim_rng.pt"))


def load_tel_checkpoint(load_path: str) -> List[Dict[str, torch.Tensor]]:
    tracker = os.path.join(load_path, "latest_checkpointed_iteration.txt")
    it = open(tracker).read().strip() if os.path.isfile(tracker) else "release"
    sub = "release" if it == "release" else f"iter_{int(it):07d}"
    dirs = sorted(glob.glob(os.path.join(load_path, sub, "mp_rank_*")))
    if not dirs:
        raise FileNotFoundError(f"no mp_rank_* directories under {os.path.join(load_path, sub)}")
    return [_strip_prefix(torch.load(os.path.join(d, "model_optim_rng.pt"), map_location="cpu", weights_only=False)["model"])
            for d in dirs]


def convert_hf_to_tel(load_path: str, save_path: str, tp: int, dtype: torch.dtype, heads: int = 24, hidden: int = 3072,
                      mlp_hidden: int = 12288, vae_path: Optional[str] = None) -> None:
    full = hf_to_tel_state(_load_any(load_path), heads)
    vae = _load_any(vae_path) if vae_path else None
    save_tel_checkpoint(save_path, shard_state(full, tp, hidden, mlp_hidden), dtype, vae)


def _parse_size(text: str) -> int:
    t = text.strip().upper()
    for suffix, mult in (("GIB", 2 ** 30), ("MIB", 2 ** 20), ("KIB", 2 ** 10), ("GB", 10 ** 9), ("MB", 10 ** 6), ("KB", 10 ** 3)):
        if t.endswith(suffix):
            return int(float(t[:-len(suffix)]) * mult)
    return int(t)


def hf_transformer_config(hf: Dict[str, torch.Tensor], heads: int, hidden: int) -> dict:
    """``config.json`` of a diffusers ``HunyuanVideoTransformer3DModel`` derived from the weights themselves (used when the
    checkpoint being converted back has no original ``config.json`` next to it)."""
    import re
    n_dual = 1 + max((int(m.group(1)) for k in hf for m in [re.match(r"transformer_blocks\.(\d+)\.", k)] if m), default=-1)
    n_single = 1 + max((int(m.group(1)) for k in hf for m in [re.match(r"single_transformer_blocks\.(\d+)\.", k)] if m), default=-1)
    n_ref = 1 + max((int(m.group(1)) for k in hf for m in [re.match(r"context_embedder\.token_refiner\.refiner_blocks\.(\d+)\.", k)] if m),
                    default=-1)
    cfg = {"_class_name": "HunyuanVideoTransformer3DModel", "num_attention_heads": heads, "attention_head_dim": hidden // heads,
           "num_layers": n_dual, "num_single_layers": n_single, "num_refiner_layers": n_ref, "mlp_ratio": 4.0, "patch_size": 2,
           "patch_size_t": 1, "qk_norm": "rms_norm", "guidance_embeds": any(k.startswith("time_text_embed.guidance_embedder") for k in hf),
           "rope_axes_dim": [16, 56, 56], "rope_theta": 256.0}
    w = hf.get("x_embedder.proj.weight")
    if w is not None:
        cfg["in_channels"] = int(w.shape[1])
    w = hf.get("proj_out.weight")
    if w is not None:
        cfg["out_channels"] = int(w.shape[0]) // 4          # patch 1 x 2 x 2
    w = hf.get("context_embedder.proj_in.weight")
    if w is not None:
        cfg["text_embed_dim"] = int(w.shape[1])
    w = hf.get("time_text_embed.text_embedder.linear_1.weight")
    if w is not None:
        cfg["pooled_projection_dim"] = int(w.shape[1])
    return cfg


def save_hf_sharded(hf: Dict[str, torch.Tensor], save_path: str, max_shard_size: str = "10GB",
                    config: Optional[dict] = None, config_from: Optional[str] = None) -> List[str]:
    """Write a diffusers-loadable transformer folder: ``diffusion_pytorch_model.safetensors`` (one shard) or
    ``diffusion_pytorch_model-0000x-of-0000y.safetensors`` + ``diffusion_pytorch_model.safetensors.index.json``, and
    ``config.json``.  The reference writes ``.bin`` shards, the same index name and copies the original config
    (``convert_hunyuanvideo.py:980-1006``); safetensors is what current diffusers looks for first."""
    from safetensors.torch import save_file
    os.makedirs(save_path, exist_ok=True)
    limit = _parse_size(max_shard_size)
    shards, cur, cur_bytes = [], {}, 0
    for k, v in hf.items():                                     # key order kept: blocks stay together in a shard
        nb = v.numel() * v.element_size()
        if cur and cur_bytes + nb > limit:
            shards.append(cur)
            cur, cur_bytes = {}, 0
        cur[k] = v.contiguous()
        cur_bytes += nb
    if cur:
        shards.append(cur)
    names = []
    if len(shards) == 1:
        names.append("diffusion_pytorch_model.safetensors")
        save_file(shards[0], os.path.join(save_path, names[0]), metadata={"format": "pt"})
    else:
        weight_map = {}
        for i, sh in enumerate(shards):
            name = f"diffusion_pytorch_model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
            names.append(name)
            save_file(sh, os.path.join(save_path, name), metadata={"format": "pt"})
            weight_map.update({k: name for k in sh})
        total = sum(v.numel() * v.element_size() for v in hf.values())
        with open(os.path.join(save_path, "diffusion_pytorch_model.safetensors.index.json"), "w") as f:
            json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    src = os.path.join(config_from, "config.json") if config_from else None
    if src and os.path.isfile(src):
        shutil.copyfile(src, os.path.join(save_path, "config.json"))
    elif config is not None:
        with open(os.path.join(save_path, "config.json"), "w") as f:
            json.dump(config, f, indent=2)
    return names


def convert_tel_to_hf(load_path: str, save_path: str, dtype: torch.dtype, heads: int = 24, hidden: int = 3072,
                      mlp_hidden: int = 12288, max_shard_size: str = "10GB") -> None:
    full = merge_shards(load_tel_checkpoint(load_path), hidden, mlp_hidden)
    hf = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tel_to_hf_state(full, heads).items()}
    # the original diffusers config, if the TeleTron checkpoint sits next to one (as the reference assumes), else derived
    save_hf_sharded(hf, save_path, max_shard_size, config=hf_transformer_config(hf, heads, hidden),
                    config_from=os.path.dirname(os.path.abspath(load_path.rstrip("/"))))


def get_args(argv=None):
    p = argparse.ArgumentParser(description="HunyuanVideo HF <-> TeleTron checkpoint converter", allow_abbrev=True)
    p.add_argument("--load-path", type=str, required=True)
    p.add_argument("--save-path", type=str, required=True)
    p.add_argument("--hf-ckpt-path", type=str, default=None, help="diffusers pipeline root (its vae/ is embedded as vae.* keys)")
    p.add_argument("--target-params-dtype", type=str, default="bf16", choices=["fp32", "fp16", "bf16"])
    p.add_argument("--target-tensor-model-parallel-size", type=int, default=1)
    p.add_argument("--target-pipeline-model-parallel-size", type=int, default=1)
    p.add_argument("--convert-checkpoint-from-megatron-to-transformers", action="store_true")
    p.add_argument("--num-attention-heads", type=int, default=24)
    p.add_argument("--hidden-size", type=int, default=3072)
    p.add_argument("--mlp-hidden-size", type=int, default=12288)
    p.add_argument("--max-shard-size", type=str, default="10GB", help="TeleTron -> HF: largest safetensors shard (e.g. 5GB, 42GB)")
    return p.parse_args(argv)


def main(argv=None):
    a = get_args(argv)
    if a.target_pipeline_model_parallel_size != 1:
        raise SystemExit("pipeline parallelism is not supported by the HunyuanVideo model (every rank owns all blocks)")
    dtype = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[a.target_params_dtype]
    if a.convert_checkpoint_from_megatron_to_transformers:
        convert_tel_to_hf(a.load_path, a.save_path, dtype, a.num_attention_heads, a.hidden_size, a.mlp_hidden_size,
                          a.max_shard_size)
    else:
        vae = os.path.join(a.hf_ckpt_path, "vae") if a.hf_ckpt_path and os.path.isdir(os.path.join(a.hf_ckpt_path, "vae")) else None
        convert_hf_to_tel(a.load_path, a.save_path, a.target_tensor_model_parallel_size, dtype, a.num_attention_heads,
                          a.hidden_size, a.mlp_hidden_size, vae)
    print(f"converted {a.load_path} -> {a.save_path}")


if __name__ == "__main__":
    main()
