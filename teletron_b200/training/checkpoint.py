"""Checkpoint save / load in the Megatron legacy layout the reference uses.

On disk (reference behaviour described at ``teletron/convert_ckpt/hunyuan/convert_hunyuanvideo.py:121-124,
333-339, 610-622`` and Megatron ``checkpointing``)::

    <dir>/latest_checkpointed_iteration.txt          "123" or "release"
    <dir>/iter_0000123/mp_rank_{tp:02d}/model_optim_rng.pt
    <dir>/iter_0000123/mp_rank_{tp:02d}/distrib_optim_{dp:03d}.pt   (sharded optimizer state)
    <dir>/release/mp_rank_{tp:02d}/model_optim_rng.pt               (converter output)

``model_optim_rng.pt`` holds ``model`` (transformer weights, keys without prefix as in
``pipeline.py:235-237``), ``checkpoint_version`` 3.0, ``args``, ``iteration``, ``optimizer``,
``opt_param_scheduler``, ``rng_state``, ``consumed_train_samples``.  Loading is non-strict and strips
a ``transformer.`` prefix and ignores ``vae.*`` / TE ``_extra_state`` keys, so both training checkpoints
and converted HF checkpoints load (``teletron/core/training.py:46-51``).
"""

from __future__ import annotations

import os
import random
from types import SimpleNamespace
from typing import Optional, Tuple

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import state as ps
from .logging import print_rank_0

TRACKER = "latest_checkpointed_iteration.txt"


def checkpoint_dir(root: str, iteration, release: bool = False) -> str:
    return os.path.join(root, "release" if release else f"iter_{int(iteration):07d}")


def model_checkpoint_name(root: str, iteration, release: bool = False, tp_rank: Optional[int] = None) -> str:
    tp_rank = ps.get_tensor_model_parallel_rank() if tp_rank is None else tp_rank
    return os.path.join(checkpoint_dir(root, iteration, release), f"mp_rank_{tp_rank:02d}", "model_optim_rng.pt")


def optim_checkpoint_name(root: str, iteration, dp_rank: int, tp_rank: Optional[int] = None) -> str:
    tp_rank = ps.get_tensor_model_parallel_rank() if tp_rank is None else tp_rank
    return os.path.join(checkpoint_dir(root, iteration), f"mp_rank_{tp_rank:02d}", f"distrib_optim_{dp_rank:03d}.pt")


def read_tracker(root: str) -> Tuple[Optional[int], bool]:
    path = os.path.join(root, TRACKER)
    if not os.path.isfile(path):
        return None, False
    s = open(path).read().strip()
    if s == "release":
        return 0, True
    return int(s), False


def _rng_state():
    st = {"random": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state()
    return st


def _set_rng_state(st):
    random.setstate(st["random"])
    np.random.set_state(st["numpy"])
    torch.set_rng_state(st["torch"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state(st["cuda"])


def _args_namespace(args) -> SimpleNamespace:
    keep = {}
    for k, v in vars(args).items():
        if isinstance(v, (int, float, str, bool, list, tuple, type(None))):
            keep[k] = v
        elif isinstance(v, torch.dtype):
            keep[k] = str(v)
    return SimpleNamespace(**keep)


def _barrier():
    if dist.is_initialized():
        dist.barrier(group=ps.get_transformer_model_group())


def save_checkpoint(iteration: int, model, optimizer, opt_param_scheduler, args, step_state: Optional[dict] = None) -> None:
    """All DiT ranks call this.  The first rank of each DP x CP group writes the model file of its
    tensor-parallel rank; every DP x CP rank writes its own optimizer shard."""
    root = args.save
    dp_rank = ps.get_data_parallel_rank(with_context_parallel=True)
    os.makedirs(os.path.dirname(model_checkpoint_name(root, iteration)), exist_ok=True)
    _barrier()
    if dp_rank == 0:
        sd = {"args": _args_namespace(args), "checkpoint_version": 3.0, "iteration": iteration,
              "model": {k: v.detach().cpu() for k, v in model.state_dict_for_save_checkpoint().items()},
              "rng_state": _rng_state(), "consumed_train_samples": getattr(args, "consumed_train_samples", 0)}
        if optimizer is not None and not args.no_save_optim:
            sd["optimizer"] = optimizer.state_dict()
        if opt_param_scheduler is not None:
            sd["opt_param_scheduler"] = opt_param_scheduler.state_dict()
        if step_state:
            sd["step_state"] = step_state
        torch.save(sd, model_checkpoint_name(root, iteration))
    if optimizer is not None and not args.no_save_optim:
        torch.save(optimizer.sharded_state_dict(), optim_checkpoint_name(root, iteration, dp_rank))
    _barrier()
    if (not dist.is_initialized()) or dist.get_rank() == 0:
        with open(os.path.join(root, TRACKER), "w") as f:
            f.write(str(iteration))
    _barrier()
    print_rank_0(f"  successfully saved checkpoint at iteration {iteration:7d} to {root}")


def normalize_model_keys(sd: dict) -> dict:
    """Accept training checkpoints (bare keys) and converter output (``transformer.*`` + ``vae.*``)."""
    out = {}
    for k, v in sd.items():
        if k.endswith("_extra_state") or k.startswith("vae."):
            continue
        if k.startswith("transformer."):
            k = k[len("transformer."):]
        out[k] = v
    return out


def load_checkpoint(model, optimizer, opt_param_scheduler, args, load_dir: Optional[str] = None, strict: bool = False) -> int:
    """Returns the iteration to resume from (0 when nothing was loaded or for ``release`` checkpoints)."""
    root = load_dir or args.load
    if root is None:
        return 0
    iteration, release = read_tracker(root)
    if iteration is None:
        print_rank_0(f"WARNING: could not find {TRACKER} in {root}; starting from random weights")
        return 0
    path = model_checkpoint_name(root, iteration, release)
    sd = torch.load(path, map_location="cpu", weights_only=False)
    target = model.module if hasattr(model, "module") else model
    target = getattr(target, "transformer", target)
    missing, unexpected = target.load_state_dict(normalize_model_keys(sd["model"]), strict=strict)
    if missing or unexpected:
        print_rank_0(f"  checkpoint load: {len(missing)} missing / {len(unexpected)} unexpected keys")
    finetune = args.finetune or release or load_dir is not None
    if optimizer is not None:
        optimizer.reload_model_params()
    if not finetune:
        if optimizer is not None and not args.no_load_optim and "optimizer" in sd:
            optimizer.load_state_dict(sd["optimizer"])
            opath = optim_checkpoint_name(root, iteration, ps.get_data_parallel_rank(with_context_parallel=True))
            if os.path.isfile(opath):
                optimizer.load_sharded_state_dict(torch.load(opath, map_location="cpu", weights_only=False))
        if opt_param_scheduler is not None and "opt_param_scheduler" in sd:
            opt_param_scheduler.load_state_dict(sd["opt_param_scheduler"])
        if not args.no_load_rng and "rng_state" in sd:
            _set_rng_state(sd["rng_state"])
        args.consumed_train_samples = sd.get("consumed_train_samples", 0)
        step_state = sd.get("step_state")
        wrapper = model.module if hasattr(model, "module") else model
        if step_state and "pipeline_step" in step_state and hasattr(wrapper, "step"):
            wrapper.step = int(step_state["pipeline_step"])      # keeps the per-step noise stream aligned
    else:
        iteration = 0
    _barrier()
    print_rank_0(f"  successfully loaded checkpoint from {root} at iteration {iteration}")
    return iteration
