"""Command-line flags with Megatron-compatible names.

The reference takes its parser from Megatron-LM and adds its own flags through
``extra_args_provider`` (``examples/hunyuanvideo/pretrain_hunyuanvideo.py:48-81``); the launch
scripts pass the set listed in ``examples/hunyuanvideo/run_unified.sh:45-92``.  Every flag used by
those scripts is accepted here with the same spelling, so the scripts carry over unchanged.
Flags that only make sense for Megatron's GPT models (``--seq-length``, ``--vocab-size`` ...) are
accepted and ignored.  ``--distributed-vae`` is registered (the reference reads it without ever
defining it, ``run_unified_dist.sh:77``).
"""

from __future__ import annotations

import argparse
import os
from typing import Callable, Optional, Sequence

import torch


def _add_model_args(p):
    g = p.add_argument_group("model")
    g.add_argument("--num-layers", type=int, default=None, help="accepted for script parity; DiT depth comes from NUM_LAYERS / NUM_SINGLE_LAYERS env or --dit-*")
    g.add_argument("--hidden-size", type=int, default=3072)
    g.add_argument("--num-attention-heads", type=int, default=24)
    g.add_argument("--seq-length", type=int, default=512)
    g.add_argument("--max-position-embeddings", type=int, default=4096)
    g.add_argument("--tokenizer-type", type=str, default="NullTokenizer")
    g.add_argument("--vocab-size", type=int, default=0)
    g.add_argument("--init-method-std", type=float, default=0.006)
    g.add_argument("--no-rope-fusion", action="store_true")
    g.add_argument("--dit-num-layers", type=int, default=None)
    g.add_argument("--dit-num-single-layers", type=int, default=None)
    g.add_argument("--model-size", type=str, default="13b", choices=["13b", "sanity", "tiny"])
    g.add_argument("--model-type", type=str, default="i2v", choices=["i2v", "t2v"])
    g.add_argument("--apply-text-mask", action="store_true")


def _add_train_args(p):
    g = p.add_argument_group("training")
    g.add_argument("--micro-batch-size", type=int, default=1)
    g.add_argument("--global-batch-size", type=int, default=None)
    g.add_argument("--train-iters", type=int, default=10)
    g.add_argument("--weight-decay", type=float, default=0.01)
    g.add_argument("--clip-grad", type=float, default=0.0)
    g.add_argument("--bf16", action="store_true")
    g.add_argument("--fp16", action="store_true")
    g.add_argument("--lr", type=float, default=1e-5)
    g.add_argument("--min-lr", type=float, default=0.0)
    g.add_argument("--lr-decay-style", type=str, default="constant", choices=["constant", "linear", "cosine", "inverse-square-root"])
    g.add_argument("--lr-decay-iters", type=int, default=None)
    g.add_argument("--lr-warmup-fraction", type=float, default=0.0)
    g.add_argument("--lr-warmup-iters", type=int, default=0)
    g.add_argument("--adam-beta1", type=float, default=0.9)
    g.add_argument("--adam-beta2", type=float, default=0.999)
    g.add_argument("--adam-eps", type=float, default=1e-8)
    g.add_argument("--recompute-granularity", type=str, default=None, choices=["full", "selective"])
    g.add_argument("--recompute-method", type=str, default="block", choices=["uniform", "block"])
    g.add_argument("--recompute-num-layers", type=int, default=None)
    g.add_argument("--recompute-save-attention", action="store_true",
                   help="with full recompute, keep each block's attention output + log-sum-exp so the recompute pass "
                        "replays attention instead of running it again")
    g.add_argument("--use-distributed-optimizer", action="store_true")
    g.add_argument("--overlap-grad-reduce", action="store_true")
    g.add_argument("--ddp-bucket-size", type=int, default=None, help="bucket size in elements")
    g.add_argument("--check-for-nan-in-loss-and-grad", action="store_true")
    g.add_argument("--master-weight-mode", type=str, default="fp32", choices=["fp32", "split16", "none"])
    g.add_argument("--optimizer-state-dtype", type=str, default="fp32", choices=["fp32", "bf16"])
    g.add_argument("--seed", type=int, default=1234)
    g.add_argument("--data-parallel-random-init", action="store_true")
    g.add_argument("--exit-interval", type=int, default=None)
    g.add_argument("--step-timeout-seconds", type=float, default=0.0, help="watchdog: abort if a step takes longer (0 = off)")
    g.add_argument("--hang-dump-seconds", type=float, default=0.0,
                   help="every N seconds, dump the Python stack of every thread of every rank to stderr (0 = off): shows where a rank sits when a job stalls")


def _add_parallel_args(p):
    g = p.add_argument_group("parallelism")
    g.add_argument("--tensor-model-parallel-size", type=int, default=1)
    g.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    g.add_argument("--virtual-pipeline-model-parallel-size", type=int, default=None)
    g.add_argument("--expert-model-parallel-size", type=int, default=1,
                   help="builds the expert-parallel groups inside data parallelism (the DiT has no expert layers)")
    g.add_argument("--context-parallel-size", type=int, default=1)
    g.add_argument("--sequence-pad-multiple", type=int, default=8,
                   help="pad every context-parallel chunk of video tokens to a multiple of this (keeps weight-gradient GEMMs on the tensor-core kernel)")
    g.add_argument("--sequence-parallel", action="store_true",
                   help="shard activations over TP between GEMMs (all-gather->GEMM / GEMM->reduce-scatter)")
    g.add_argument("--allow-library-fallback", action="store_true",
                   help="let GEMM / attention cases that the sm_100a kernels do not take run on cuBLAS / SDPA (logged once per "
                        "shape) instead of raising")
    g.add_argument("--fused-comm", action="store_true",
                   help="use the in-kernel NVLink collectives (fused Ulysses all-to-all, AG-GEMM, GEMM-RS)")
    g.add_argument("--comm-barrier-timeout-seconds", type=float, default=10.0,
                   help="budget of every device-side barrier of the in-kernel collectives; when it runs out the kernel "
                        "records a status word and returns")
    g.add_argument("--comm-check-interval", type=int, default=1,
                   help="read the kernels' status words every N steps, after the gradient sync and before the optimizer "
                        "update (one small all-reduce and one host read); 0 = never")
    g.add_argument("--distributed-backend", type=str, default=None, choices=[None, "nccl", "gloo"])
    g.add_argument("--distributed-timeout-minutes", type=float, default=10)
    g.add_argument("--distributed-vae", action="store_true")
    g.add_argument("--distributed-vae-world-size", type=int, default=0)
    g.add_argument("--encoder-preset", type=str, default="default", choices=["default", "tiny"],
                   help="size of the VAE / text encoders on the encoder ranks (tiny: CPU tests)")
    g.add_argument("--encoder-text-dim", type=int, default=None)
    g.add_argument("--encoder-pooled-dim", type=int, default=None)
    g.add_argument("--encoder-max-text-len", type=int, default=256)
    g.add_argument("--nccl-communicator-config-path", type=str, default=None,
                   help="YAML file {group kind: {cga_cluster_size, max_ctas, min_ctas}} applied to the NCCL communicators of those groups")
    g.add_argument("--tp-comm-overlap", action="store_true",
                   help="overlap tensor-parallel communication with the GEMMs: here that is the sequence-parallel layout with the "
                        "all-gather -> GEMM / GEMM -> reduce-scatter kernels, so the flag turns on --sequence-parallel and --fused-comm")
    g.add_argument("--local-rank", "--local_rank", type=int, default=None)


def _add_data_args(p):
    g = p.add_argument_group("data")
    g.add_argument("--data-path", type=str, nargs="*", default=None)
    g.add_argument("--split", type=str, default="949,50,1")
    g.add_argument("--dataloader-type", type=str, default="single", choices=["single", "cyclic", "external"])
    g.add_argument("--num-workers", type=int, default=1)
    g.add_argument("--dataset-type", type=str, default="KoalaDataset", choices=["KoalaDataset", "FakeDataset"])
    g.add_argument("--num-frames", type=int, default=33)
    g.add_argument("--video-resolution", type=int, nargs=2, default=[1280, 720], metavar=("W", "H"))
    g.add_argument("--koala-opt", type=str, default=None)
    # both flags are store_false in the reference (passing them DISABLES the feature, pretrain_hunyuanvideo.py:58-61)
    g.add_argument("--vae-slicing", action="store_false")
    g.add_argument("--vae-tiling", action="store_false")
    g.add_argument("--tokenizer", type=str, default=None)
    g.add_argument("--tokenizer-mode", type=str, default="llama")
    g.add_argument("--eval-interval", type=int, default=10000)
    g.add_argument("--eval-iters", type=int, default=0)


def _add_flow_args(p):
    g = p.add_argument_group("flow matching")
    g.add_argument("--flow-resolution-shifting", action="store_true")
    g.add_argument("--flow-base-image-seq-len", type=int, default=256)
    g.add_argument("--flow-max-image-seg-len", type=int, default=4096)
    g.add_argument("--flow-base-shift", type=float, default=0.5)
    g.add_argument("--flow-max-shift", type=float, default=1.15)
    g.add_argument("--flow-shift", type=float, default=1.0)
    g.add_argument("--flow-weighting-scheme", type=str, default="none",
                   choices=["sigma_sqrt", "logit_normal", "mode", "cosmap", "none"])
    g.add_argument("--flow-logit-mean", type=float, default=0.0)
    g.add_argument("--flow-logit-std", type=float, default=1.0)
    g.add_argument("--flow-mode-scale", type=float, default=1.29)
    g.add_argument("--sanity-check", action="store_true")


def _add_io_args(p):
    g = p.add_argument_group("checkpoint / logging")
    g.add_argument("--save", type=str, default=None)
    g.add_argument("--load", type=str, default=None)
    g.add_argument("--pretrained-checkpoint", type=str, default=None)
    g.add_argument("--save-interval", type=int, default=None)
    g.add_argument("--no-load-optim", action="store_true")
    g.add_argument("--no-load-rng", action="store_true")
    g.add_argument("--no-save-optim", action="store_true")
    g.add_argument("--finetune", action="store_true")
    g.add_argument("--log-interval", type=int, default=1)
    g.add_argument("--tensorboard-dir", type=str, default=None)
    g.add_argument("--tensorboard-queue-size", type=int, default=10)
    g.add_argument("--wandb-project", type=str, default=None, help="log to Weights & Biases when the package is installed")
    g.add_argument("--wandb-exp-name", type=str, default=None)
    g.add_argument("--wandb-save-dir", type=str, default=None)
    g.add_argument("--jsonl-log", type=str, default=None)
    g.add_argument("--timing-log-level", type=int, default=0, choices=[0, 1, 2])
    g.add_argument("--timing-log-option", type=str, default="minmax", choices=["max", "minmax", "all"])
    g.add_argument("--profile", action="store_true")
    g.add_argument("--profile-step-start", type=int, default=10)
    g.add_argument("--profile-step-end", type=int, default=12)
    g.add_argument("--profile-ranks", type=int, nargs="+", default=[0])


def build_parser(extra_args_provider: Optional[Callable] = None) -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="teletron_b200 arguments", allow_abbrev=False)
    for add in (_add_model_args, _add_train_args, _add_parallel_args, _add_data_args, _add_flow_args, _add_io_args):
        add(p)
    if extra_args_provider is not None:
        p = extra_args_provider(p) or p
    return p


def validate_args(args, world_size: Optional[int] = None):
    """Derive world layout and batch sizes (what Megatron's ``validate_args`` does for the reference,
    including the encoder-rank world-size surgery of ``teletron/training/training.py:61-75``)."""
    args.rank = int(os.environ.get("RANK", "0"))
    args.world_size = int(os.environ.get("WORLD_SIZE", "1")) if world_size is None else world_size
    if args.local_rank is None:
        args.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.distributed_vae_world_size and not args.distributed_vae:
        args.distributed_vae = True
    enc = args.distributed_vae_world_size if args.distributed_vae else 0
    if args.distributed_vae and enc <= 0:
        raise ValueError("--distributed-vae needs --distributed-vae-world-size > 0")
    args.dit_world_size = args.world_size - enc
    if args.pipeline_model_parallel_size != 1:
        raise ValueError("pipeline parallelism is not supported by this model (the reference builds the "
                         "groups but every rank owns all blocks, pipeline.py:239-240)")
    if args.tp_comm_overlap and args.tensor_model_parallel_size > 1:
        args.sequence_parallel = True
        args.fused_comm = True
    mp = args.tensor_model_parallel_size * args.context_parallel_size
    if args.dit_world_size % mp:
        raise ValueError(f"DiT world size {args.dit_world_size} not divisible by tp*cp={mp}")
    args.data_parallel_size = args.dit_world_size // mp
    if args.global_batch_size is None:
        args.global_batch_size = args.micro_batch_size * args.data_parallel_size
    per = args.micro_batch_size * args.data_parallel_size
    if args.global_batch_size % per:
        raise ValueError(f"global batch {args.global_batch_size} not divisible by micro-batch x dp = {per}")
    args.num_microbatches = args.global_batch_size // per
    if (args.num_frames - 1) % 4:
        raise ValueError("--num-frames must be 4n+1")
    args.params_dtype = torch.bfloat16 if args.bf16 else (torch.float16 if args.fp16 else torch.float32)
    if args.lr_decay_iters is None:
        args.lr_decay_iters = args.train_iters
    if args.lr_warmup_fraction:
        args.lr_warmup_iters = int(args.lr_warmup_fraction * args.lr_decay_iters)
    tiny = args.model_size == "tiny"
    if args.encoder_text_dim is None:
        args.encoder_text_dim = 64 if tiny else 4096
    if args.encoder_pooled_dim is None:
        args.encoder_pooled_dim = 32 if tiny else 768
    args.iteration = 0
    args.consumed_train_samples = 0
    return args


def parse_args(extra_args_provider: Optional[Callable] = None, argv: Optional[Sequence[str]] = None,
               ignore_unknown_args: bool = False):
    parser = build_parser(extra_args_provider)
    if ignore_unknown_args:
        args, _ = parser.parse_known_args(argv)
    else:
        args = parser.parse_args(argv)
    return validate_args(args)


_GLOBAL_ARGS = None


def set_args(args) -> None:
    global _GLOBAL_ARGS
    _GLOBAL_ARGS = args


def get_args():
    if _GLOBAL_ARGS is None:
        raise RuntimeError("arguments are not initialised; call initialize() first")
    return _GLOBAL_ARGS
