"""Training driver: initialisation, model/optimizer setup, the step loop and ``pretrain()``.

Public contract follows the reference (``teletron/training/training.py:47-268``,
``teletron/core/training.py:20-66`` and the Megatron ``train()`` loop it delegates to):
``pretrain(train_valid_test_datasets_provider, model_provider, forward_step_func,
producer_process=..., extra_args_provider=...)``.  ``forward_step_func(data_iterator, model)``
returns ``(output_tensor, loss_func)`` and ``loss_func(output_tensor)`` returns
``(loss, {"name": value})`` exactly as in ``examples/hunyuanvideo/pretrain_hunyuanvideo.py:133-160``.

Nothing is monkey-patched (the reference swaps four Megatron internals at import,
``teletron/megatron_adaptor.py:15-48``): this module owns the loop.
"""

from __future__ import annotations

import datetime
import os
import random
import time
from typing import Callable, Dict, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..data.loader import build_pretraining_data_loader
from ..parallel import state as ps
from ..parallel.grad_buffer import DistributedDataParallel
from . import args as args_mod
from .checkpoint import load_checkpoint, save_checkpoint
from .logging import MetricLogger, Timers, model_flops_per_sample, peak_bf16_tflops, print_rank_0, print_rank_last
from .optimizer import DistributedOptimizer, OptimizerParamScheduler
from ..ops import nvtx_range
from ..ops._lib import CommTimeoutError
from .watchdog import StepWatchdog

_TIMERS: Optional[Timers] = None


def get_timers() -> Timers:
    global _TIMERS
    if _TIMERS is None:
        _TIMERS = Timers()
    return _TIMERS


def set_random_seed(seed: int, data_parallel_random_init: bool = False) -> None:
    if data_parallel_random_init:
        seed = seed + 10 * ps.get_data_parallel_rank()
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def initialize(extra_args_provider: Optional[Callable] = None, argv=None, args_defaults: Optional[dict] = None,
               ignore_unknown_args: bool = False):
    """Parse flags, start ``torch.distributed`` (NCCL on GPU, gloo on CPU), build all groups, seed
    DiT ranks (``teletron/training/training.py:47-125``)."""
    global _TIMERS
    parser = args_mod.build_parser(extra_args_provider)
    if args_defaults:
        parser.set_defaults(**args_defaults)
    args = parser.parse_known_args(argv)[0] if ignore_unknown_args else parser.parse_args(argv)
    args = args_mod.validate_args(args)
    args_mod.set_args(args)
    _TIMERS = Timers(args.timing_log_level, args.timing_log_option)
    if args.hang_dump_seconds > 0:
        import faulthandler
        faulthandler.dump_traceback_later(args.hang_dump_seconds, repeat=True)
    use_cuda = torch.cuda.is_available()
    if use_cuda:
        torch.cuda.set_device(args.local_rank % torch.cuda.device_count())
    if args.world_size > 1 and not dist.is_initialized():
        backend = args.distributed_backend or ("nccl" if use_cuda else "gloo")
        kw = {}
        # Eager NCCL initialisation (communicators split from the world one) is used unless encoder ranks stream to DiT
        # ranks: with it, point-to-point calls run on the group's collective communicator, and a two-rank stream group
        # that is not the whole world failed there ("Send: invalid root"); lazily initialised groups give every
        # send/recv pair its own two-rank communicator, the long-standing path.
        if use_cuda and backend == "nccl" and not args.distributed_vae:
            kw["device_id"] = torch.device("cuda", torch.cuda.current_device())
        dist.init_process_group(backend=backend, world_size=args.world_size, rank=args.rank,
                                timeout=datetime.timedelta(minutes=args.distributed_timeout_minutes), **kw)
    enc = args.distributed_vae_world_size if args.distributed_vae else 0
    ps.initialize_model_parallel(args.tensor_model_parallel_size, args.context_parallel_size, enc,
                                 timeout_minutes=args.distributed_timeout_minutes,
                                 pipeline_model_parallel_size=args.pipeline_model_parallel_size,
                                 virtual_pipeline_model_parallel_size=args.virtual_pipeline_model_parallel_size,
                                 expert_model_parallel_size=args.expert_model_parallel_size,
                                 nccl_communicator_config_path=args.nccl_communicator_config_path)
    if ps.is_dit_rank():
        set_random_seed(args.seed, args.data_parallel_random_init)
    if use_cuda:
        from ..ops import fallback
        fallback.set_strict(not args.allow_library_fallback)
    if args.fused_comm:
        from ..models.hunyuanvideo import blocks
        from ..parallel import symm_mem
        blocks.set_fused_comm(True)
        symm_mem.set_barrier_timeout_seconds(args.comm_barrier_timeout_seconds)
    args.device = torch.device("cuda", torch.cuda.current_device()) if use_cuda else torch.device("cpu")
    return args


def setup_model_and_optimizer(model_provider: Callable, args):
    """Model -> bf16 on device -> DDP over DP x CP -> sharded AdamW -> LR schedule -> checkpoint load."""
    timers = get_timers()
    timers("model-and-optimizer-setup", log_level=0).start()
    model = model_provider()
    model = model.to(device=args.device, dtype=args.params_dtype) if not getattr(model, "_placed", False) else model
    group = ps.get_data_parallel_group(with_context_parallel=True)
    bucket_bytes = (args.ddp_bucket_size * 2) if args.ddp_bucket_size else (512 << 20)
    ddp = DistributedDataParallel(model, group, use_distributed_optimizer=args.use_distributed_optimizer,
                                  overlap_grad_reduce=args.overlap_grad_reduce, bucket_bytes=bucket_bytes,
                                  check_for_nan_in_grad=args.check_for_nan_in_loss_and_grad,
                                  tp_group=ps.get_tensor_model_parallel_group(),
                                  fused_comm=args.fused_comm)
    if args.data_parallel_random_init:
        ddp.broadcast_params()
    master_mode = args.master_weight_mode if args.params_dtype != torch.float32 else "none"
    state_dtype = torch.bfloat16 if args.optimizer_state_dtype == "bf16" else torch.float32
    opt = DistributedOptimizer(ddp, lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=args.adam_eps,
                               weight_decay=args.weight_decay, clip_grad=args.clip_grad, master_mode=master_mode,
                               state_dtype=state_dtype)
    sched = OptimizerParamScheduler(opt, max_lr=args.lr, min_lr=args.min_lr, lr_warmup_steps=args.lr_warmup_iters,
                                    lr_decay_steps=args.lr_decay_iters, lr_decay_style=args.lr_decay_style)
    timers("model-and-optimizer-setup").stop()
    args.iteration = 0
    if args.load is not None:
        timers("load-checkpoint", log_level=0).start()
        args.iteration = load_checkpoint(ddp, opt, sched, args, strict=False)
        timers("load-checkpoint").stop()
    elif args.pretrained_checkpoint is not None:
        load_checkpoint(ddp, opt, sched, args, load_dir=args.pretrained_checkpoint, strict=False)
    return ddp, opt, sched


def train_step(forward_step_func, data_iterator, model: DistributedDataParallel, optimizer, scheduler, args):
    """zero grads -> micro-batches (forward + backward) -> grad sync -> optimizer -> LR schedule."""
    timers = get_timers()
    optimizer.zero_grad()
    losses = {}
    n_mb = args.num_microbatches
    for i in range(n_mb):
        ctx = model.no_sync() if i < n_mb - 1 else _nullcontext()
        with ctx:
            timers("forward", log_level=1).start()
            with nvtx_range("forward"):
                out, loss_func = forward_step_func(data_iterator, model)
                loss, reduced = loss_func(out)
            timers("forward").stop()
            timers("backward", log_level=1).start()
            with nvtx_range("backward"):
                (loss / n_mb).backward()
            timers("backward").stop()
        for k, v in reduced.items():
            losses.setdefault(k, []).append(v.detach() if torch.is_tensor(v) else torch.tensor(v))
    timers("grad-sync", log_level=1).start()
    with nvtx_range("grad-sync"):
        model.finish_grad_sync()
    timers("grad-sync").stop()
    if getattr(args, "comm_check_interval", 1) and _STEP_COUNTER[0] % max(1, getattr(args, "comm_check_interval", 1)) == 0:
        # a bounded device-side wait that ran out (a peer that stalled or left) has left this step's activations or
        # gradients incomplete: find out here, on every rank together, before the update is applied
        from ..ops import status as _status
        group = ps.get_transformer_model_group() if ps.model_parallel_is_initialized() else None
        _status.check_all(group, what=f"training step {_STEP_COUNTER[0]}")
    _STEP_COUNTER[0] += 1
    timers("optimizer", log_level=1).start()
    with nvtx_range("optimizer"):
        ok = optimizer.step()
    timers("optimizer").stop()
    if ok:
        scheduler.step(1)
    avg = {k: torch.stack([t.float().reshape(()) for t in v]).mean() for k, v in losses.items()}
    return avg, (0 if ok else 1), optimizer.last_grad_norm


_STEP_COUNTER = [0]


class _Peekable:
    """Iterator that can say whether another item exists (it keeps one item fetched ahead)."""

    _END = object()

    def __init__(self, it):
        self._it = iter(it)
        self._next = None
        self._primed = False

    def _prime(self):
        if not self._primed:
            self._next = next(self._it, self._END)
            self._primed = True

    def has_next(self) -> bool:
        self._prime()
        return self._next is not self._END

    def __iter__(self):
        return self

    def __next__(self):
        self._prime()
        if self._next is self._END:
            raise StopIteration
        item, self._primed = self._next, False
        return item


class _nullcontext:
    def __enter__(self):
        return None

    def __exit__(self, *a):
        return False


def average_losses_across_data_parallel_group(losses):
    """Mean of scalar losses over the data-parallel group (call site X17 of the reference)."""
    t = torch.stack([l.detach().float().reshape(()) for l in losses])
    g = ps.get_data_parallel_group()
    if g is not None:
        dist.all_reduce(t, group=g)
        t = t / dist.get_world_size(g)
    return t


def evaluate(forward_step_func, data_iterator, model, args, max_iters: Optional[int] = None) -> Dict[str, float]:
    """Mean of the reduced losses over ``eval_iters`` forward passes without gradients (the reference gets this loop from
    Megatron's ``evaluate_and_print_results``; its scripts set the interval so high that it never runs)."""
    n = args.eval_iters if max_iters is None else max_iters
    was_training = model.training
    model.eval()
    sums: Dict[str, float] = {}
    done = 0
    # the diffusion wrapper draws its noise from (seed, step): validation must not advance the training stream
    inner = model.module if hasattr(model, "module") else model
    saved_step = getattr(inner, "step", None)
    if saved_step is not None:
        inner.step = 1_000_000_007        # a fixed stream of its own: every validation sees the same noise and timesteps
    if data_iterator is not None and not isinstance(data_iterator, _Peekable):
        data_iterator = _Peekable(data_iterator)
    group = ps.get_transformer_model_group() if (ps.model_parallel_is_initialized() and dist.is_initialized()) else None
    with torch.no_grad():
        for _ in range(n):
            # Only the source rank of a TP x CP block holds the iterator; the others are already inside the batch broadcast
            # when it runs dry.  So the ranks agree BEFORE every batch: the minimum over the job of "I still have one".
            more = 1 if (data_iterator is None or data_iterator.has_next()) else 0
            if group is not None and dist.get_world_size(group) > 1:
                t = torch.tensor([more], dtype=torch.int32, device=args.device)
                dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
                more = int(t.item())
            if not more:
                break
            try:
                out, loss_func = forward_step_func(data_iterator, model)
            except StopIteration:
                break
            _, reduced = loss_func(out)
            for k, v in reduced.items():
                sums[k] = sums.get(k, 0.0) + float(v)
            done += 1
    if saved_step is not None:
        inner.step = saved_step
    if was_training:
        model.train()
    return {k: v / max(1, done) for k, v in sums.items()}


def train(forward_step_func, model, optimizer, scheduler, train_data_iterator, args, on_step_end=None,
          valid_data_iterator=None, do_valid: Optional[bool] = None):
    """``do_valid``: whether a validation set exists; only the source rank of each TP x CP block holds the iterator, so
    the other ranks (which take part through the batch broadcast) must be told."""
    if do_valid is None:
        do_valid = valid_data_iterator is not None
    if valid_data_iterator is not None:
        valid_data_iterator = _Peekable(valid_data_iterator)      # one wrapper for the whole run: it holds an item fetched ahead
    timers = get_timers()
    logger = MetricLogger(args.jsonl_log, args.tensorboard_dir, args.tensorboard_queue_size,
                          wandb_project=getattr(args, "wandb_project", None), wandb_name=getattr(args, "wandb_exp_name", None),
                          wandb_dir=getattr(args, "wandb_save_dir", None), config=vars(args))
    watchdog = StepWatchdog(args.step_timeout_seconds) if args.step_timeout_seconds > 0 else None
    model.train()
    iteration = args.iteration
    use_cuda = torch.cuda.is_available()
    tokens = getattr(args, "tokens_per_sample", None)
    flops = getattr(args, "flops_per_sample", None)
    peak = peak_bf16_tflops()
    skipped_total = 0
    while iteration < args.train_iters:
        if args.profile and use_cuda and iteration == args.profile_step_start and args.rank in args.profile_ranks:
            from .. import ops as _ops
            _ops.set_nvtx(True)
            torch.cuda.cudart().cudaProfilerStart()
        if watchdog:
            watchdog.beat(iteration)
        timers("interval-time", log_level=0).start()
        try:
            losses, skipped, grad_norm = train_step(forward_step_func, train_data_iterator, model, optimizer, scheduler, args)
        except CommTimeoutError as e:
            # every rank raises at the same point (the status is agreed on over the job): leave with the watchdog's exit
            # code so that the restart wrapper relaunches from the last checkpoint
            print(f"[rank {args.rank}] {e}", flush=True)
            if watchdog:
                watchdog.stop()
            logger.close()
            raise SystemExit(75)
        timers("interval-time").stop()
        iteration += 1
        skipped_total += skipped
        args.iteration = iteration
        args.consumed_train_samples += args.global_batch_size
        if iteration % args.log_interval == 0:
            stats = timers.collect(["interval-time"])
            ms = stats["interval-time"]["max_ms"] / args.log_interval if args.log_interval else 0.0
            metrics = {"elapsed_ms_per_iter": ms, "lr": optimizer.lr, "skipped": skipped_total,
                       "consumed_samples": args.consumed_train_samples}
            for k, v in losses.items():
                metrics[k] = float(v)
            if grad_norm is not None:
                metrics["grad_norm"] = grad_norm
            if ms > 0:
                sps = args.global_batch_size / (ms / 1e3)
                metrics["samples_per_s"] = sps
                metrics["frames_per_s"] = sps * args.num_frames
                if tokens:
                    metrics["tokens_per_s"] = sps * tokens
                if flops:
                    per_gpu = flops * sps / max(1, args.dit_world_size) / 1e12
                    metrics["tflops_per_gpu"] = per_gpu
                    metrics["mfu"] = per_gpu / peak
            if use_cuda:
                metrics["peak_mem_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
            line = f" iteration {iteration:8d}/{args.train_iters:8d} | consumed samples: {args.consumed_train_samples:12d}"
            line += f" | elapsed time per iteration (ms): {ms:.1f} | learning rate: {optimizer.lr:.3E}"
            line += f" | global batch size: {args.global_batch_size:5d}"
            for k, v in losses.items():
                line += f" | {k}: {float(v):.6E}"
            if grad_norm is not None:
                line += f" | grad norm: {grad_norm:.3f}"
            if "samples_per_s" in metrics:
                line += f" | samples/s: {metrics['samples_per_s']:.4f} | frames/s: {metrics['frames_per_s']:.2f}"
            if "mfu" in metrics:
                line += f" | TFLOP/s/GPU: {metrics['tflops_per_gpu']:.1f} | MFU: {metrics['mfu']:.3f}"
            line += f" | number of skipped iterations: {skipped:3d} |"
            print_rank_0(line)
            logger.log(iteration, metrics)
            if args.timing_log_level > 0:
                timers.log(normalizer=args.log_interval)
        if do_valid and args.eval_iters > 0 and args.eval_interval and iteration % args.eval_interval == 0:
            timers("evaluate", log_level=0).start()
            val = evaluate(forward_step_func, valid_data_iterator, model, args)
            timers("evaluate").stop()
            line = f" validation loss at iteration {iteration} | " + " | ".join(f"{k}: {v:.6E}" for k, v in val.items())
            print_rank_last(line)
            logger.log(iteration, {f"valid_{k}": v for k, v in val.items()})
        if on_step_end is not None:
            on_step_end(iteration, losses)
        if args.save and args.save_interval and iteration % args.save_interval == 0:
            save_checkpoint(iteration, model, optimizer, scheduler, args, _step_state(model))
        if args.profile and use_cuda and iteration == args.profile_step_end and args.rank in args.profile_ranks:
            torch.cuda.cudart().cudaProfilerStop()
            from .. import ops as _ops
            _ops.set_nvtx(False)
        if args.exit_interval and iteration % args.exit_interval == 0:
            break
    if watchdog:
        watchdog.stop()
    logger.close()
    return iteration


def _step_state(model):
    m = model.module if hasattr(model, "module") else model
    return {"pipeline_step": getattr(m, "step", 0)}


def build_train_valid_test_data_iterators(provider: Callable, args, dp_rank=None, dp_size=None):
    """Only the source rank of each TP x CP block builds a loader (``training.py:296-317``); the
    explicit ``dp_rank`` / ``dp_size`` serve encoder ranks building a consumer's loader."""
    is_src = ps.get_tensor_context_parallel_rank() == 0 or dp_rank is not None
    if not is_src:
        return None, None, None
    train_ds, valid_ds, test_ds = provider([args.train_iters * args.global_batch_size, 0, 0])
    mk = lambda ds, consumed: build_pretraining_data_loader(  # noqa: E731
        ds, consumed, args.micro_batch_size, args.dataloader_type, args.num_workers, args.seed, dp_rank, dp_size)
    tl = mk(train_ds, args.consumed_train_samples)
    vl = mk(valid_ds, 0) if valid_ds is not None else None
    tel = mk(test_ds, 0) if test_ds is not None else None
    it = lambda l: iter(l) if l is not None else None  # noqa: E731
    return it(tl), it(vl), it(tel)


def pretrain(train_valid_test_datasets_provider: Callable, model_provider: Callable, forward_step_func: Callable,
             producer_process: Optional[Callable] = None, extra_args_provider: Optional[Callable] = None,
             args_defaults: Optional[dict] = None, argv=None):
    """Full training program; encoder ranks branch into ``producer_process`` and never build the DiT."""
    args = initialize(extra_args_provider, argv, args_defaults)
    timers = get_timers()
    if not ps.is_dit_rank():
        if producer_process is None:
            raise RuntimeError("encoder ranks were requested but no producer_process was given")
        producer_process(args, train_valid_test_datasets_provider)
        if dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()
        return None
    start = torch.tensor([time.time()], dtype=torch.float64, device=args.device)
    if dist.is_initialized() and ps.get_transformer_model_group() is not None and args.dit_world_size > 1:
        dist.all_reduce(start, op=dist.ReduceOp.MIN, group=ps.get_transformer_model_group())
    print_rank_0(f"time to initialize (seconds): {time.time() - float(start):.3f}")
    model, optimizer, scheduler = setup_model_and_optimizer(model_provider, args)
    consumer = None
    train_it = valid_it = None
    if args.distributed_vae:
        from ..encoder_service import EncoderConsumer
        pairs = ps.get_consumer_pairs()
        if pairs:
            consumer = EncoderConsumer(pairs, args, device=args.device)
            consumer.handshake(args.iteration)
    else:
        timers("train/valid/test-data-iterators-setup", log_level=0).start()
        train_it, valid_it, _ = build_train_valid_test_data_iterators(train_valid_test_datasets_provider, args)
        timers("train/valid/test-data-iterators-setup").stop()
    args.encoder_consumer = consumer
    print_rank_0("done with setup ...")
    print_rank_0("training ...")
    do_valid = torch.tensor([1 if valid_it is not None else 0], device=args.device)
    if dist.is_initialized() and args.dit_world_size > 1:
        dist.all_reduce(do_valid, op=dist.ReduceOp.MAX, group=ps.get_transformer_model_group())
    iteration = train(forward_step_func, model, optimizer, scheduler, train_it, args, valid_data_iterator=valid_it,
                      do_valid=bool(do_valid.item()))
    if args.save and iteration != 0 and (not args.save_interval or iteration % args.save_interval != 0):
        save_checkpoint(iteration, model, optimizer, scheduler, args, _step_state(model))
    if consumer is not None:
        consumer.close()
    if dist.is_initialized():
        dist.barrier()
        if os.environ.get("TELETRON_B200_KEEP_PG") != "1":
            dist.destroy_process_group()
    return model
