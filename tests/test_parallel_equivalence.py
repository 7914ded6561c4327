"""TP / CP layouts must reproduce the single-process loss and gradients (the assertion the reference's
``test/test_scripts/run_test_cases.sh`` leaves to a human comparing two logs)."""

import pytest
import torch

from dist_utils import run_distributed


# tp * cp = 4 needs at least 4 heads: 4 x 32 instead of the tiny model's 2 x 64
HEADS4 = dict(num_attention_heads=4, attention_head_dim=32, rope_axes_dim=(8, 12, 12))


def _make_batch():
    g = torch.Generator().manual_seed(7)
    return dict(latents=torch.randn(1, 16, 3, 8, 8, generator=g), prompt_embeds=torch.randn(1, 16, 64, generator=g),
                clip_text_embed=torch.randn(1, 32, generator=g))


def _full_grads(pipe, tp, tp_group):
    """name -> full (unsharded) gradient, gathered over TP."""
    import torch.distributed as dist
    from teletron_b200.models.hunyuanvideo.model import unshard_tensors
    out = {}
    for n, p in pipe.transformer.named_parameters():
        g = p.grad.detach().clone()
        if tp > 1 and getattr(p, "partition_dim", None) is not None:
            parts = [torch.empty_like(g) for _ in range(tp)]
            dist.all_gather(parts, g, group=tp_group)
            g = unshard_tensors(parts, p.partition_dim, p.partitions)
        out[n] = g
    return out


def _run(rank, world, tp, cp, recompute, frames, sp=False, heads4=False):
    import torch.distributed as dist
    from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, tiny_config
    from teletron_b200.parallel import state as ps
    ps.initialize_model_parallel(tp, cp)
    torch.manual_seed(0)
    cfg = tiny_config(recompute_granularity="full" if recompute else None, sequence_parallel=sp, **(HEADS4 if heads4 else {}))
    pipe = HunyuanPipeline(cfg, FlowConfig(model_type="t2v"))
    batch = _make_batch()
    if frames != 3:
        g = torch.Generator().manual_seed(7)
        batch["latents"] = torch.randn(1, 16, frames, 6, 6, generator=g)
    loss = pipe(batch)[0]
    loss.backward()
    from teletron_b200.parallel.grad_buffer import allreduce_tp_partial_grads
    allreduce_tp_partial_grads(list(pipe.transformer.parameters()), ps.get_tensor_model_parallel_group())
    grads = _full_grads(pipe, tp, ps.get_tensor_model_parallel_group())
    # parameter grads are partial sums over CP ranks, scaled so that the DP x CP *average* is the true grad
    if cp > 1:
        for n in grads:
            dist.all_reduce(grads[n], group=ps.get_context_parallel_group())
            grads[n] /= cp
    return float(loss.detach()), {k: v for k, v in grads.items()}


def _single(recompute=False, frames=3, heads4=False):
    from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, tiny_config
    from teletron_b200.parallel import state as ps
    ps.destroy_model_parallel()
    torch.manual_seed(0)
    pipe = HunyuanPipeline(tiny_config(**(HEADS4 if heads4 else {})), FlowConfig(model_type="t2v"))
    batch = _make_batch()
    if frames != 3:
        g = torch.Generator().manual_seed(7)
        batch["latents"] = torch.randn(1, 16, frames, 6, 6, generator=g)
    loss = pipe(batch)[0]
    loss.backward()
    return float(loss.detach()), {n: p.grad.clone() for n, p in pipe.transformer.named_parameters()}


@pytest.mark.parametrize("tp,cp,recompute,frames", [(1, 2, False, 3), (2, 1, False, 3), (1, 2, True, 3), (1, 2, False, 5)])
def test_layout_matches_single_process(tp, cp, recompute, frames):
    # frames=5 with a 6x6 latent gives 45 video tokens: not divisible by cp=2 -> exercises the padding path
    ref_loss, ref_grads = _single(frames=frames)
    results = run_distributed(_run, 2, tp, cp, recompute, frames)
    for loss, grads in results:
        assert abs(loss - ref_loss) < 1e-5 * max(1.0, abs(ref_loss))
        for n, g in ref_grads.items():
            torch.testing.assert_close(grads[n], g, rtol=2e-4, atol=2e-6, msg=lambda m, n=n: f"{n}: {m}")


@pytest.mark.parametrize("world,tp,cp,recompute,frames", [(2, 2, 1, False, 3), (2, 2, 1, True, 3), (4, 2, 2, False, 3),
                                                          (4, 2, 2, False, 5)])
def test_sequence_parallel_matches_single_process(world, tp, cp, recompute, frames):
    """Token-sharded residual stream over TP (all-gather into column-parallel, reduce-scatter out of row-parallel
    linears): same loss and gradients as one process.  frames=5 gives 45 video tokens, padded to a multiple of cp*tp."""
    ref_loss, ref_grads = _single(frames=frames, heads4=world == 4)
    results = run_distributed(_run, world, tp, cp, recompute, frames, True, world == 4)
    for loss, grads in results:
        assert abs(loss - ref_loss) < 1e-5 * max(1.0, abs(ref_loss))
        for n, g in ref_grads.items():
            torch.testing.assert_close(grads[n], g, rtol=2e-4, atol=2e-6, msg=lambda m, n=n: f"{n}: {m}")
