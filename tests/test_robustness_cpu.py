"""Host-side failure handling of the training loop, on CPU: a status word set by a bounded device-side wait stops the step
before the optimizer update, and a validation set that runs dry ends the evaluation on every rank together."""

import os
import sys
import types

import pytest
import torch

from dist_utils import run_distributed

EXAMPLE = os.path.join(os.path.dirname(__file__), "..", "examples", "hunyuanvideo")


def test_train_step_raises_before_the_update_when_a_status_word_is_set():
    sys.path.insert(0, EXAMPLE)
    import pretrain_hunyuanvideo as entry
    from teletron_b200.ops import gemm_tcgen05
    from teletron_b200.ops._lib import CommTimeoutError
    from teletron_b200.training import initialize, setup_model_and_optimizer, train_step
    argv = ["--model-size", "tiny", "--dataset-type", "FakeDataset", "--num-frames", "9", "--video-resolution", "64", "64",
            "--text-len", "16", "--train-iters", "2", "--lr", "1e-3", "--num-workers", "0"]
    args = initialize(entry.extra_args_provider, argv)
    model, opt, sched = setup_model_and_optimizer(entry.model_provider, args)
    g = torch.Generator().manual_seed(0)
    batch = {"latents": torch.randn(1, 16, 3, 8, 8, generator=g), "prompt_embeds": torch.randn(1, 16, 64, generator=g),
             "clip_text_embed": torch.randn(1, 32, generator=g)}

    def fwd(_it, m):
        return m(batch), lambda out: (out[0].mean(), {"loss": out[0].mean().detach()})

    train_step(fwd, None, model, opt, sched, args)                      # a clean step goes through
    before = torch.cat([p.detach().reshape(-1).clone() for p in model.module.parameters()])
    word = torch.tensor([3, 0, 0, 0], dtype=torch.int32)               # what a kernel's timed-out wait leaves behind
    gemm_tcgen05._STATUS[torch.device("cpu")] = word
    try:
        with pytest.raises(CommTimeoutError):
            train_step(fwd, None, model, opt, sched, args)
        after = torch.cat([p.detach().reshape(-1) for p in model.module.parameters()])
        assert torch.equal(before, after), "the optimizer update was applied to a step with incomplete data"
        assert int(word[0]) == 0                                        # cleared, so the next step starts clean
        train_step(fwd, None, model, opt, sched, args)
    finally:
        gemm_tcgen05._STATUS.pop(torch.device("cpu"), None)


def _short_validation(rank, world):
    import torch.distributed as dist
    from teletron_b200.parallel import state as ps
    from teletron_b200.training.pretrain import evaluate
    ps.initialize_model_parallel(1, 2)
    model = torch.nn.Linear(2, 2)
    seen = []

    def forward_step(it, m):
        # the source rank of the TP x CP block reads the item, everyone takes part in the broadcast
        t = torch.zeros(1)
        if it is not None:
            t += next(it)
        dist.broadcast(t, src=0, group=ps.get_tensor_context_parallel_group())
        seen.append(float(t))
        return t, lambda out: (out.sum(), {"loss": out.sum()})

    args = types.SimpleNamespace(eval_iters=4, device=torch.device("cpu"))
    it = iter([torch.tensor([1.0]), torch.tensor([3.0])]) if rank == 0 else None
    res = evaluate(forward_step, it, model, args)
    ps.destroy_model_parallel()
    return res["loss"], seen


def test_validation_set_that_runs_dry_ends_on_all_ranks_together():
    out = run_distributed(_short_validation, 2, timeout=120)
    for loss, seen in out:
        assert seen == [1.0, 3.0] and loss == 2.0
