"""Compute + collective fused kernels on 2 GPUs (child processes, NCCL rendezvous on 127.0.0.1, NVLS off), each
checked against the unfused NCCL / PyTorch composition of the same op; plus the bounded-wait status path on 1 GPU."""

import ctypes
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run_ranks(body: str, world: int = 2, timeout: int = 600):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    script = textwrap.dedent("""
        import os, sys, torch, torch.distributed as dist
        sys.path.insert(0, %r)
        rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
        def rel(a, b):
            return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()
    """ % ROOT) + textwrap.dedent(body) + textwrap.dedent("""
        torch.cuda.synchronize()
        dist.barrier()
        dist.destroy_process_group()
        print("RANK_OK", rank)
    """)
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        procs.append(subprocess.Popen([sys.executable, "-c", script], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and "RANK_OK" in out, f"rank {r} failed:\n{out[-4000:]}"
    return outs


def test_barrier_wait_runs_out_and_reports_status():
    """A flag that nothing sets: the barrier kernel gives up after its cycle budget and records a status word;
    the context stays usable (no trap, no hang)."""
    from teletron_b200.ops import _lib
    from teletron_b200.ops._lib import call
    dev = torch.device("cuda", 0)
    mine = torch.zeros(512, dtype=torch.int64, device=dev)
    silent_peer = torch.zeros(512, dtype=torch.int64, device=dev)      # stands in for a rank that never arrives
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    table = (ctypes.c_void_p * 2)(mine.data_ptr(), silent_peer.data_ptr())
    call("tt_comm_barrier", table, ctypes.c_int(0), ctypes.c_int(2), ctypes.c_ulonglong(1), ctypes.c_longlong(2_000_000),
         _lib.ptr(status), _lib.stream())
    torch.cuda.synchronize()
    assert int(status[0]) == 3                       # TT_ERR_TIMEOUT
    assert int(silent_peer[0]) == 1                  # our own arrival was published
    assert torch.ones(4, device=dev).sum().item() == 4.0     # the context still works


def test_tp_all_gather_gemm_and_gemm_reduce_scatter():
    _run_ranks("""
        from teletron_b200.ops import fused_comm as FC
        g = torch.Generator(device="cuda").manual_seed(5)
        rows, K, N = 384, 512, 768
        x_full = torch.randn(world * rows, K, device="cuda", generator=g).bfloat16()
        w_full = (torch.randn(N, K, device="cuda", generator=g) * 0.05).bfloat16()
        bias = torch.randn(N, device="cuda", generator=g).bfloat16()
        ws = FC.TPWorkspace(dist.group.WORLD, rows, K, N)
        # all-gather -> GEMM (column-parallel shard of the weight rows)
        w_col = w_full[rank * N // world:(rank + 1) * N // world].contiguous()
        y = FC.fused_all_gather_linear(ws, x_full[rank * rows:(rank + 1) * rows].contiguous(), w_col, bias[rank * N // world:(rank + 1) * N // world].contiguous())
        ref = x_full.float() @ w_col.float().t() + bias[rank * N // world:(rank + 1) * N // world].float()
        assert rel(y, ref) < 8e-3, rel(y, ref)
        # GEMM -> reduce-scatter (row-parallel shard of the weight columns)
        ks = K // world
        xk = x_full[:, rank * ks:(rank + 1) * ks].contiguous()
        wk = w_full[:, rank * ks:(rank + 1) * ks].contiguous()
        z = FC.fused_linear_reduce_scatter(ws, xk, wk, bias)
        zref = (x_full.float() @ w_full.float().t() + bias.float())[rank * rows:(rank + 1) * rows]
        assert rel(z, zref) < 1e-2, rel(z, zref)
        for _ in range(3):       # reuse of the staging buffers across calls
            z2 = FC.fused_linear_reduce_scatter(ws, xk, wk, bias)
            assert torch.equal(z2, z)
        ws.heap.check()
    """)


def test_sequence_parallel_mlp_fused_matches_nccl_path():
    """The model's MLP under sequence parallelism: fused all-gather -> GEMM / GEMM -> reduce-scatter (forward and
    backward) against the NCCL all-gather / reduce-scatter composition; 1100 rows per rank (not a tile multiple)."""
    _run_ranks("""
        from teletron_b200.parallel import state as ps
        from teletron_b200.models.hunyuanvideo import blocks as B
        ps.initialize_model_parallel(world, 1)
        torch.manual_seed(3)
        rows, dim, hidden = 1100, 512, 1536
        mlp = B.ParallelMLP(dim, hidden, "gelu_tanh", tp=world, sequence_parallel=True, device="cuda", dtype=torch.bfloat16)
        g = torch.Generator(device="cuda").manual_seed(11 + rank)
        with torch.no_grad():
            for p_ in mlp.parameters():
                p_.copy_((torch.randn(p_.shape, device="cuda", generator=g) * 0.05).to(p_.dtype))
        x = torch.randn(1, rows, dim, device="cuda", generator=g).bfloat16()
        dy = torch.randn(1, rows, dim, device="cuda", generator=g).bfloat16()
        res = {}
        for fused in (False, True, True):
            B.set_fused_comm(fused)
            xi = x.clone().requires_grad_(True)
            for p_ in mlp.parameters():
                p_.grad = None
            y = mlp(xi)
            y.backward(dy)
            res[fused] = [y.detach(), xi.grad] + [p_.grad.clone() for p_ in mlp.parameters()]
        names = ["y", "dx"] + [n for n, _ in mlp.named_parameters()]
        for n, a, b in zip(names, res[True], res[False]):
            assert torch.isfinite(a.float()).all(), n
            assert rel(a, b) < 1.5e-2, (n, rel(a, b))
        for ws in B._WORKSPACES.values():
            ws.heap.check()
    """)


def test_grad_reduce_scatter_and_param_all_gather():
    _run_ranks("""
        from teletron_b200.ops import fused_comm as FC
        from teletron_b200.parallel.symm_mem import SymmetricHeap
        n = 8 * 4096
        heap = SymmetricHeap(dist.group.WORLD, 4 * n + 4096)
        goff, poff = heap.alloc(2 * n), heap.alloc(2 * n)
        g = torch.Generator(device="cuda").manual_seed(100 + rank)
        grad = heap.tensor(goff, (n,), torch.bfloat16)
        grad.copy_(torch.randn(n, device="cuda", generator=g).bfloat16())
        all_grads = [torch.empty(n, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        dist.all_gather(all_grads, grad.clone())
        shard = n // world
        out = torch.empty(shard, device="cuda", dtype=torch.bfloat16)
        heap.barrier()
        FC.fused_grad_reduce_scatter(heap, goff, rank * shard, shard, out, 1.0 / world)
        heap.barrier()
        ref = sum(t.float() for t in all_grads)[rank * shard:(rank + 1) * shard] / world
        assert rel(out, ref) < 5e-3
        FC.fused_param_all_gather(heap, poff, rank * shard, out)
        heap.barrier()
        params = heap.tensor(poff, (n,), torch.bfloat16)
        gathered = [torch.empty(shard, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
        dist.all_gather(gathered, out)
        assert torch.equal(params, torch.cat(gathered))
        heap.check()
    """)


def test_fused_ulysses_model_matches_nccl_path():
    """One dual + one single block at full width, cp = 2: loss and gradients of the fused-collective path against the
    NCCL all_to_all path."""
    _run_ranks("""
        from teletron_b200 import ops
        from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, hunyuan_13b
        from teletron_b200.models.hunyuanvideo import blocks
        from teletron_b200.parallel import state as ps
        ps.initialize_model_parallel(1, 2)
        cfg = hunyuan_13b(in_channels=16, num_layers=1, num_single_layers=1, recompute_granularity="full")
        gen = torch.Generator().manual_seed(0)
        batch = {"latents": torch.randn(1, 16, 3, 30, 34, generator=gen), "prompt_embeds": torch.randn(1, 40, 4096, generator=gen),
                 "clip_text_embed": torch.randn(1, 768, generator=gen)}       # 3*15*17 = 765 video tokens: odd -> padded to 766
        res = {}
        # poison recycled allocator blocks so that any buffer a kernel leaves partly unwritten shows up as NaN
        junk = [torch.full((64 << 20,), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(8)]
        del junk
        from teletron_b200.parallel.grad_buffer import DistributedDataParallel
        for fused in (True, False):
            blocks.set_fused_comm(fused)
            pipe = HunyuanPipeline(cfg, FlowConfig(model_type="t2v"), device=torch.device("cuda", rank), dtype=torch.bfloat16)
            ddp = DistributedDataParallel(pipe, ps.get_data_parallel_group(with_context_parallel=True))
            for it in range(2):
                ddp.zero_grad_buffer()
                pipe.step = 0
                loss = pipe(batch)[0]
                loss.backward()
            res[fused] = (float(loss.detach()), {n: p.grad.float().clone() for n, p in pipe.transformer.named_parameters() if p.grad is not None})
            assert all(torch.isfinite(g).all() for g in res[fused][1].values()), "non-finite gradient"
        assert abs(res[True][0] - res[False][0]) < 2e-2 * abs(res[False][0]), (res[True][0], res[False][0])
        bad = []
        for n, gref in res[False][1].items():
            if n.endswith("to_k.bias"):
                continue
            r = rel(res[True][1][n], gref)
            if r > 0.08:
                bad.append((n, r))
        assert not bad, bad[:8]
        from teletron_b200.ops.gemm_tcgen05 import check_status
        check_status()
    """, timeout=900)


def test_fused_ulysses_several_layers_without_per_block_recompute():
    """Two dual + two single blocks, cp = 2, first without recompute and then with two blocks per checkpoint: every layer
    shares one collective workspace, so the tensors that the fused ops save for backward must be private copies; loss and
    gradients against the NCCL all_to_all path."""
    _run_ranks("""
        from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, hunyuan_13b
        from teletron_b200.models.hunyuanvideo import blocks
        from teletron_b200.ops import fused_comm as FC
        from teletron_b200.parallel import state as ps
        from teletron_b200.parallel.grad_buffer import DistributedDataParallel
        ps.initialize_model_parallel(1, 2)
        gen = torch.Generator().manual_seed(0)
        batch = {"latents": torch.randn(1, 16, 3, 30, 34, generator=gen), "prompt_embeds": torch.randn(1, 40, 4096, generator=gen),
                 "clip_text_embed": torch.randn(1, 768, generator=gen)}
        mask = torch.zeros(1, 40, dtype=torch.bool)
        mask[:, :25] = True                     # 15 padded text tokens: a masked key range at the head of the fused layout
        batch["prompt_attention_mask"] = mask
        for kw in (dict(recompute_granularity=None, apply_text_mask=True),
                   dict(recompute_granularity="full", recompute_method="uniform", recompute_num_layers=2)):
            cfg = hunyuan_13b(in_channels=16, num_layers=2, num_single_layers=2, **kw)
            res = {}
            for fused in (True, False):
                blocks.set_fused_comm(fused)
                saves0 = FC.COUNTERS["private_saves"]
                pipe = HunyuanPipeline(cfg, FlowConfig(model_type="t2v"), device=torch.device("cuda", rank), dtype=torch.bfloat16)
                ddp = DistributedDataParallel(pipe, ps.get_data_parallel_group(with_context_parallel=True))
                ddp.zero_grad_buffer()
                pipe.step = 0
                loss = pipe(batch)[0]
                loss.backward()
                res[fused] = (float(loss.detach()), {n: p.grad.float().clone() for n, p in pipe.transformer.named_parameters() if p.grad is not None})
                if fused:
                    assert FC.COUNTERS["private_saves"] > saves0, "no private copies were taken"
                del pipe, ddp
            assert abs(res[True][0] - res[False][0]) < 2e-2 * abs(res[False][0]), (kw, res[True][0], res[False][0])
            bad = []
            for n, gref in res[False][1].items():
                if n.endswith("to_k.bias"):
                    continue
                r = rel(res[True][1][n], gref)
                if r > 0.08:
                    bad.append((n, r))
            assert not bad, (kw, bad[:8])
        from teletron_b200.ops.gemm_tcgen05 import check_status
        check_status()
    """, timeout=900)


def test_fused_workspace_is_reused_across_clip_lengths():
    """Clips of different lengths through one model: the collective workspace is re-laid-out in place for a shorter clip and
    replaced (collectively) by a larger one for a longer clip; the loss of every clip equals the NCCL path's."""
    _run_ranks("""
        from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, hunyuan_13b
        from teletron_b200.models.hunyuanvideo import blocks
        from teletron_b200.parallel import state as ps
        ps.initialize_model_parallel(1, 2)
        cfg = hunyuan_13b(in_channels=16, num_layers=1, num_single_layers=1, recompute_granularity="full")
        gen = torch.Generator().manual_seed(0)
        def clip(f, h, w):
            return {"latents": torch.randn(1, 16, f, h, w, generator=gen), "prompt_embeds": torch.randn(1, 40, 4096, generator=gen),
                    "clip_text_embed": torch.randn(1, 768, generator=gen)}
        clips = [clip(3, 30, 34), clip(3, 30, 50), clip(2, 30, 34), clip(3, 30, 50)]
        pipe = HunyuanPipeline(cfg, FlowConfig(model_type="t2v"), device=torch.device("cuda", rank), dtype=torch.bfloat16)
        losses = {}
        for fused in (True, False):
            blocks.set_fused_comm(fused)
            out = []
            for i, b in enumerate(clips):
                for p_ in pipe.parameters():
                    p_.grad = None
                pipe.step = i
                loss = pipe(b)[0]
                loss.backward()
                out.append((float(loss.detach()), float(sum(p_.grad.float().abs().sum() for p_ in pipe.transformer.parameters() if p_.grad is not None))))
            losses[fused] = out
        kinds = [k for k in blocks._WORKSPACES if k[0] == "ulysses"]
        assert len(kinds) == 1, kinds                    # one workspace served all four clips
        for (a, ga), (b, gb) in zip(losses[True], losses[False]):
            assert abs(a - b) < 2e-2 * abs(b), (losses[True], losses[False])
            assert abs(ga - gb) < 5e-2 * abs(gb), (ga, gb)
        from teletron_b200.ops.gemm_tcgen05 import check_status
        check_status()
        for ws in blocks._WORKSPACES.values():
            ws.heap.check()
    """, timeout=900)


def test_sequence_parallel_model_fused_matches_plain_tensor_parallel():
    """One dual + one single block at full width, tp = 2: token-sharded residual stream with the fused all-gather -> GEMM /
    GEMM -> reduce-scatter MLPs against plain tensor parallelism (replicated activations, NCCL all-reduce)."""
    _run_ranks("""
        from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, hunyuan_13b
        from teletron_b200.models.hunyuanvideo import blocks
        from teletron_b200.parallel import state as ps
        from teletron_b200.parallel.grad_buffer import allreduce_tp_partial_grads
        ps.initialize_model_parallel(2, 1)
        gen = torch.Generator().manual_seed(0)
        batch = {"latents": torch.randn(1, 16, 3, 60, 64, generator=gen), "prompt_embeds": torch.randn(1, 40, 4096, generator=gen),
                 "clip_text_embed": torch.randn(1, 768, generator=gen)}       # 3*30*32 = 2880 video tokens: 1440 per rank
        junk = [torch.full((64 << 20,), float("nan"), device="cuda", dtype=torch.bfloat16) for _ in range(8)]
        del junk
        res = {}
        for sp in (True, False):
            blocks.set_fused_comm(sp)
            cfg = hunyuan_13b(in_channels=16, num_layers=1, num_single_layers=1, recompute_granularity="full", sequence_parallel=sp)
            pipe = HunyuanPipeline(cfg, FlowConfig(model_type="t2v"), device=torch.device("cuda", rank), dtype=torch.bfloat16)
            for it in range(2):
                for p_ in pipe.transformer.parameters():
                    p_.grad = None
                pipe.step = 0
                loss = pipe(batch)[0]
                loss.backward()
            allreduce_tp_partial_grads(list(pipe.transformer.parameters()), ps.get_tensor_model_parallel_group())
            res[sp] = (float(loss.detach()), {n: p_.grad.float().clone() for n, p_ in pipe.transformer.named_parameters() if p_.grad is not None})
            assert all(torch.isfinite(g).all() for g in res[sp][1].values()), "non-finite gradient"
        assert abs(res[True][0] - res[False][0]) < 2e-2 * abs(res[False][0]), (res[True][0], res[False][0])
        bad = []
        for n, gref in res[False][1].items():
            if n.endswith("to_k.bias"):
                continue
            r = rel(res[True][1][n], gref)
            if r > 0.08:
                bad.append((n, r))
        assert not bad, bad[:8]
        from teletron_b200.ops.gemm_tcgen05 import check_status
        check_status()
        for ws in blocks._WORKSPACES.values():
            ws.heap.check()
    """, timeout=900)
