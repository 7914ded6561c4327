"""Spawn helper for multi-process CPU tests (gloo, file-store rendezvous: no ports, no hostnames)."""

import os
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world_size, init_file, fn, args, ret):
    try:
        os.environ["RANK"] = str(rank)
        os.environ["WORLD_SIZE"] = str(world_size)
        os.environ["LOCAL_RANK"] = str(rank)
        torch.set_num_threads(2)
        dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world_size)
        out = fn(rank, world_size, *args)
        ret[rank] = ("ok", out)
    except Exception:
        ret[rank] = ("error", traceback.format_exc())
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_distributed(fn, world_size, *args, timeout=240):
    """Run ``fn(rank, world_size, *args)`` on ``world_size`` gloo ranks; returns the list of results."""
    ctx = mp.get_context("spawn")
    mgr = ctx.Manager()
    ret = mgr.dict()
    fd, init_file = tempfile.mkstemp(prefix="ttb200_pg_")
    os.close(fd)
    os.unlink(init_file)
    procs = [ctx.Process(target=_worker, args=(r, world_size, init_file, fn, args, ret)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    for p in procs:
        if p.is_alive():
            p.terminate()
            raise RuntimeError("distributed test timed out")
    results = []
    for r in range(world_size):
        status, out = ret.get(r, ("error", "no result (process died)"))
        if status != "ok":
            raise RuntimeError(f"rank {r} failed:\n{out}")
        results.append(out)
    if os.path.exists(init_file):
        os.unlink(init_file)
    return results
