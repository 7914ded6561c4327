"""One place that reads every status word the kernels' bounded waits can set.

The tcgen05 kernels (``gemm_tcgen05.status_tensor``) and the device-side barriers of the symmetric heaps
(``SymmetricHeap._status``) record ``TT_ERR_TIMEOUT`` when a wait runs out and then return, so the CUDA context stays
usable - but the kernels queued behind them run on incomplete data.  :func:`check_all` is what a training step calls
at its synchronisation point, before the optimizer update: it reads all words with one device -> host copy, agrees on
the result across the job (so that every rank leaves the step together) and raises :class:`CommTimeoutError`.

The reference has no device-side waits of its own; its hangs surface as NCCL watchdog timeouts
(``teletron/training/training.py:47-125`` passes ``--distributed-timeout-minutes`` to ``init_process_group``).
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist

from . import _lib


def status_tensors(device: Optional[torch.device] = None) -> List[torch.Tensor]:
    from . import gemm_tcgen05
    from ..parallel import symm_mem
    out = [t for d, t in gemm_tcgen05._STATUS.items() if device is None or d == device]
    out += [h._status for h in list(symm_mem.LIVE_HEAPS) if device is None or h._status.device == device]
    return out


LAST_CHECK_HOST_TIME = 0.0      # host clock just before the last check blocked on the device (used by the step breakdown)


def check_all(group=None, device: Optional[torch.device] = None, what: str = "training step") -> None:
    """Raise :class:`teletron_b200.ops._lib.CommTimeoutError` on every rank of ``group`` if a bounded device-side wait ran
    out on any of them since the last check.  Costs one small all-reduce and one device -> host read."""
    if device is None and torch.cuda.is_available():
        device = torch.device("cuda", torch.cuda.current_device())       # one process drives one GPU
    words = status_tensors(device)
    multi = group is not None and dist.is_initialized() and dist.get_world_size(group) > 1
    if not words and not multi:
        return
    if words:
        code = torch.stack([w[0].to(torch.int32) for w in words]).max().reshape(1)
    else:
        on_gpu = torch.cuda.is_available() and dist.get_backend(group) == "nccl"
        code = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", torch.cuda.current_device()) if on_gpu else "cpu")
    global LAST_CHECK_HOST_TIME
    import time
    LAST_CHECK_HOST_TIME = time.perf_counter()
    if code.is_cuda and _lib.available():
        # the norm kernels' shared-memory rings report through a word inside the library (a 4-byte read that waits for the device)
        ns = int(_lib.lib().tt_norm_status())
        if ns:
            code = torch.maximum(code, torch.full_like(code, ns))
    local = code.clone()
    if multi:
        dist.all_reduce(code, op=dist.ReduceOp.MAX, group=group)
    worst = int(code.item())
    if worst:
        mine = int(local.item())
        for w in words:
            w.zero_()
        where = "on this rank" if mine else "on another rank"
        raise _lib.CommTimeoutError(f"{what}: a bounded device-side wait ran out {where} (status {worst}); the data of this "
                                    f"step is incomplete and the optimizer update was not applied")
