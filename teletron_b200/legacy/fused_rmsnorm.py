"""``fused_rmsnorm`` with the reference's entry points (``teletron_op/fused_rmsnorm/rms_ops.cpp:47-61``), served by the
sm_100a RMSNorm kernels: any row count (the reference's kernels assume multiples of 16, ``rms_forward.cu:58-99``), any
column count that is a multiple of 8, checked arguments, current stream.

The reference's backward reconstructs the normalised input as ``y / w``; this one is given the saved *input* ``x``
instead (argument ``x_or_y``), which stays finite when a weight is zero."""

import torch

from ..ops import _lib
from ..ops._lib import c_float, c_int, c_long, call, check, ptr, stream

BF16 = torch.bfloat16


def torch_launch_rms_forward(out, x, weight, invvar, rows: int, cols: int, eps: float = 1e-6):
    check(out, BF16, "out"), check(x, BF16, "x"), check(weight, BF16, "weight"), check(invvar, torch.float32, "invvar")
    if x.numel() != rows * cols or weight.numel() != cols:
        raise _lib.NativeError("shape mismatch")
    call("tt_rmsnorm_fwd", ptr(x), ptr(weight), ptr(out), ptr(invvar), c_long(rows), c_int(cols), c_float(eps), stream())


def torch_launch_rms_backward(dx, dweight, dout, x_or_y, weight, invvar, rows: int, cols: int):
    for t, n in ((dx, "dx"), (dweight, "dweight"), (dout, "dout"), (x_or_y, "x"), (weight, "weight")):
        check(t, BF16, n)
    check(invvar, torch.float32, "invvar")
    nblk = _lib.lib().tt_norm_partial_blocks(c_long(rows), c_int(1))
    partials = torch.empty(nblk * cols, dtype=torch.float32, device=dx.device)
    call("tt_rmsnorm_bwd", ptr(dout), ptr(x_or_y), ptr(weight), ptr(invvar), ptr(dx), ptr(partials), ptr(dweight),
         c_long(rows), c_int(cols), stream())
