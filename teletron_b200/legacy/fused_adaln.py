"""``fused_adaln`` with the reference's entry points (``teletron_op/fused_adaln/adaln_ops.cpp:52-65``), served by the
sm_100a LayerNorm + modulation kernels.  Unlike the reference's binding (``adaln_ops.cpp:6-50``) every argument is
checked for dtype, device, contiguity and shape, any column count that is a multiple of 8 is accepted, and launches go
to the caller's current stream.

``torch_launch_adaln_forward(out, x, scale, shift, x_norm, invvar, rows, cols, eps)`` writes
``out = LN(x) * (1 + scale) + shift``, ``x_norm = LN(x)`` and ``invvar = rstd``;
``torch_launch_adaln_backward(dx, dscale, dshift, dout, x_norm, scale, invvar, rows, cols)`` consumes them."""

import torch

from ..ops import _lib
from ..ops._lib import c_float, c_int, c_long, call, check, ptr, stream

BF16 = torch.bfloat16


def torch_launch_adaln_forward(out, x, scale, shift, x_norm, invvar, rows: int, cols: int, eps: float = 1e-6):
    for t, n in ((out, "out"), (x, "x"), (scale, "scale"), (shift, "shift"), (x_norm, "x_norm")):
        check(t, BF16, n)
    check(invvar, torch.float32, "invvar")
    if x.numel() != rows * cols or scale.numel() != cols or shift.numel() != cols:
        raise _lib.NativeError("shape mismatch")
    mean = torch.empty(rows, dtype=torch.float32, device=x.device)
    call("tt_ln_mod_fwd", ptr(x), ptr(None), ptr(None), ptr(scale), ptr(shift), ptr(None), ptr(out), ptr(mean), ptr(invvar),
         c_long(rows), c_int(cols), c_long(rows), c_float(eps), stream())
    x_norm.copy_(((x.float().view(rows, cols) - mean[:, None]) * invvar[:, None]).to(BF16).view_as(x_norm))


def torch_launch_adaln_backward(dx, dscale, dshift, dout, x_norm, scale, invvar, rows: int, cols: int):
    for t, n in ((dx, "dx"), (dscale, "dscale"), (dshift, "dshift"), (dout, "dout"), (x_norm, "x_norm"), (scale, "scale")):
        check(t, BF16, n)
    check(invvar, torch.float32, "invvar")
    # x_norm is already normalised: feed it as the input with mean 0 and rstd 1, then apply the saved rstd
    zeros = torch.zeros(rows, dtype=torch.float32, device=dx.device)
    ones = torch.ones(rows, dtype=torch.float32, device=dx.device)
    nblk = _lib.lib().tt_norm_partial_blocks(c_long(rows), c_int(1))
    partials = torch.empty(nblk * 2 * cols, dtype=torch.float32, device=dx.device)
    call("tt_ln_mod_bwd", ptr(dout), ptr(None), ptr(x_norm), ptr(None), ptr(None), ptr(scale), ptr(zeros), ptr(ones), ptr(dx),
         ptr(None), ptr(partials), ptr(dscale), ptr(dshift), ptr(None), c_long(rows), c_int(cols), c_long(rows), stream())
    dx.copy_((dx.float().view(rows, cols) * invvar[:, None]).to(BF16).view_as(dx))
