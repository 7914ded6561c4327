"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some hosts of this library own every byte of device memory themselves (a C program with a fixed pool, a plugin in
another runtime) and cannot let a call allocate; ``tt_rmsnorm_bwd_noalloc`` keeps its scratch inside the library.
This test drives it with raw pointers only and checks it against the regular entry point (which takes the scratch
from the caller), twice in a row because both calls share the library's one scratch array.  The file name sorts last
so that a run stopping at the first failure has already been through every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def test_noalloc_rmsnorm_backward_matches_regular_entry_point():
    from teletron_b200.ops import _lib
    lib = _lib.lib()
    fn = lib.tt_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    dev = torch.device("cuda", 0)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    g = torch.Generator(device="cuda").manual_seed(11)
    # two different problems back to back: the second call finds the first call's leftovers in the shared scratch
    for rows, cols in ((5000, 128), (777, 1024)):
        x = torch.randn(rows, cols, device=dev, generator=g).bfloat16()
        w = (1 + 0.2 * torch.randn(cols, device=dev, generator=g)).bfloat16()
        dy = torch.randn(rows, cols, device=dev, generator=g).bfloat16()
        y = torch.empty_like(x)
        rstd = torch.empty(rows, dtype=torch.float32, device=dev)
        assert lib.tt_rmsnorm_fwd(vp(x), vp(w), vp(y), vp(rstd), ctypes.c_long(rows), ctypes.c_int(cols),
                                  ctypes.c_float(1e-6), stream) == 0
        # regular entry point: scratch supplied by the caller
        nblk = lib.tt_norm_partial_blocks(ctypes.c_long(rows), ctypes.c_int(1))
        partials = torch.empty(nblk * cols, dtype=torch.float32, device=dev)
        dx_ref, dw_ref = torch.empty_like(x), torch.empty(cols, dtype=torch.bfloat16, device=dev)
        assert lib.tt_rmsnorm_bwd(vp(dy), vp(x), vp(w), vp(rstd), vp(dx_ref), vp(partials), vp(dw_ref),
                                  ctypes.c_long(rows), ctypes.c_int(cols), stream) == 0
        # allocation-free entry point: outputs are preallocated here, nothing is allocated inside the call
        dx, dw = torch.empty_like(x), torch.empty(cols, dtype=torch.bfloat16, device=dev)
        # one call first, so that the one-time set-up (module load, symbol look-up) is not mistaken for an allocation
        assert fn(vp(dy), vp(x), vp(w), vp(rstd), vp(dx), vp(dw), ctypes.c_long(rows), ctypes.c_int(cols), stream) == 0
        dx.zero_()
        dw.zero_()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info(dev)        # the driver's view: sees a cudaMalloc that PyTorch's counter cannot
        rc = fn(vp(dy), vp(x), vp(w), vp(rstd), vp(dx), vp(dw), ctypes.c_long(rows), ctypes.c_int(cols), stream)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(dev)
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        assert free_after >= free_before, (free_before, free_after)
        assert torch.equal(dx, dx_ref)
        assert _rel(dw, dw_ref) < 1e-2
        # and against plain PyTorch in fp32: dx = rstd * (w dy - xhat * mean(w dy xhat)), dw = sum_rows dy * xhat
        xf, wf, dyf = x.float(), w.float(), dy.float()
        xhat = xf * rstd[:, None]
        wdy = wf * dyf
        dx32 = rstd[:, None] * (wdy - xhat * (wdy * xhat).mean(dim=1, keepdim=True))
        assert _rel(dx, dx32) < 1e-2
        assert _rel(dw, (dyf * xhat).sum(0)) < 1e-2
    # beyond the compiled-in maximum: refused with a clear code, nothing launched
    cols = 2048
    x = torch.zeros(8, cols, device=dev, dtype=torch.bfloat16)
    rc = fn(vp(x), vp(x), vp(x[0]), vp(torch.zeros(8, device=dev)), vp(x.clone()), vp(x[0].clone()), ctypes.c_long(8),
            ctypes.c_int(cols), stream)
    assert rc == 4          # TT_ERR_LIMIT
