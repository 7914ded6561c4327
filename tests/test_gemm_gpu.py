"""tcgen05 GEMM against an fp32 PyTorch matmul: all three operand layouts, tails in M / N / K, epilogues."""

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(128, 256, 64), (256, 512, 128), (300, 384, 200), (1000, 3072, 3072), (77, 128, 1024), (4096, 9216, 256),
          (130, 8, 8), (2048, 264, 72)]


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _mk(shape, g, k=1.0):
    return (torch.randn(*shape, device="cuda", generator=g) * k).bfloat16()


@pytest.mark.parametrize("M,N,K", SHAPES)
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_layouts(M, N, K, layout):
    from teletron_b200.ops import gemm_tcgen05 as G
    if layout == "tn" and M % 8:
        pytest.skip("tn needs M % 8 == 0")
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    if layout == "nt":
        a, b = _mk((M, K), g), _mk((N, K), g)
        ref = a.float() @ b.float().t()
    elif layout == "nn":
        a, b = _mk((M, K), g), _mk((K, N), g)
        ref = a.float() @ b.float()
    else:
        a, b = _mk((K, M), g), _mk((K, N), g)
        ref = a.float().t() @ b.float()
    assert G.supported(a, b, layout)
    c = G.gemm(a, b, layout)
    G.check_status()
    assert c.shape == (M, N)
    assert _rel(c, ref) < 6e-3, _rel(c, ref)
    # tails must not be written outside the output
    assert torch.isfinite(c).all()


def test_bias_and_gelu_epilogues():
    from teletron_b200.ops import gemm_tcgen05 as G
    g = torch.Generator(device="cuda").manual_seed(0)
    M, N, K = 520, 768, 320
    a, w, bias = _mk((M, K), g), _mk((N, K), g, 0.05), _mk((N,), g)
    u_ref = a.float() @ w.float().t() + bias.float()
    c = G.gemm(a, w, "nt", bias)
    assert _rel(c, u_ref) < 6e-3
    for epi, approx in ((1, "none"), (2, "tanh")):
        y, u = G.gemm(a, w, "nt", bias, epi=epi)
        assert _rel(u, u_ref) < 6e-3
        assert _rel(y, torch.nn.functional.gelu(u_ref, approximate=approx)) < 8e-3
    # dgrad with fused activation backward: (dy @ W) * gelu'(u)
    dy, w2 = _mk((M, 256), g), _mk((256, N), g, 0.05)
    uu = _mk((M, N), g)
    for epi, approx in ((3, "none"), (4, "tanh")):
        got = G.gemm(dy, w2, "nn", epi=epi, aux=uu)
        uf = uu.float().requires_grad_()
        torch.nn.functional.gelu(uf, approximate=approx).backward(dy.float() @ w2.float())
        assert _rel(got, uf.grad) < 8e-3
    G.check_status()


def test_strided_views_and_determinism():
    from teletron_b200.ops import gemm_tcgen05 as G
    g = torch.Generator(device="cuda").manual_seed(1)
    big = _mk((512, 1024), g)
    a = big[:, 256:768]                       # row pitch 1024, 512 columns
    w = _mk((384, 512), g)
    assert G.supported(a, w, "nt")
    c1 = G.gemm(a, w, "nt")
    assert _rel(c1, a.float() @ w.float().t()) < 6e-3
    for _ in range(10):
        assert torch.equal(G.gemm(a, w, "nt"), c1)
    G.check_status()


def test_large_k_weight_gradient_shape():
    from teletron_b200.ops import gemm_tcgen05 as G
    g = torch.Generator(device="cuda").manual_seed(2)
    tokens = 8200
    dy, x = _mk((tokens, 1536), g, 0.1), _mk((tokens, 768), g)
    dw = G.gemm(dy, x, "tn")
    G.check_status()
    assert _rel(dw, dy.float().t() @ x.float()) < 6e-3


@pytest.mark.parametrize("M,N,K,layout", [(300, 264, 192, "nt"), (130, 136, 320, "nn"), (264, 520, 200, "tn")])
def test_output_window_is_the_only_memory_written(M, N, K, layout):
    """The output is a window inside a larger buffer pre-filled with a guard pattern: rows above and below, and the
    columns left and right of the window, must come back untouched (ragged last tiles must not spill)."""
    from teletron_b200.ops import gemm_tcgen05 as G
    g = torch.Generator(device="cuda").manual_seed(M + N)
    if layout == "nt":
        a, b = _mk((M, K), g), _mk((N, K), g)
        ref = a.float() @ b.float().t()
    elif layout == "nn":
        a, b = _mk((M, K), g), _mk((K, N), g)
        ref = a.float() @ b.float()
    else:
        a, b = _mk((K, M), g), _mk((K, N), g)
        ref = a.float().t() @ b.float()
    pad_r, pad_c = 5, 8                                   # the column offset keeps the window 16-byte aligned
    guard = torch.full((M + 2 * pad_r, N + 2 * pad_c), -777.0, device="cuda", dtype=torch.bfloat16)
    window = guard[pad_r:pad_r + M, pad_c:pad_c + N]
    if not G.supported(a, b, layout):
        pytest.skip("shape outside the kernel's gate")
    G.gemm(a, b, layout, out=window)
    G.check_status()
    assert _rel(window, ref) < 8e-3
    mask = torch.ones_like(guard, dtype=torch.bool)
    mask[pad_r:pad_r + M, pad_c:pad_c + N] = False
    assert bool((guard[mask] == -777.0).all())


PAIR_SHAPES = [(256, 256, 64), (2560, 2048, 512), (2313, 2056, 200), (4096, 9216, 256), (1100, 4360, 72)]


@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
@pytest.mark.parametrize("layout", ["nt", "nn", "tn"])
def test_cta_pair_kernel_layouts(M, N, K, layout):
    """The CTA-pair kernel (cluster of 2, tcgen05.mma.cta_group::2, 256 x 256 tiles) on whole tiles and on M / N / K tails,
    forced for every shape, against fp32; two runs give the same bits."""
    from teletron_b200.ops import gemm_tcgen05 as G
    if layout == "tn" and M % 8:
        pytest.skip("tn needs M % 8 == 0")
    g = torch.Generator(device="cuda").manual_seed(M + N + K)
    if layout == "nt":
        a, b = _mk((M, K), g), _mk((N, K), g)
        ref = a.float() @ b.float().t()
    elif layout == "nn":
        a, b = _mk((M, K), g), _mk((K, N), g)
        ref = a.float() @ b.float()
    else:
        a, b = _mk((K, M), g), _mk((K, N), g)
        ref = a.float().t() @ b.float()
    old = (G.PAIR_KERNEL, G.PAIR_MIN_TILES)
    G.PAIR_KERNEL, G.PAIR_MIN_TILES = True, 1
    try:
        n0 = G.COUNTERS["pair"]
        c = torch.full((M + 2, N), float("nan"), device="cuda", dtype=torch.bfloat16)       # rows beyond M must stay untouched
        G.gemm(a, b, layout, out=c[:M])
        c2 = G.gemm(a, b, layout)
        G.check_status()
        assert G.COUNTERS["pair"] == n0 + 2
    finally:
        G.PAIR_KERNEL, G.PAIR_MIN_TILES = old
    assert torch.isnan(c[M:].float()).all()
    assert torch.isfinite(c[:M].float()).all()
    assert _rel(c[:M], ref) < 6e-3, _rel(c[:M], ref)
    assert torch.equal(c[:M], c2)


def test_cta_pair_kernel_epilogues():
    from teletron_b200.ops import gemm_tcgen05 as G
    g = torch.Generator(device="cuda").manual_seed(3)
    M, N, K = 1032, 1544, 320
    a, w, bias = _mk((M, K), g), _mk((N, K), g, 0.05), _mk((N,), g)
    u_ref = a.float() @ w.float().t() + bias.float()
    old = (G.PAIR_KERNEL, G.PAIR_MIN_TILES)
    G.PAIR_KERNEL, G.PAIR_MIN_TILES = True, 1
    try:
        assert _rel(G.gemm(a, w, "nt", bias), u_ref) < 6e-3
        for epi, approx in ((1, "none"), (2, "tanh")):
            y, u = G.gemm(a, w, "nt", bias, epi=epi)
            assert _rel(u, u_ref) < 6e-3
            assert _rel(y, torch.nn.functional.gelu(u_ref, approximate=approx)) < 8e-3
        dy, w2 = _mk((M, 256), g), _mk((256, N), g, 0.05)
        uu = _mk((M, N), g)
        for epi, approx in ((3, "none"), (4, "tanh")):
            got = G.gemm(dy, w2, "nn", epi=epi, aux=uu)
            uf = uu.float().requires_grad_()
            torch.nn.functional.gelu(uf, approximate=approx).backward(dy.float() @ w2.float())
            assert _rel(got, uf.grad) < 8e-3
        G.check_status()
    finally:
        G.PAIR_KERNEL, G.PAIR_MIN_TILES = old
