"""Numerics of every sm_100a kernel against the plain PyTorch fp32 reference of the same op."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _close(a, b, rtol=2e-2, atol=2e-2, name=""):
    torch.testing.assert_close(a.float(), b.float(), rtol=rtol, atol=atol, msg=lambda m: f"{name}: {m}")


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


@pytest.fixture(autouse=True)
def _native_loaded():
    from teletron_b200.ops import _lib
    assert _lib.available(), "native library must be built for GPU tests: " + _lib.load_error()


@pytest.mark.parametrize("B,S,C", [(1, 1000, 3072), (2, 77, 3072), (1, 513, 128), (3, 64, 8192), (1, 33, 1024)])
def test_layernorm_modulate(B, S, C):
    from teletron_b200.ops import cuda_ops, reference
    g = torch.Generator(device="cuda").manual_seed(0)
    x = (torch.randn(B, S, C, device=_dev(), generator=g) * 2 + 0.5).bfloat16().requires_grad_()
    sc = (torch.randn(B, C, device=_dev(), generator=g) * 0.3).bfloat16().requires_grad_()
    sh = (torch.randn(B, C, device=_dev(), generator=g) * 0.3).bfloat16().requires_grad_()
    dy = torch.randn(B, S, C, device=_dev(), generator=g).bfloat16()
    y = cuda_ops.layernorm_modulate(x, sc, sh, 1e-6)
    y.backward(dy)
    got = (y.detach(), x.grad.clone(), sc.grad.clone(), sh.grad.clone())
    xr, scr, shr = (t.detach().float().requires_grad_() for t in (x, sc, sh))
    yr = reference.layernorm_modulate(xr, scr, shr, 1e-6)
    yr.backward(dy.float())
    for a, b, n in zip(got, (yr.detach(), xr.grad, scr.grad, shr.grad), ("y", "dx", "dscale", "dshift")):
        assert _rel(a, b) < 1e-2, (n, _rel(a, b))


@pytest.mark.parametrize("B,S,C", [(1, 700, 3072), (2, 50, 256)])
def test_gate_residual_layernorm_modulate(B, S, C):
    from teletron_b200.ops import cuda_ops, reference
    g = torch.Generator(device="cuda").manual_seed(1)
    mk = lambda *s, k=1.0: (torch.randn(*s, device=_dev(), generator=g) * k).bfloat16().requires_grad_()  # noqa: E731
    res, br = mk(B, S, C), mk(B, S, C)
    gate, sc, sh = mk(B, C, k=0.5), mk(B, C, k=0.3), mk(B, C, k=0.3)
    d1 = torch.randn(B, S, C, device=_dev(), generator=g).bfloat16()
    d2 = torch.randn(B, S, C, device=_dev(), generator=g).bfloat16()
    nr, y = cuda_ops.gate_residual_layernorm_modulate(res, br, gate, sc, sh, 1e-6)
    torch.autograd.backward([nr, y], [d1, d2])
    got = [nr.detach(), y.detach()] + [t.grad.clone() for t in (res, br, gate, sc, sh)]
    refs = [t.detach().float().requires_grad_() for t in (res, br, gate, sc, sh)]
    # the kernel rounds the new residual to bf16 before normalising it: mirror that in the oracle
    nr_r = reference.gate_residual(*refs[:3])
    nr_q = nr_r + (nr_r.detach().bfloat16().float() - nr_r.detach())
    y_r = reference.layernorm_modulate(nr_q, refs[3], refs[4], 1e-6)
    torch.autograd.backward([nr_r, y_r], [d1.float(), d2.float()])
    want = [nr_r.detach(), y_r.detach()] + [t.grad for t in refs]
    for a, b, n in zip(got, want, ("new_res", "y", "dres", "dbranch", "dgate", "dscale", "dshift")):
        assert _rel(a, b) < 1.5e-2, (n, _rel(a, b))


def test_gate_residual():
    from teletron_b200.ops import cuda_ops, reference
    g = torch.Generator(device="cuda").manual_seed(2)
    res = torch.randn(2, 333, 3072, device=_dev(), generator=g).bfloat16().requires_grad_()
    br = torch.randn(2, 333, 3072, device=_dev(), generator=g).bfloat16().requires_grad_()
    gate = torch.randn(2, 3072, device=_dev(), generator=g).bfloat16().requires_grad_()
    d = torch.randn(2, 333, 3072, device=_dev(), generator=g).bfloat16()
    out = cuda_ops.gate_residual(res, br, gate)
    out.backward(d)
    refs = [t.detach().float().requires_grad_() for t in (res, br, gate)]
    o = reference.gate_residual(*refs)
    o.backward(d.float())
    assert _rel(out, o) < 1e-2
    for a, b in zip((res.grad, br.grad, gate.grad), (t.grad for t in refs)):
        assert _rel(a, b) < 1e-2


@pytest.mark.parametrize("rows,C", [(4097, 128), (100, 3072), (7, 64)])
def test_rmsnorm(rows, C):
    from teletron_b200.ops import cuda_ops, reference
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(rows, C, device=_dev(), generator=g).bfloat16().requires_grad_()
    w = (1 + 0.2 * torch.randn(C, device=_dev(), generator=g)).bfloat16().requires_grad_()
    d = torch.randn(rows, C, device=_dev(), generator=g).bfloat16()
    y = cuda_ops.rmsnorm(x, w, 1e-6)
    y.backward(d)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = reference.rmsnorm(xr, wr, 1e-6)
    yr.backward(d.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("B,S,T,heads", [(1, 300, 40, 3), (2, 130, 0, 2)])
def test_qkv_projection(B, S, T, heads):
    """QKV GEMM + split + QK-RMSNorm + RoPE + head-major layout, one and two streams, fwd and bwd."""
    from teletron_b200.ops import cuda_ops, reference
    H = heads * 128
    g = torch.Generator(device="cuda").manual_seed(4)
    mk = lambda *s, k=1.0: (torch.randn(*s, device=_dev(), generator=g) * k).bfloat16().requires_grad_()  # noqa: E731
    x, w, b = mk(B, S, H), mk(3 * H, H, k=0.03), mk(3 * H, k=0.1)
    qw, kw = mk(128, k=0.2), mk(128, k=0.2)
    ang = torch.rand(S, 64, device=_dev(), generator=g) * 6.28
    cos, sin = ang.cos().repeat_interleave(2, 1), ang.sin().repeat_interleave(2, 1)
    params = [x, w, b, qw, kw]
    if T:
        x2, w2, b2, qw2, kw2 = mk(B, T, H), mk(3 * H, H, k=0.03), mk(3 * H, k=0.1), mk(128, k=0.2), mk(128, k=0.2)
        params += [x2, w2, b2, qw2, kw2]
        q, k, v = cuda_ops.joint_qkv_projection(x, w, b, qw, kw, cos, sin, x2, w2, b2, qw2, kw2, heads, 1e-6)
    else:
        q, k, v = cuda_ops.qkv_projection(x, w, b, qw, kw, cos, sin, heads, 1e-6, rope_len=S - 30)
    douts = [torch.randn_like(q) for _ in range(3)]
    torch.autograd.backward([q, k, v], douts)
    refs = [p.detach().float().requires_grad_() for p in params]
    if T:
        qr, kr, vr = reference.joint_qkv_projection(*refs[:5], cos, sin, *refs[5:], heads, 1e-6)
    else:
        qr, kr, vr = reference.qkv_projection(*refs, cos[:S - 30], sin[:S - 30], heads, 1e-6, rope_len=S - 30)
    torch.autograd.backward([qr, kr, vr], [d.float() for d in douts])
    for a, r, n in zip((q, k, v), (qr, kr, vr), "qkv"):
        assert _rel(a, r) < 1.5e-2, (n, _rel(a, r))
    names = ["x", "w", "b", "qw", "kw", "x2", "w2", "b2", "qw2", "kw2"]
    for p, r, n in zip(params, refs, names):
        assert _rel(p.grad, r.grad) < 2e-2, (n, _rel(p.grad, r.grad))


@pytest.mark.parametrize("act", [None, "gelu", "gelu_tanh"])
def test_linear(act):
    from teletron_b200.ops import cuda_ops, reference
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.randn(2, 300, 512, device=_dev(), generator=g).bfloat16().requires_grad_()
    w = (torch.randn(1024, 512, device=_dev(), generator=g) * 0.05).bfloat16().requires_grad_()
    b = torch.randn(1024, device=_dev(), generator=g).bfloat16().requires_grad_()
    d = torch.randn(2, 300, 1024, device=_dev(), generator=g).bfloat16()
    y = cuda_ops.linear(x, w, b, act)
    y.backward(d)
    refs = [t.detach().float().requires_grad_() for t in (x, w, b)]
    yr = reference.linear(*refs, act)
    yr.backward(d.float())
    assert _rel(y, yr) < 1e-2
    for a, r in zip((x.grad, w.grad, b.grad), (t.grad for t in refs)):
        assert _rel(a, r) < 1.5e-2


def test_linear_merged_keeps_the_two_gradients_apart():
    """Projection of ``[x1 | x2]``: value and all four gradients against fp32; both halves of dW come from GEMMs that
    write column slices of one matrix, both input gradients from GEMMs that read column slices of the weight."""
    from teletron_b200.ops import cuda_ops, gemm, reference
    g = torch.Generator(device="cuda").manual_seed(6)
    x1 = torch.randn(1, 2104, 384, device=_dev(), generator=g).bfloat16().requires_grad_()
    x2 = torch.randn(1, 2104, 1536, device=_dev(), generator=g).bfloat16().requires_grad_()
    w = (torch.randn(768, 1920, device=_dev(), generator=g) * 0.05).bfloat16().requires_grad_()
    b = torch.randn(768, device=_dev(), generator=g).bfloat16().requires_grad_()
    d = torch.randn(1, 2104, 768, device=_dev(), generator=g).bfloat16()
    before = (gemm.COUNTERS["tcgen05"], gemm.COUNTERS["cublas"])
    y = cuda_ops.linear_merged(x1, x2, w, b)
    y.backward(d)
    assert gemm.COUNTERS["tcgen05"] - before[0] == 5 and gemm.COUNTERS["cublas"] == before[1]
    refs = [t.detach().float().requires_grad_() for t in (x1, x2, w, b)]
    yr = reference.linear_merged(*refs)
    yr.backward(d.float())
    assert _rel(y, yr) < 1e-2
    for a, r in zip((x1.grad, x2.grad, w.grad, b.grad), (t.grad for t in refs)):
        assert _rel(a, r) < 1.5e-2


@pytest.mark.parametrize("mode,state", [("fp32", torch.float32), ("split16", torch.bfloat16), ("none", torch.float32),
                                        ("split16", torch.float32)])
def test_adamw(mode, state):
    from teletron_b200.ops import cuda_ops
    from teletron_b200.ops.optim import _unpack16, adamw_update_reference
    n = 8 * 1000 + 8
    g = torch.Generator(device="cuda").manual_seed(6)
    p0 = torch.randn(n, device=_dev(), generator=g).bfloat16()
    sets = []
    for _ in range(2):
        p = p0.clone()
        m = torch.zeros(n, device=_dev(), dtype=state)
        v = torch.zeros(n, device=_dev(), dtype=state)
        master = p.float() if mode == "fp32" else None
        lo = torch.zeros(n, device=_dev(), dtype=torch.int16) if mode == "split16" else None
        sets.append((p, m, v, master, lo))
    for step in range(1, 4):
        grad = (torch.randn(n, device=_dev(), generator=g) * 0.1).bfloat16()
        kw = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=step, grad_scale=0.5)
        p, m, v, master, lo = sets[0]
        cuda_ops.adamw_update(p, grad, m, v, master, lo, **kw)
        p, m, v, master, lo = sets[1]
        adamw_update_reference(p, grad, m, v, master, lo, **kw)
    (pa, ma, va, msa, loa), (pb, mb, vb, msb, lob) = sets
    wa = msa if mode == "fp32" else (_unpack16(pa, loa) if mode == "split16" else pa.float())
    wb = msb if mode == "fp32" else (_unpack16(pb, lob) if mode == "split16" else pb.float())
    tol = 1e-5 if state == torch.float32 and mode != "none" else 2e-2
    assert _rel(wa, wb) < tol
    assert _rel(ma, mb) < 2e-2 and _rel(va, vb) < 2e-2


def test_block_cuda_matches_torch():
    """One dual + one single block at full width: CUDA op layer vs the PyTorch reference ops, loss and grads."""
    from teletron_b200 import ops
    from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, hunyuan_13b
    from teletron_b200.parallel import state as ps
    ps.destroy_model_parallel()
    dev = _dev()
    cfg = hunyuan_13b(in_channels=16, num_layers=1, num_single_layers=1)
    g = torch.Generator().manual_seed(0)
    batch = {"latents": torch.randn(1, 16, 2, 16, 16, generator=g), "prompt_embeds": torch.randn(1, 24, 4096, generator=g),
             "clip_text_embed": torch.randn(1, 768, generator=g)}
    out = {}
    for impl in ("torch", "cuda"):
        with ops.impl(impl):
            pipe = HunyuanPipeline(cfg, FlowConfig(model_type="t2v"), device=dev, dtype=torch.bfloat16)
            loss = pipe(batch)[0]
            loss.backward()
            out[impl] = (float(loss.detach()), {n: p.grad.float().clone() for n, p in pipe.transformer.named_parameters()
                                      if p.grad is not None})
    assert abs(out["cuda"][0] - out["torch"][0]) < 2e-2 * abs(out["torch"][0])
    bad = []
    for n, gt in out["torch"][1].items():
        if n.endswith("to_k.bias"):
            continue        # softmax is invariant to a shift of all keys: this gradient is pure rounding noise
        r = _rel(out["cuda"][1][n], gt)
        if r > 0.08:
            bad.append((n, r))
    assert not bad, bad[:10]


def test_recompute_with_saved_attention_matches_plain_recompute():
    """The block checkpoint that replays attention from the saved (out, lse) gives the same loss and gradients."""
    from teletron_b200 import ops
    from teletron_b200.models.hunyuanvideo import FlowConfig, HunyuanPipeline, hunyuan_13b
    from teletron_b200.ops import attention_backend
    from teletron_b200.parallel import state as ps
    ps.destroy_model_parallel()
    dev = _dev()
    g = torch.Generator().manual_seed(0)
    batch = {"latents": torch.randn(1, 16, 2, 16, 16, generator=g), "prompt_embeds": torch.randn(1, 24, 4096, generator=g),
             "clip_text_embed": torch.randn(1, 768, generator=g)}
    out = {}
    with ops.impl("cuda"):
        for save in (False, True):
            cfg = hunyuan_13b(in_channels=16, num_layers=1, num_single_layers=1, recompute_granularity="full",
                              recompute_save_attention=save)
            pipe = HunyuanPipeline(cfg, FlowConfig(model_type="t2v"), device=dev, dtype=torch.bfloat16)
            before = attention_backend.COUNTERS["tcgen05"]
            loss = pipe(batch)[0]
            loss.backward()
            out[save] = (float(loss.detach()), torch.cat([p.grad.float().reshape(-1) for p in pipe.transformer.parameters()
                                                         if p.grad is not None]),
                         attention_backend.COUNTERS["tcgen05"] - before)
    assert out[True][0] == out[False][0]
    assert _rel(out[True][1], out[False][1]) < 1e-3


def test_flow_noise_mix_and_loss_with_gradient():
    """Noise mix and weighted flow-matching loss (one kernel each) against fp32 PyTorch, gradient included."""
    from teletron_b200 import ops
    from teletron_b200.ops import reference
    g = torch.Generator(device="cuda").manual_seed(21)
    B, shape = 2, (2, 16, 3, 12, 20)
    lat, noise = (torch.randn(shape, device="cuda", generator=g).bfloat16() for _ in range(2))
    sigma = torch.rand(B, device="cuda", generator=g)
    mixed = ops.noise_mix(lat, noise, sigma)
    want = (1 - sigma.view(B, 1, 1, 1, 1)) * lat.float() + sigma.view(B, 1, 1, 1, 1) * noise.float()
    assert _rel(mixed, want) < 6e-3
    pred = torch.randn(shape, device="cuda", generator=g).bfloat16().requires_grad_()
    weight = torch.rand(B, device="cuda", generator=g) + 0.5
    loss = ops.flow_match_loss(pred, noise, lat, weight)
    (loss * 3.0).backward()
    ref_pred = pred.detach().float().requires_grad_()
    ref = reference.flow_match_loss(ref_pred, noise, lat, weight)
    (ref * 3.0).backward()
    assert abs(float(loss) - float(ref)) < 1e-4 * abs(float(ref))
    assert _rel(pred.grad, ref_pred.grad) < 6e-3
    # same bits on a second run: the partial sums are added in a fixed order
    assert float(ops.flow_match_loss(pred.detach(), noise, lat, weight)) == float(loss)
