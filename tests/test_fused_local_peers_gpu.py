"""The compute + collective fused kernels on ONE GPU, each checked against plain PyTorch in fp32.

Every kernel is launched once per emulated rank with pointer tables that name local buffers ("local peers"), so the
instruction stream, tile schedule, routing arithmetic and flag protocol are those of the multi-GPU run while no launch
ever waits for another one.  Covered: the fused QKV projection with its sequence -> head scatter (video and text
forms) and its backward gather, attention with the head -> sequence push, the projection that pulls its operand per
head, the data-gradient GEMM that pushes head columns, all-gather -> GEMM, GEMM -> reduce-scatter with the partial
sum, and the gradient reduce-scatter / parameter all-gather / fused reduce + AdamW + all-gather kernels.
"""

import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _imports():
    from teletron_b200.ops._lib import c_float, c_int, c_long, call, ptr, stream
    from teletron_b200.ops.gemm_tcgen05 import check_status, status_tensor
    return c_float, c_int, c_long, call, ptr, stream, check_status, status_tensor


def table(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12)).item()


def _rnd(gen, *shape, scale=1.0):
    return (torch.randn(*shape, device="cuda", generator=gen) * scale).to(BF16)


def _rope(x, cos, sin):
    """Interleaved pairs (2i, 2i+1) with per-element tables, as the kernels apply it."""
    xr = torch.stack([-x[..., 1::2], x[..., 0::2]], dim=-1).flatten(-2)
    return x * cos + xr * sin


def _qkv_ref(raw, qw, kw, cos, sin, heads, rope):
    """raw [rows, heads * 384] (fp32 of the bf16 projection) -> q, k, v [heads, rows, 128] in fp32."""
    r = raw.view(raw.shape[0], heads, 3, 128)
    outs = []
    for which, w in ((0, qw), (1, kw)):
        t = r[:, :, which]
        t = t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
        if rope:
            t = _rope(t, cos[:, None], sin[:, None])
        outs.append(t.transpose(0, 1))
    outs.append(r[:, :, 2].transpose(0, 1))
    return outs


@pytest.mark.parametrize("s", [200, 1672])       # 128-wide tiles (few tiles) and 256-wide tiles; the last row tile is partial
def test_fused_qkv_scatter_and_its_backward_gather(s):
    c_float, c_int, c_long, call, ptr, stream, check_status, status_tensor = _imports()
    gen = torch.Generator(device="cuda").manual_seed(1)
    n, heads, T, K = 4, 8, 40, 256
    hl = heads // n
    S_tot = T + n * s
    w, b = _rnd(gen, heads * 384, K, scale=0.05), _rnd(gen, heads * 384, scale=0.1)
    qw, kw = (1 + 0.2 * torch.randn(128, device="cuda", generator=gen)).to(BF16), (1 + 0.2 * torch.randn(128, device="cuda", generator=gen)).to(BF16)
    ang = torch.rand(n * s, 64, device="cuda", generator=gen) * 6.28
    cos, sin = ang.cos().repeat_interleave(2, dim=1).contiguous(), ang.sin().repeat_interleave(2, dim=1).contiguous()
    xs = [_rnd(gen, s, K) for _ in range(n)]
    xt = _rnd(gen, T, K)
    qb, kb, vb = ([torch.full((hl, S_tot, 128), float("nan"), device="cuda", dtype=BF16) for _ in range(n)] for _ in range(3))
    aux = [torch.empty(s, heads * 384, device="cuda", dtype=BF16) for _ in range(n)]
    auxt = [torch.empty(T, heads * 384, device="cuda", dtype=BF16) for _ in range(n)]
    st = status_tensor(torch.device("cuda", 0))
    for me in range(n):
        c, sn = cos[me * s:(me + 1) * s].contiguous(), sin[me * s:(me + 1) * s].contiguous()
        call("tt_qkv_gemm_fused", ptr(xs[me]), ptr(w), ptr(b), ptr(qw), ptr(kw), ptr(c), ptr(sn), table(qb), table(kb), table(vb),
             c_int(n), c_int(me), ptr(aux[me]), c_int(s), c_int(heads), c_int(K), c_int(s), c_int(S_tot), c_int(T + me * s),
             c_int(s), c_int(0), c_float(1e-6), ptr(st), stream())
        # replicated text tokens: every rank computes all heads and keeps its own (no RoPE)
        local = [[t[me]] * n for t in (qb, kb, vb)]
        call("tt_qkv_gemm_fused", ptr(xt), ptr(w), ptr(b), ptr(qw), ptr(kw), None, None, table(local[0]), table(local[1]),
             table(local[2]), c_int(n), c_int(me), ptr(auxt[me]), c_int(T), c_int(heads), c_int(K), c_int(T), c_int(S_tot),
             c_int(0), c_int(0), c_int(1), c_float(1e-6), ptr(st), stream())
    torch.cuda.synchronize()
    check_status()
    for me in range(n):
        raw = (xs[me].float() @ w.float().t() + b.float()).to(BF16)
        assert rel(aux[me], raw) < 4e-3
        q, k, v = _qkv_ref(aux[me].float(), qw, kw, cos[me * s:(me + 1) * s], sin[me * s:(me + 1) * s], heads, True)
        for name, ref, bufs in (("q", q, qb), ("k", k, kb), ("v", v, vb)):
            for r in range(n):
                got = bufs[r][:, T + me * s:T + (me + 1) * s]
                assert torch.isfinite(got.float()).all(), (name, me, r)
                assert rel(got, ref[r * hl:(r + 1) * hl]) < 6e-3, (name, me, r)
        qt, kt, vt = _qkv_ref(auxt[me].float(), qw, kw, None, None, heads, False)
        for name, ref, bufs in (("q", qt, qb), ("k", kt, kb), ("v", vt, vb)):
            assert rel(bufs[me][:, :T], ref[me * hl:(me + 1) * hl]) < 6e-3, ("text", name, me)

    # backward: gradients sit head-sharded at their owners; rank `me` gathers its tokens' rows from every owner and
    # applies RoPE^T and the RMSNorm backward.  Reference: autograd of the fp32 composition above.
    dq, dk, dv = ([_rnd(gen, hl, S_tot, 128) for _ in range(n)] for _ in range(3))
    from teletron_b200.ops import _lib
    for me in range(n):
        raw = aux[me].float().requires_grad_(True)
        qwf, kwf = qw.float().requires_grad_(True), kw.float().requires_grad_(True)
        q, k, v = _qkv_ref(raw, qwf, kwf, cos[me * s:(me + 1) * s], sin[me * s:(me + 1) * s], heads, True)
        sl = slice(T + me * s, T + (me + 1) * s)
        gq = torch.cat([t[:, sl] for t in dq]).float()
        gk = torch.cat([t[:, sl] for t in dk]).float()
        gv = torch.cat([t[:, sl] for t in dv]).float()
        torch.autograd.backward([q, k, v], [gq, gk, gv])
        dqkv = torch.empty_like(aux[me])
        nw = _lib.lib().tt_qkv_partial_warps(c_long(s), c_int(heads))
        partials = torch.empty(nw * 256, dtype=torch.float32, device="cuda")
        dqw, dkw = torch.empty(128, dtype=BF16, device="cuda"), torch.empty(128, dtype=BF16, device="cuda")
        c, sn = cos[me * s:(me + 1) * s].contiguous(), sin[me * s:(me + 1) * s].contiguous()
        call("tt_qkv_post_bwd_peer", table(dq), table(dk), table(dv), c_int(n), ptr(aux[me]), ptr(qw), ptr(kw), ptr(c), ptr(sn),
             ptr(dqkv), ptr(partials), ptr(dqw), ptr(dkw), c_long(s), c_int(heads), c_long(s), c_long(S_tot), c_long(T + me * s),
             c_long(s), c_float(1e-6), stream())
        torch.cuda.synchronize()
        assert rel(dqkv, raw.grad) < 8e-3, me
        assert rel(dqw, qwf.grad) < 1e-2 and rel(dkw, kwf.grad) < 1e-2, me


def _attention_ref(q, k, v, kv_len=None, mask=None):
    s = (q.float() @ k.float().transpose(-1, -2)) / math.sqrt(q.shape[-1])
    if kv_len is not None:
        s[..., kv_len:] = float("-inf")
    if mask is not None:
        s[..., mask[0]:mask[1]] = float("-inf")
    return torch.softmax(s, dim=-1) @ v.float()


@pytest.mark.parametrize("coalesced", [1, 0])
def test_attention_with_head_to_sequence_push_and_pulling_projection(coalesced):
    c_float, c_int, c_long, call, ptr, stream, check_status, status_tensor = _imports()
    from teletron_b200.ops import _lib
    _lib.lib().tt_set_coalesced_peer_stores(ctypes.c_int(coalesced))
    gen = torch.Generator(device="cuda").manual_seed(2)
    n, heads, s, T = 2, 4, 300, 56
    hl = heads // n
    S_tot = T + n * s
    kv_len = S_tot - 7                                  # context-parallel padding at the sequence tail is masked,
                                                        # and so are the last 16 (padded) text tokens at its head
    st = status_tensor(torch.device("cuda", 0))
    q, k, v = ([_rnd(gen, hl, S_tot, 128) for _ in range(n)] for _ in range(3))
    g = [torch.full((T + s, heads * 128), float("nan"), device="cuda", dtype=BF16) for _ in range(n)]
    o_tok = []
    pitch = (S_tot + 63) // 64 * 64
    for me in range(n):
        out = torch.empty(1, S_tot, hl * 128, device="cuda", dtype=BF16)
        lse = torch.full((1, hl, pitch), float("inf"), dtype=torch.float32, device="cuda")
        call("tt_attn_fwd_push", ptr(q[me]), ptr(k[me]), ptr(v[me]), ptr(out), ptr(lse), c_int(hl), c_int(S_tot), c_int(kv_len),
             c_int(T - 16), c_int(T), c_int(pitch), c_float(1.0 / math.sqrt(128)), ptr(st), stream(), table(g), c_int(n), c_int(me), c_int(T), c_int(s),
             c_long(heads * 128))
        o_tok.append(out[0])
    torch.cuda.synchronize()
    check_status()
    ref = torch.cat([_attention_ref(q[r], k[r], v[r], kv_len, (T - 16, T)) for r in range(n)])          # [heads, S_tot, 128]
    ref_tok = ref.transpose(0, 1).reshape(S_tot, heads * 128)
    for me in range(n):
        want = torch.cat([ref_tok[:T], ref_tok[T + me * s:T + (me + 1) * s]])
        assert torch.isfinite(g[me].float()).all()
        assert rel(g[me], want) < 8e-3, me
        assert rel(o_tok[me], ref_tok[:, me * hl * 128:(me + 1) * hl * 128]) < 8e-3

    # pull form: the projection GEMM fetches its A operand per head block from the rank that owns the heads
    N_out = 384
    w, bias = _rnd(gen, N_out, heads * 128, scale=0.05), _rnd(gen, N_out, scale=0.1)
    span = hl * 128
    for me in range(n):
        y = torch.empty(s, N_out, device="cuda", dtype=BF16)
        call("tt_gemm_comm_bf16", table(o_tok), c_int(n), c_int(1), c_long(S_tot), c_int(span), c_int(T + me * s), None, c_long(0),
             ptr(w), c_int(0), c_long(w.stride(0)), ptr(y), c_long(N_out), ptr(bias), c_int(s), c_int(N_out), c_int(heads * 128),
             c_int(0), c_int(me), c_int(0), None, c_int(0), c_int(0), c_long(0), None, None, c_int(0), ptr(st), stream())
        torch.cuda.synchronize()
        a = torch.cat([o_tok[r][T + me * s:T + (me + 1) * s] for r in range(n)], dim=1).float()
        assert rel(y, a @ w.float().t() + bias.float()) < 6e-3, me

    # data gradient of that projection: every head block's columns are pushed to the owner of the heads
    do = [torch.full((S_tot, span), float("nan"), device="cuda", dtype=BF16) for _ in range(n)]
    for me in range(n):
        dy = _rnd(gen, s, N_out)
        call("tt_gemm_comm_bf16", table([dy]), c_int(n), c_int(0), c_long(s), c_int(0), c_int(0), None, c_long(0), ptr(w), c_int(1),
             c_long(w.stride(0)), None, c_long(0), None, c_int(s), c_int(heads * 128), c_int(N_out), c_int(0), c_int(me), c_int(1),
             table(do), c_int(span), c_int(T + me * s), c_long(span), None, None, c_int(0), ptr(st), stream())
        torch.cuda.synchronize()
        want = dy.float() @ w.float()
        for r in range(n):
            assert rel(do[r][T + me * s:T + (me + 1) * s], want[:, r * span:(r + 1) * span]) < 6e-3, (me, r)
    check_status()
    _lib.lib().tt_set_coalesced_peer_stores(ctypes.c_int(1))


@pytest.mark.parametrize("coalesced", [1, 0])
def test_all_gather_gemm_and_gemm_reduce_scatter(coalesced):
    c_float, c_int, c_long, call, ptr, stream, check_status, status_tensor = _imports()
    from teletron_b200.ops import _lib
    _lib.lib().tt_set_coalesced_peer_stores(ctypes.c_int(coalesced))
    gen = torch.Generator(device="cuda").manual_seed(3)
    n, rows, K, N = 4, 328, 512, 768                     # 328 rows per rank: partial last tile in every segment
    st = status_tensor(torch.device("cuda", 0))
    blocks = [_rnd(gen, rows, K) for _ in range(n)]
    x_full = torch.cat(blocks).float()
    w_full, bias = _rnd(gen, N, K, scale=0.05), _rnd(gen, N, scale=0.1)
    flags = torch.zeros(n * ((rows + 127) // 128), dtype=torch.int32, device="cuda")
    for me in range(n):
        wc = w_full[me * N // n:(me + 1) * N // n].contiguous()
        bc = bias[me * N // n:(me + 1) * N // n].contiguous()
        out = torch.empty(n * rows, N // n, device="cuda", dtype=BF16)
        aux = torch.empty_like(out)
        stage = torch.zeros(n * rows, K, device="cuda", dtype=BF16)
        call("tt_gemm_ag_bf16", table(blocks), c_int(n), c_int(me), c_int(rows), ptr(wc), c_int(0), c_long(K), ptr(out),
             c_long(N // n), ptr(bc), ptr(aux), c_int(N // n), c_int(K), c_int(2), ptr(stage), ptr(flags), c_int(me + 1),
             ptr(st), stream())
        torch.cuda.synchronize()
        pre = x_full @ wc.float().t() + bc.float()
        assert rel(aux, pre) < 6e-3, me
        assert rel(out, torch.nn.functional.gelu(pre, approximate="tanh")) < 8e-3, me
        for r in range(n):
            if r != me:
                assert torch.equal(stage[r * rows:(r + 1) * rows], blocks[r]), (me, r)
    check_status()

    # GEMM -> reduce-scatter: rank `me` multiplies its K shard for all rows and pushes row block i to zone i, slot me
    ks = K // n
    zones = [torch.full((n, rows, N), float("nan"), device="cuda", dtype=BF16) for _ in range(n)]
    for me in range(n):
        xk = torch.cat(blocks)[:, me * ks:(me + 1) * ks].contiguous()
        wk = w_full[:, me * ks:(me + 1) * ks].contiguous()
        call("tt_gemm_comm_bf16", table([xk]), c_int(n), c_int(0), c_long(n * rows), c_int(0), c_int(0), None, c_long(0), ptr(wk),
             c_int(0), c_long(ks), None, c_long(0), None, c_int(n * rows), c_int(N), c_int(ks), c_int(rows), c_int(me), c_int(2),
             table(zones), c_int(0), c_int(0), c_long(N), None, None, c_int(0), ptr(st), stream())
    torch.cuda.synchronize()
    check_status()
    full = x_full @ w_full.float().t() + bias.float()
    for r in range(n):
        out = torch.empty(rows, N, device="cuda", dtype=BF16)
        call("tt_partial_sum", ptr(zones[r]), c_int(n), c_long(rows), c_int(N), ptr(bias), None, None, c_long(rows), ptr(out), stream())
        torch.cuda.synchronize()
        assert rel(out, full[r * rows:(r + 1) * rows]) < 1e-2, r
    _lib.lib().tt_set_coalesced_peer_stores(ctypes.c_int(1))


@pytest.mark.parametrize("state_dtype,master", [(torch.float32, "fp32"), (BF16, "split16")])
def test_gradient_reduce_scatter_and_fused_adamw_all_gather(state_dtype, master):
    c_float, c_int, c_long, call, ptr, stream, check_status, status_tensor = _imports()
    from teletron_b200.ops.optim import _unpack16
    gen = torch.Generator(device="cuda").manual_seed(4)
    n, count = 3, 3 * 8 * 1000
    shard = count // n
    grads = [_rnd(gen, count, scale=0.1) for _ in range(n)]
    p0 = _rnd(gen, count)
    params = [p0.clone() for _ in range(n)]
    gsum = sum(t.float() for t in grads) / n
    # stand-alone reduce-scatter and all-gather kernels
    for me in range(n):
        out = torch.empty(shard, device="cuda", dtype=BF16)
        call("tt_reduce_scatter_bf16", table(grads), c_int(n), c_long(me * shard), ptr(out), c_long(shard), c_float(1.0 / n), stream())
        assert rel(out, gsum[me * shard:(me + 1) * shard]) < 4e-3
        dst = [torch.zeros(count, device="cuda", dtype=BF16) for _ in range(n)]
        call("tt_all_gather_push_bf16", table(dst), c_int(n), c_long(me * shard), ptr(out), c_long(shard), stream())
        torch.cuda.synchronize()
        assert all(torch.equal(d[me * shard:(me + 1) * shard], out) for d in dst)
    # fused reduce + AdamW + all-gather, three steps, against torch.optim.AdamW on fp32 weights
    ref = torch.nn.Parameter(p0.float().clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    m = [torch.zeros(shard, device="cuda", dtype=state_dtype) for _ in range(n)]
    v = [torch.zeros(shard, device="cuda", dtype=state_dtype) for _ in range(n)]
    mast = [p0[r * shard:(r + 1) * shard].float().clone() if master == "fp32" else None for r in range(n)]
    lo = [torch.zeros(shard, device="cuda", dtype=torch.int16) if master == "split16" else None for r in range(n)]
    for step in range(1, 4):
        grads = [_rnd(gen, count, scale=0.1) for _ in range(n)]
        ref.grad = sum(t.float() for t in grads) / n
        opt.step()
        for me in range(n):
            call("tt_rs_adamw_ag", table(grads), c_int(n), table(params), c_int(n), c_int(me), c_long(me * shard), ptr(m[me]),
                 ptr(v[me]), ptr(mast[me]), ptr(lo[me]), c_long(shard), c_int(1 if state_dtype == BF16 else 0), c_float(1e-2),
                 c_float(0.9), c_float(0.95), c_float(1e-8), c_float(0.1), c_int(step), c_float(1.0 / n), stream())
        torch.cuda.synchronize()
        assert all(torch.equal(params[0], p) for p in params[1:]), "replicas differ after the all-gather"
    if master == "fp32":
        got = torch.cat(mast)
        assert rel(got, ref.detach()) < 1e-5
    else:
        got = torch.cat([_unpack16(params[0][r * shard:(r + 1) * shard], lo[r]) for r in range(n)])
        assert rel(got, ref.detach()) < 3e-3          # bf16 moments
    assert rel(params[0], ref.detach()) < 4e-3
