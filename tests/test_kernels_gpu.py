"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op.

The reference project checks only add and matmul on the GPU against its CPU ops
(test/test_cuda.lua:29-85); here every kernel is covered, at tile-multiple and ragged shapes.
"""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    from luatorch_b200 import _C
    return _C


def _gemm(C, a, b, M, N, K, a_mn=False, b_mn=True, out_dtype=torch.bfloat16, **kw):
    c = torch.zeros(M, (N + 7) // 8 * 8, device="cuda", dtype=out_dtype)
    C.gemm(a, b, c, M, N, K, a.stride(0), b.stride(0), c.stride(0), a_mn, b_mn, 1, 1, 0, 0, 0, 0,
           0, 0, kw.get("alpha", 1.0), kw.get("accumulate", False), kw.get("bias"),
           kw.get("act", 0), kw.get("residual"),
           kw["residual"].stride(0) if kw.get("residual") is not None else 0, kw.get("aux_out"),
           kw.get("aux_in"), kw["aux_in"].stride(0) if kw.get("aux_in") is not None else 0, 0)
    return c[:, :N]


def gelu_ref(x):
    return 0.5 * x * (1 + torch.tanh(0.7978845608 * (x + 0.044715 * x ** 3)))


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 768, 768), (300, 200, 136), (1000, 1000, 72)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (False, False), (True, True), (True, False)])
def test_gemm_layouts(C, M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    A = torch.randn(M, K, device="cuda") * 0.5
    B = torch.randn(K, N, device="cuda") * 0.5
    a = (A.t().contiguous() if a_mn else A).bfloat16()
    b = (B if b_mn else B.t().contiguous()).bfloat16()
    if (a.stride(0) % 8) or (b.stride(0) % 8):
        pytest.skip("row stride not 16-byte aligned")
    ref = A.bfloat16().float() @ B.bfloat16().float()
    out = _gemm(C, a, b, M, N, K, a_mn, b_mn).float()
    assert C.gemm_device_error() == 0
    torch.testing.assert_close(out, ref, atol=0.08, rtol=0.02)


def test_gemm_epilogues(C):
    torch.manual_seed(1)
    M, N, K = 384, 512, 256
    a = (torch.randn(M, K, device="cuda") * 0.3).bfloat16()
    w = (torch.randn(K, N, device="cuda") * 0.3).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    base = a.float() @ w.float()
    out = _gemm(C, a, w, M, N, K, bias=bias).float()
    torch.testing.assert_close(out, base + bias.float(), atol=0.06, rtol=0.02)
    aux = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    out = _gemm(C, a, w, M, N, K, bias=bias, act=1, aux_out=aux).float()
    torch.testing.assert_close(aux.float(), base + bias.float(), atol=0.06, rtol=0.02)
    torch.testing.assert_close(out, gelu_ref(base + bias.float()), atol=0.06, rtol=0.02)
    out = _gemm(C, a, w, M, N, K, bias=bias, residual=res).float()
    torch.testing.assert_close(out, base + bias.float() + res.float(), atol=0.08, rtol=0.02)
    # dgelu epilogue
    x = torch.randn(M, N, device="cuda").bfloat16()
    xf = x.float().requires_grad_(True)
    gelu_ref(xf).sum().backward()
    out = _gemm(C, a, w, M, N, K, act=2, aux_in=x).float()
    torch.testing.assert_close(out, base * xf.grad, atol=0.08, rtol=0.03)
    # fp32 output + accumulate
    c = torch.ones(M, N, device="cuda")
    C.gemm(a, w, c, M, N, K, K, N, N, False, True, 1, 1, 0, 0, 0, 0, 0, 0, 0.5, True, None, 0,
           None, 0, None, None, 0, 0)
    torch.testing.assert_close(c, 0.5 * base + 1.0, atol=0.02, rtol=0.01)


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(768, 768, 8192, True, True), (768, 2304, 4096, True, True),
                                             (384, 512, 4096, False, True)])
def test_gemm_split_k(C, M, N, K, a_mn, b_mn):
    """Long-K, few-tile products (weight gradients) run as K slices + a fixed-order reduction."""
    torch.manual_seed(3)
    A = torch.randn(M, K, device="cuda") * 0.1
    B = torch.randn(K, N, device="cuda") * 0.1
    a = (A.t().contiguous() if a_mn else A).bfloat16()
    b = (B if b_mn else B.t().contiguous()).bfloat16()
    ref = A.bfloat16().float() @ B.bfloat16().float()
    out = _gemm(C, a, b, M, N, K, a_mn, b_mn).float()
    torch.testing.assert_close(out, ref, atol=0.05, rtol=0.02)
    # accumulate into an existing bf16 gradient, twice: results must be bit-identical
    g1 = torch.ones(M, N, device="cuda", dtype=torch.bfloat16)
    g2 = g1.clone()
    for g in (g1, g2):
        C.gemm(a, b, g, M, N, K, a.stride(0), b.stride(0), N, a_mn, b_mn, 1, 1, 0, 0, 0, 0, 0, 0,
               1.0, True, None, 0, None, 0, None, None, 0, 0)
    torch.testing.assert_close(g1.float(), ref + 1.0, atol=0.06, rtol=0.02)
    assert torch.equal(g1, g2)
    assert C.gemm_device_error() == 0


def test_gemm_simt_fallback_and_batched(C):
    torch.manual_seed(2)
    a = torch.randn(64, 256, device="cuda").bfloat16()
    w = torch.randn(256, 10, device="cuda").bfloat16()  # row stride 10: not TMA addressable
    out = torch.zeros(64, 10, device="cuda", dtype=torch.bfloat16)
    C.gemm(a, w, out, 64, 10, 256, 256, 10, 10, False, True, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, False,
           None, 0, None, 0, None, None, 0, 0)
    torch.testing.assert_close(out.float(), a.float() @ w.float(), atol=0.15, rtol=0.02)
    # batched: [6, 256, 64] x [6, 64, 192]
    A = torch.randn(6, 256, 64, device="cuda").bfloat16()
    Bm = torch.randn(6, 64, 192, device="cuda").bfloat16()
    out = torch.zeros(6, 256, 192, device="cuda", dtype=torch.bfloat16)
    C.gemm(A, Bm, out, 256, 192, 64, 64, 192, 192, False, True, 3, 2, 256 * 64, 3 * 256 * 64,
           64 * 192, 3 * 64 * 192, 256 * 192, 3 * 256 * 192, 1.0, False, None, 0, None, 0, None,
           None, 0, 0)
    torch.testing.assert_close(out.float(), torch.bmm(A.float(), Bm.float()), atol=0.1, rtol=0.02)
    assert C.gemm_device_error() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [1, 7, 1024, 100003])
def test_elementwise(C, dtype, n):
    torch.manual_seed(3)
    a = torch.randn(n, device="cuda").to(dtype)
    b = (torch.randn(n, device="cuda") + 2.0).to(dtype)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    af, bf = a.float(), b.float()
    for op, ref in enumerate([af + bf, af - bf, af * bf, af / bf]):
        torch.testing.assert_close(C.binary(op, a, b, False).float(), ref, **tol)
    torch.testing.assert_close(C.scalar(0, a, 1.5, False).float(), af + 1.5, **tol)
    torch.testing.assert_close(C.scalar(1, a, 1.5, False).float(), af * 1.5, **tol)
    torch.testing.assert_close(C.scalar(4, a, 0.0, False).float(), (af > 0).float(), **tol)
    refs = [-af, af.abs(), torch.where(af < 0, torch.zeros_like(af), af.clamp_min(0).sqrt()),
            torch.where(af <= 0, torch.full_like(af, -math.inf), af.clamp_min(1e-30).log()),
            af.exp(), af.relu(), af.sigmoid(), af.tanh(), gelu_ref(af), af * af.sigmoid()]
    for op, ref in enumerate(refs):
        torch.testing.assert_close(C.unary(op, a).float(), ref, equal_nan=True, **tol)
    # activation backward
    for op, fn in [(5, torch.relu), (6, torch.sigmoid), (7, torch.tanh), (8, gelu_ref),
                   (9, lambda t: t * torch.sigmoid(t))]:
        x = af.clone().requires_grad_(True)
        fn(x).backward(bf)
        torch.testing.assert_close(C.unary_backward(op, a, b).float(), x.grad, **tol)
    # div by zero -> 0
    z = torch.zeros(n, device="cuda", dtype=dtype)
    assert torch.all(C.binary(3, a, z, False) == 0)


def test_broadcast_colsum_cast_transpose(C):
    torch.manual_seed(4)
    a = torch.randn(333, 72, device="cuda")
    bias = torch.randn(72, device="cuda")
    torch.testing.assert_close(C.add_broadcast(a, bias), a + bias)
    torch.testing.assert_close(C.column_sum(a, None, False), a.sum(0), atol=1e-4, rtol=1e-5)
    out = torch.ones(72, device="cuda")
    C.column_sum(a.bfloat16(), out, True)
    torch.testing.assert_close(out, a.bfloat16().float().sum(0) + 1, atol=1e-3, rtol=1e-4)
    torch.testing.assert_close(C.cast(a, torch.bfloat16), a.bfloat16())
    torch.testing.assert_close(C.cast(a.bfloat16(), torch.float32), a.bfloat16().float())
    torch.testing.assert_close(C.cast(a, torch.float16), a.half())
    torch.testing.assert_close(C.transpose2d(a), a.t().contiguous())
    hi, lo = C.split_bf16(a)
    torch.testing.assert_close(hi.float() + lo.float(), a, atol=1e-4, rtol=1e-4)


def test_rng_and_dropout(C):
    x = torch.empty(1 << 20, device="cuda")
    C.fill_random(x, 1234, 0, False)
    assert 0.0 <= x.min().item() and x.max().item() < 1.0
    assert abs(x.mean().item() - 0.5) < 5e-3
    y = torch.empty(1 << 20, device="cuda")
    C.fill_random(y, 1234, 0, False)
    assert torch.equal(x, y)  # same (seed, offset) => same stream
    C.fill_random(x, 1234, 0, True)
    assert abs(x.mean().item()) < 5e-3 and abs(x.std().item() - 1.0) < 5e-3
    ones = torch.ones(1 << 20, device="cuda", dtype=torch.bfloat16)
    d = C.dropout(ones, 0.2, 7, 0)
    keep = (d != 0).float().mean().item()
    assert abs(keep - 0.8) < 5e-3
    torch.testing.assert_close(d[d != 0].float().mean().item(), 1.25, atol=1e-2, rtol=0)
    assert torch.equal(d, C.dropout(ones, 0.2, 7, 0))


@pytest.mark.parametrize("n", [5, 4096, 1000003])
def test_reductions(C, n):
    torch.manual_seed(5)
    a = torch.randn(n, device="cuda")
    b = torch.randn(n, device="cuda")
    for _ in range(2):  # second call checks that the ticket was re-armed
        torch.testing.assert_close(C.reduce(0, a, 1.0)[0], a.double().sum().float(), atol=1e-2, rtol=1e-4)
        assert C.reduce(1, a, 1.0)[0].item() == a.max().item()
        assert C.reduce(2, a, 1.0)[0].item() == a.min().item()
        torch.testing.assert_close(C.dot(a, b)[0], (a.double() * b.double()).sum().float(), atol=1e-2, rtol=1e-4)
    r1, r2 = C.reduce(0, a, 1.0), C.reduce(0, a, 1.0)
    assert torch.equal(r1, r2)  # fixed summation order
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    C.check_finite_scale(a, 0.5, False, flag)
    assert flag.item() == 0
    a2 = a.clone()
    a2[n // 2] = float("inf")
    C.check_finite_scale(a2, 0.5, False, flag)
    assert flag.item() == 1


@pytest.mark.parametrize("rows,cols", [(4, 10), (33, 1000), (16, 50257)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_and_cross_entropy(C, rows, cols, dtype):
    torch.manual_seed(6)
    ld = (cols + 7) // 8 * 8 if rows % 2 == 0 else cols + 1   # odd row counts: rows not 16-byte aligned
    full = (torch.randn(rows, ld, device="cuda") * 3).to(dtype)
    logits = full[:, :cols]
    labels = torch.randint(0, cols, (rows,), device="cuda")
    ref = torch.softmax(logits.float(), -1)
    tol = dict(atol=1e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=5e-3, rtol=2e-2)
    torch.testing.assert_close(C.softmax(logits.contiguous()).float(), ref, **tol)
    lf = logits.float().clone().requires_grad_(True)
    loss_ref = torch.nn.functional.cross_entropy(lf, labels)
    loss_ref.backward()
    for lab in (labels, labels.int(), labels.float()):
        loss, lse, err = C.cross_entropy_forward(logits, cols, lab)
        assert err[0].item() == 0
        torch.testing.assert_close(loss[0], loss_ref.detach(), atol=1e-4, rtol=1e-4)
        out = torch.zeros_like(full)
        C.cross_entropy_backward(logits, cols, lab, lse, 1.0 / rows, None, out[:, :cols])
        torch.testing.assert_close(out[:, :cols].float(), lf.grad, atol=1e-3 if dtype == torch.bfloat16 else 1e-6, rtol=2e-2)
    bad = labels.clone()
    bad[0] = cols
    word = C.cross_entropy_forward(logits, cols, bad)[2].tolist()
    assert word[0] == 1 and word[1] == 0 and word[2] == cols      # flag, row, offending label


@pytest.mark.parametrize("rows,cols,ld", [(64, 1000, 1000), (33, 50257, 50264), (19, 50257, 50257),
                                          (21, 1003, 1005)])
def test_cross_entropy_fused_forward_backward(C, rows, cols, ld):
    """One kernel: loss + log-sum-exp, logits overwritten by (softmax - onehot) * scale.
    Odd leading dimensions start every row at another offset within 16 bytes."""
    torch.manual_seed(4)
    buf = torch.zeros(rows, ld, device="cuda", dtype=torch.bfloat16)
    buf[:, :cols] = (torch.randn(rows, cols, device="cuda") * 2).bfloat16()
    labels = torch.randint(0, cols, (rows,), device="cuda")
    x = buf[:, :cols].float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(x, labels)
    ref.backward()
    loss, lse, err = C.cross_entropy_fused(buf, cols, labels, 1.0 / rows)
    assert err[0].item() == 0
    torch.testing.assert_close(loss[0], ref.detach(), atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(lse, torch.logsumexp(x.detach(), dim=1), atol=2e-3, rtol=2e-3)
    torch.testing.assert_close(buf[:, :cols].float(), x.grad, atol=2e-4, rtol=3e-2)


@pytest.mark.parametrize("dtype,B,Cc,H,W,k,stride,pad,ld", [
    (torch.bfloat16, 4, 32, 32, 32, 3, 2, 1, 288),     # conv net layer 2: 16-byte rows
    (torch.bfloat16, 2, 3, 32, 32, 3, 1, 1, 32),       # layer 1: patch 27 padded to 32
    (torch.bfloat16, 3, 64, 16, 16, 3, 2, 1, 576),
    (torch.float32, 3, 5, 9, 11, 3, 2, 1, 48),
    (torch.float32, 2, 4, 12, 10, 5, 1, 2, 100),
])
def test_im2col_col2im_vector_paths(C, dtype, B, Cc, H, W, k, stride, pad, ld):
    """The 16-byte-store im2col (padding columns zeroed by the kernel) and the col2im that
    stages the contributing cols rows in shared memory, against unfold / fold in fp32."""
    torch.manual_seed(12)
    x = torch.randn(B, Cc, H, W, device="cuda").to(dtype)
    patch = Cc * k * k
    cols = C.im2col(x.reshape(-1), B, Cc, H, W, k, stride, pad, ld)
    assert cols.shape[1] == ld
    unf = torch.nn.functional.unfold(x.float(), k, padding=pad, stride=stride)
    ref = unf.transpose(1, 2).reshape(-1, patch)
    assert torch.equal(cols[:, :patch].float(), ref)
    assert torch.all(cols[:, patch:] == 0)
    g = torch.randn(cols.shape[0], ld, device="cuda").to(dtype)
    din = C.col2im(g[:, :patch], B, Cc, H, W, k, stride, pad)
    L = unf.shape[-1]
    ref_din = torch.nn.functional.fold(g[:, :patch].float().view(B, L, patch).transpose(1, 2), (H, W), k,
                                       padding=pad, stride=stride)
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(din.view(B, Cc, H, W).float(), ref_din, **tol)


def test_pointwise_losses(C):
    torch.manual_seed(7)
    p = torch.randn(1000, device="cuda")
    t = torch.randn(1000, device="cuda")
    torch.testing.assert_close(C.pointwise_loss(0, p, t)[0], ((p - t) ** 2).mean())
    torch.testing.assert_close(C.pointwise_loss(1, p, t)[0], (p - t).abs().mean())
    torch.testing.assert_close(C.pointwise_loss_backward(0, p, t, 1.0), 2 * (p - t) / 1000)
    torch.testing.assert_close(C.pointwise_loss_backward(1, p, t, 1.0), torch.sign(p - t) / 1000)


@pytest.mark.parametrize("rows,cols", [(8, 8), (100, 768), (37, 2048), (19, 1000), (5, 3001)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_layernorm(C, rows, cols, dtype):
    torch.manual_seed(8)
    x = torch.randn(rows, cols, device="cuda").to(dtype)
    g = (torch.randn(cols, device="cuda") * 0.5 + 1).to(dtype)
    b = torch.randn(cols, device="cuda").to(dtype)
    dy = torch.randn(rows, cols, device="cuda").to(dtype)
    add = torch.randn(rows, cols, device="cuda").to(dtype)
    xf, gf, bf = (t.float().clone().requires_grad_(True) for t in (x, g, b))
    ref = torch.nn.functional.layer_norm(xf, (cols,), gf, bf, 1e-5)
    ref.backward(dy.float())
    y, mean, rstd = C.layernorm_forward(x, g, b, 1e-5)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=4e-2, rtol=3e-2)
    torch.testing.assert_close(y.float(), ref.detach(), **tol)
    dg = torch.zeros(cols, device="cuda")
    db = torch.zeros(cols, device="cuda")
    dx = C.layernorm_backward(x, dy, g, mean, rstd, add, dg, db, False)
    torch.testing.assert_close(dx.float(), xf.grad + add.float(), **tol)
    ptol = dict(atol=1e-3, rtol=1e-3) if dtype == torch.float32 else dict(atol=0.15, rtol=3e-2)
    torch.testing.assert_close(dg, gf.grad, **ptol)
    torch.testing.assert_close(db, bf.grad, **ptol)
    dg2, db2 = torch.zeros_like(dg), torch.zeros_like(db)
    C.layernorm_backward(x, dy, g, mean, rstd, None, dg2, db2, False)
    assert torch.equal(dg, dg2) and torch.equal(db, db2)  # reproducible
    # the same launches can also sum the columns of dx (bias gradient of the producing Linear)
    dg3, db3 = torch.zeros_like(dg), torch.zeros_like(db)
    dxs = torch.full((cols,), 2.0, device="cuda")
    dx3, done = C.layernorm_backward_dxsum(x, dy, g, mean, rstd, add, dg3, db3, False, dxs, True)
    assert torch.equal(dx3, dx) and torch.equal(dg3, dg) and torch.equal(db3, db)
    if done:      # shapes the fused kernels cover; otherwise the caller sums dx itself
        want = (xf.grad + add.float()).sum(0) + 2.0
        torch.testing.assert_close(dxs, want, atol=1e-3 * rows ** 0.5 if dtype == torch.float32 else 0.3,
                                   rtol=1e-3 if dtype == torch.float32 else 3e-2)
    else:
        assert torch.all(dxs == 2.0)


def test_gelu_bias(C):
    torch.manual_seed(9)
    x = torch.randn(50, 264, device="cuda").bfloat16()
    b = torch.randn(264, device="cuda").bfloat16()
    dy = torch.randn(50, 264, device="cuda").bfloat16()
    z = (x.float() + b.float()).requires_grad_(True)
    ref = gelu_ref(z)
    ref.backward(dy.float())
    torch.testing.assert_close(C.gelu_bias_forward(x, b).float(), ref.detach(), atol=3e-2, rtol=2e-2)
    torch.testing.assert_close(C.gelu_bias_backward(x, b, dy).float(), z.grad, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding(C, dtype):
    torch.manual_seed(10)
    vocab, dim, B, S = 1000, 72, 4, 33
    table = torch.randn(vocab, dim, device="cuda").to(dtype)
    pos = torch.randn(64, dim, device="cuda").to(dtype)
    ids = torch.randint(0, vocab, (B * S,), device="cuda")
    ids[:10] = 5  # a crowded bucket
    out, err = C.embedding_forward(table, ids, pos, S)
    assert err[0].item() == 0
    ref = table.float()[ids] + pos.float()[torch.arange(B * S, device="cuda") % S]
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    out2, _ = C.embedding_forward(table, ids.float(), None, 1)
    torch.testing.assert_close(out2.float(), table.float()[ids])
    dy = torch.randn(B * S, dim, device="cuda").to(dtype)
    dt = torch.full((vocab, dim), 7.0, device="cuda")
    C.embedding_backward(dy, ids, dt, False)
    ref_dt = torch.zeros(vocab, dim, device="cuda").index_add_(0, ids, dy.float())
    torch.testing.assert_close(dt, ref_dt, atol=1e-4, rtol=1e-4)
    dt2 = torch.empty_like(dt)
    C.embedding_backward(dy, ids, dt2, False)
    assert torch.equal(dt, dt2)
    dp = torch.full((64, dim), 3.0, device="cuda")
    C.positional_backward(dy, dp, B, S, False)
    ref_dp = torch.zeros(64, dim, device="cuda")
    ref_dp[:S] = dy.float().view(B, S, dim).sum(0)
    torch.testing.assert_close(dp, ref_dp, atol=1e-4, rtol=1e-4)
    bad = ids.clone()
    bad[3] = vocab + 1
    word = C.embedding_forward(table, bad, None, 1)[1].tolist()
    assert word[0] == 1 and word[1] == 3 and word[2] == vocab + 1     # flag, position, offending id


def test_im2col_col2im(C):
    torch.manual_seed(11)
    B, Cc, H, W, k, stride, pad = 3, 5, 9, 11, 3, 2, 1
    x = torch.randn(B, Cc, H, W, device="cuda")
    cols = C.im2col(x.reshape(-1), B, Cc, H, W, k, stride, pad, 0)
    unf = torch.nn.functional.unfold(x, k, padding=pad, stride=stride)  # [B, C*k*k, L]
    ref = unf.transpose(1, 2).reshape(-1, Cc * k * k)
    torch.testing.assert_close(cols, ref)
    g = torch.randn_like(cols)
    din = C.col2im(g, B, Cc, H, W, k, stride, pad)
    L = unf.shape[-1]
    ref_din = torch.nn.functional.fold(g.view(B, L, -1).transpose(1, 2), (H, W), k, padding=pad, stride=stride)
    torch.testing.assert_close(din.view(B, Cc, H, W), ref_din, atol=1e-5, rtol=1e-5)
    nhwc = torch.randn(B * 20, 7, device="cuda")
    nchw = C.relayout(nhwc, B, 7, 20, True)
    torch.testing.assert_close(nchw.view(B, 7, 20), nhwc.view(B, 20, 7).transpose(1, 2).contiguous())
    torch.testing.assert_close(C.relayout(nchw, B, 7, 20, False).view(B * 20, 7), nhwc)


def test_adamw_and_sgd_flat(C):
    torch.manual_seed(12)
    n = 4096 + 256
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    shadow = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    seg_end = torch.tensor([4096, n], device="cuda", dtype=torch.int64)
    seg_wd = torch.tensor([0.1, 0.0], device="cuda")
    pr, mr, vr = p.clone(), m.clone(), v.clone()
    lr, b1, b2, eps = 1e-2, 0.9, 0.999, 1e-8
    for t in range(1, 4):
        bc1, bc2 = 1 - b1 ** t, 1 - b2 ** t
        C.adamw_flat(p, shadow, g.bfloat16(), m, v, seg_end, seg_wd, lr, b1, b2, eps, bc1, bc2, 1.0, None)
        gg = g.bfloat16().float()
        wd = torch.cat([torch.full((4096,), 0.1), torch.zeros(256)]).cuda()
        pr = pr * (1 - lr * wd)
        mr = b1 * mr + (1 - b1) * gg
        vr = b2 * vr + (1 - b2) * gg * gg
        pr = pr - lr * (mr / bc1) / ((vr / bc2).sqrt() + eps)
    torch.testing.assert_close(p, pr, atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(shadow, pr.bfloat16(), atol=1e-2, rtol=1e-2)
    skip = torch.ones(1, device="cuda", dtype=torch.int32)
    before = p.clone()
    C.adamw_flat(p, shadow, g, m, v, None, None, lr, b1, b2, eps, 0.1, 0.1, 1.0, skip)
    assert torch.equal(p, before)
    # SGD momentum
    p2, vel = torch.randn(1001, device="cuda"), torch.zeros(1001, device="cuda")
    g2 = torch.randn(1001, device="cuda")
    ref_p, ref_v = p2.clone(), vel.clone()
    for _ in range(3):
        C.sgd_flat(p2, None, g2, vel, 0.1, 0.9, False, 1.0)
        ref_v = 0.9 * ref_v + g2
        ref_p = ref_p - 0.1 * ref_v
    torch.testing.assert_close(p2, ref_p, atol=1e-6, rtol=1e-5)


def _attn_ref(q, k, v, causal, scale):
    # q, k, v: [B, S, H, D] fp32
    qh, kh, vh = (t.permute(0, 2, 1, 3) for t in (q, k, v))
    s = torch.matmul(qh, kh.transpose(-1, -2)) * scale
    if causal:
        S = q.shape[1]
        mask = torch.triu(torch.ones(S, S, device=q.device, dtype=torch.bool), 1)
        s = s.masked_fill(mask, float("-inf"))
    p = torch.softmax(s, -1)
    return torch.matmul(p, vh).permute(0, 2, 1, 3), torch.logsumexp(s, -1)


@pytest.mark.parametrize("B,S,H,D", [(1, 128, 1, 64), (2, 256, 3, 64), (1, 384, 2, 128), (2, 200, 2, 64)])
@pytest.mark.parametrize("causal", [True, False])
def test_flash_attention(C, B, S, H, D, causal):
    torch.manual_seed(13)
    E = H * D
    qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.7).bfloat16()  # fused-projection layout
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    scale = 1.0 / math.sqrt(D)
    qf, kf, vf = (t.float().clone().requires_grad_(True) for t in (q, k, v))
    ref_o, ref_lse = _attn_ref(qf, kf, vf, causal, scale)
    o, lse = C.flash_forward(q, k, v, causal, scale)
    assert C.attention_device_error() == 0
    torch.testing.assert_close(o.float(), ref_o.detach(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(lse, ref_lse.detach(), atol=2e-2, rtol=1e-3)
    d_o = (torch.randn(B, S, H, D, device="cuda") * 0.5).bfloat16()
    ref_o.backward(d_o.float())
    dq, dk, dv = C.flash_backward(q, k, v, o, lse, d_o, causal, scale, None)
    assert C.attention_device_error() == 0
    torch.testing.assert_close(dv.float(), vf.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(dk.float(), kf.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(dq.float(), qf.grad, atol=3e-2, rtol=3e-2)
    # packed gradient output (layout of the fused qkv activation)
    packed = torch.empty(B, S, 3, H, D, device="cuda", dtype=torch.bfloat16)
    C.flash_backward(q, k, v, o, lse, d_o, causal, scale, packed)
    assert torch.equal(packed[:, :, 0], dq) and torch.equal(packed[:, :, 2], dv)


@pytest.mark.parametrize("B,S,H,D,sl", [(8, 1024, 12, 64, (slice(6, 8), slice(9, 12))),
                                        (4, 2048, 16, 128, (slice(3, 4), slice(14, 16)))])
def test_flash_attention_model_shapes(C, B, S, H, D, sl):
    """The two benchmark shapes (8 and 16 key tiles: the K/V rings wrap many times, all heads
    and batches launched); a slice of (batch, head) pairs is compared with fp32 attention."""
    torch.manual_seed(14)
    qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.7).bfloat16()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    scale = 1.0 / math.sqrt(D)
    o, lse = C.flash_forward(q, k, v, True, scale)
    d_o = (torch.randn(B, S, H, D, device="cuda") * 0.5).bfloat16()
    dq, dk, dv = C.flash_backward(q, k, v, o, lse, d_o, True, scale, None)
    assert C.attention_device_error() == 0
    bs, hs = sl
    qf, kf, vf = (t[bs][:, :, hs].float().clone().requires_grad_(True) for t in (q, k, v))
    ref_o, ref_lse = _attn_ref(qf, kf, vf, True, scale)
    ref_o.backward(d_o[bs][:, :, hs].float())
    torch.testing.assert_close(o[bs][:, :, hs].float(), ref_o.detach(), atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(lse[bs][:, hs], ref_lse.detach(), atol=2e-2, rtol=1e-3)
    torch.testing.assert_close(dv[bs][:, :, hs].float(), vf.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(dk[bs][:, :, hs].float(), kf.grad, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(dq[bs][:, :, hs].float(), qf.grad, atol=3e-2, rtol=3e-2)
    # bitwise reproducible (no atomics anywhere in the backward)
    dq2, dk2, dv2 = C.flash_backward(q, k, v, o, lse, d_o, True, scale, None)
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


def test_bounded_wait_reports_instead_of_hanging():
    # one GPU: a flag nobody sets makes the wait run out; the context stays usable
    import torch
    from luatorch_b200 import _C
    flag = torch.zeros(1, device="cuda", dtype=torch.int32)
    status = torch.zeros(8, device="cuda", dtype=torch.int32)
    _C.wait_flag_bounded(flag, 1, 200_000_000, status)      # about 0.1 s of SM clocks
    torch.cuda.synchronize()
    assert status[0].item() == 100
    flag.fill_(5)
    status.zero_()
    _C.wait_flag_bounded(flag, 5, 200_000_000, status)
    torch.cuda.synchronize()
    assert status[0].item() == 0
    assert float(torch.ones(4, device="cuda").sum()) == 4.0


@pytest.mark.parametrize("D,causal", [(32, True), (96, False)])
def test_tensor_attention_api_other_head_dims_run_on_the_tensor_core_path(D, causal):
    """`Tensor.flash_attention` / `_backend.attention` for head dims the flash kernels do not
    cover: scores, softmax and P V as batched tcgen05 GEMMs plus the score-softmax kernel (no
    library GEMM on the GPU), output and log-sum-exp against fp32 attention."""
    from luatorch_b200 import _backend as B
    torch.manual_seed(21)
    BH, S = 6, 128
    q, k, v = ((torch.randn(BH, S, D, device="cuda") * 0.7).bfloat16() for _ in range(3))
    g0 = sum(lf_launches()[:1])
    o, lse = B.attention(q, k, v, causal)
    assert sum(lf_launches()[:1]) >= g0 + 2            # the batched GEMMs of this package ran
    qf, kf, vf = q.float(), k.float(), v.float()
    s = qf @ kf.transpose(-1, -2) / math.sqrt(D)
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1), float("-inf"))
    torch.testing.assert_close(o.float(), torch.softmax(s, -1) @ vf, atol=3e-2, rtol=3e-2)
    torch.testing.assert_close(lse.float(), torch.logsumexp(s, -1), atol=3e-2, rtol=1e-2)


def lf_launches():
    import luatorch_b200 as lf
    return lf.launch_counts()


@pytest.mark.parametrize("pair", ["0", "1"])
def test_gemm_single_cta_and_cta_pair_kernels_agree_with_fp32(pair):
    """The same products with the CTA-pair kernel forbidden and forced (the choice is read once
    per process, so each setting runs in a process of its own): the LM-head shape
    N = 50264 / K = 768 (197 column tiles, a ragged last one), a square K = 768 product, a long-K
    weight-gradient form (A transposed) and a transposed-B form, against fp32 matmul."""
    import subprocess, sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    body = r'''
import sys, torch
sys.path.insert(0, %r)
from luatorch_b200 import _backend as B, _C
torch.manual_seed(31)
cases = [(1024, 50264, 768, False, False), (512, 768, 768, False, False), (768, 2304, 4096, True, False),
         (1024, 768, 3072, False, True)]
for M, N, K, a_t, b_t in cases:
    a = (torch.randn((K, M) if a_t else (M, K), device="cuda") * 0.1).bfloat16()
    b = (torch.randn((N, K) if b_t else (K, N), device="cuda") * 0.1).bfloat16()
    c = B.gemm(a, b, a_t=a_t, b_t=b_t)
    af = a.float().t() if a_t else a.float()
    bf = b.float().t() if b_t else b.float()
    ref = af @ bf
    err = (c.float() - ref).abs().max().item()
    tol = 0.02 * (K ** 0.5) * 0.01 + 0.02
    assert err < tol, (M, N, K, a_t, b_t, err, tol)
assert _C.gemm_device_error() == 0
print("CASE_OK")
''' % root
    env = dict(os.environ, LT_GEMM_PAIR=pair)
    r = subprocess.run([sys.executable, "-c", body], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "CASE_OK" in r.stdout, (r.stdout[-1500:], r.stderr[-2500:])


def test_late_wait_kernels_match_serial_order():
    """A weight-gradient GEMM marked independent of the kernel before it (it starts in that
    kernel's tail and waits for it before exiting) gives the bits of the serial order, every
    time, and what follows sees all of it finished."""
    from luatorch_b200 import _backend as B
    torch.manual_seed(21)
    M, K, N = 4096, 768, 3072
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(K, N, device="cuda") * 0.05).bfloat16()
    g = torch.randn(M, N, device="cuda").bfloat16()
    ref_dx = B.gemm(g, w, b_t=True)
    ref_y = B.gemm(ref_dx, w)
    ref_dw = torch.empty(K, N, device="cuda")
    B.gemm(x, g, a_t=True, out=ref_dw)
    ref_db = torch.empty(N, device="cuda")
    B.column_sum(g, ref_db, False)
    torch.testing.assert_close(ref_dw, x.float().t() @ g.float(), atol=0.5, rtol=2e-2)
    torch.testing.assert_close(ref_db, g.float().sum(0), atol=1e-2, rtol=1e-3)
    for it in range(12):
        dw = torch.full((K, N), float("nan"), device="cuda")
        db = torch.full((N,), float("nan"), device="cuda")
        dx = B.gemm(g, w, b_t=True)
        B.gemm(x, g, a_t=True, out=dw, overlap_prev=1)
        B.column_sum(g, db, False)
        y = B.gemm(dx, w)                                  # a consumer right behind the chain
        assert torch.equal(dx, ref_dx) and torch.equal(dw, ref_dw) and torch.equal(db, ref_db), it
        assert torch.equal(y, ref_y), it


@pytest.mark.parametrize("M,N,K,bias,out_dtype,acc,two", [
    (32, 27, 131072, False, torch.float32, True, True),   # conv weight gradient: odd N, very long K
    (128, 10, 8192, True, torch.bfloat16, False, True),   # classifier head: bias added by the reduction
    (64, 288, 32768, False, torch.float32, False, False),
])
def test_gemm_split_k_any_width_and_bias(M, N, K, bias, out_dtype, acc, two):
    """Long-K products with a single output tile are cut along K whatever the output width:
    workspace rows are padded to four floats and the closing pass adds the bias."""
    from luatorch_b200 import _backend as B
    torch.manual_seed(22)
    a = (torch.randn(K, M, device="cuda") * 0.1).bfloat16()        # stored [K, M]: a_t
    ldb = (N + 7) // 8 * 8
    bfull = torch.zeros(K, ldb, device="cuda", dtype=torch.bfloat16)
    bfull[:, :N] = (torch.randn(K, N, device="cuda") * 0.1).bfloat16()
    b = bfull[:, :N]
    bv = torch.randn(N, device="cuda").bfloat16() if bias else None
    ldc = (N + 7) // 8 * 8 if out_dtype == torch.bfloat16 else N
    out_full = torch.full((M, ldc), 0.25, device="cuda", dtype=out_dtype)
    out = out_full[:, :N]
    before = sum(lf_launches())
    B.gemm(a, b, a_t=True, out=out, accumulate=acc, bias=bv, n_valid=N)
    if two:
        assert sum(lf_launches()) - before == 2        # sliced product + closing pass
    ref = a.float().t() @ b.float()
    if bias:
        ref = ref + bv.float()
    if acc:
        ref = ref + 0.25
    tol = dict(atol=2e-2, rtol=2e-3) if out_dtype == torch.float32 else dict(atol=0.15, rtol=2e-2)
    torch.testing.assert_close(out.float(), ref, **tol)
    if ldc > N:
        assert torch.all(out_full[:, N:] == 0.25)      # nothing written beyond the logical width


def test_flash_backward_second_generation_at_head_dim_128():
    """LT_FLASH_BWD2_D128=1 runs the tensor-memory-operand backward (the default at head dim 64)
    at head dim 128 too; the switch is read once per process, so it runs in its own.  Gradients
    against fp32 attention."""
    import subprocess, sys, os
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    body = r'''
import sys, math, torch
sys.path.insert(0, %r)
from luatorch_b200 import _C
torch.manual_seed(33)
B, S, H, D = 2, 512, 3, 128
qkv = (torch.randn(B, S, 3, H, D, device="cuda") * 0.5).bfloat16()
q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
sc = 1.0 / math.sqrt(D)
o, lse = _C.flash_forward(q, k, v, True, sc)
d_o = (torch.randn_like(o.float()) * 0.5).bfloat16()
dq, dk, dv = _C.flash_backward(q, k, v, o, lse, d_o, True, sc, None)[:3]
qf, kf, vf = (t.float().permute(0, 2, 1, 3).requires_grad_(True) for t in (q, k, v))
s = qf @ kf.transpose(-1, -2) * sc
s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool, device="cuda"), 1), float("-inf"))
ref = torch.softmax(s, -1) @ vf
ref.backward(d_o.float().permute(0, 2, 1, 3))
for name, got, want in (("dq", dq, qf.grad), ("dk", dk, kf.grad), ("dv", dv, vf.grad)):
    err = (got.float().permute(0, 2, 1, 3) - want).abs().max().item()
    assert err < 0.06 * max(1.0, want.abs().max().item()), (name, err)
print("BWD2_D128_OK")
''' % root
    env = dict(os.environ, LT_FLASH_BWD2_D128="1")
    r = subprocess.run([sys.executable, "-c", body], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and "BWD2_D128_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-2000:])
