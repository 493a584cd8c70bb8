"""Ported assertions of test_autograd.lua, test_nn.lua, test_optim.lua and test_training.lua
(test/test_autograd.lua:11-113, test/test_nn.lua:18-127, test/test_optim.lua:17-84,
test/test_training.lua:11-104) plus gradient checks of every layer against torch.autograd."""
import math

import pytest
import torch

import luatorch_b200 as lf

T, ag, nn = lf.Tensor, lf.autograd, lf.nn


def vec(vals, shape=None):
    return T.from_list(vals, shape or [len(vals)])


def test_add_mul_matmul_grads_and_accumulation():
    ag.zero_graph()
    a, b = ag.watch(vec([1, 2, 3])), ag.watch(vec([4, 5, 6]))
    out = ag.mul(ag.add(a, b), b)
    ag.backward(out)
    assert a.grad.tolist() == [4, 5, 6]
    assert b.grad.tolist() == [9, 12, 15]          # (a+b) + b
    ag.zero_graph()
    ag.zero_grad([a, b])
    assert a.grad is None
    s = ag.add(a, a)
    ag.backward(s)
    assert a.grad.tolist() == [2, 2, 2]            # used twice -> accumulated
    ag.zero_graph()
    x, w = ag.watch(vec([1, 2, 3, 4], [2, 2])), ag.watch(vec([1, 0, 0, 1], [2, 2]))
    y = ag.relu(ag.matmul(x, w))
    ag.backward(y)
    assert x.grad.tolist() == [[1, 1], [1, 1]] and w.grad.tolist() == [[4, 4], [6, 6]]


def test_no_grad_and_enabled_flag():
    ag.zero_graph()
    a = ag.watch(vec([1.0]))
    with ag.no_grad():
        ag.add(a, a)
    assert len(ag.graph) == 0
    ag.add(a, a)
    assert len(ag.graph) == 1


def _torch_layer_check(build, torch_fn, x_shape, tol=1e-4, seed=0):
    """Compare a layer's output and gradients with the same math in torch.autograd."""
    lf.manual_seed(seed)
    ag.zero_graph()
    layer = build()
    x = T.new(list(x_shape)).randn()
    ag.watch(x)
    y = layer(x)
    y = y[0] if isinstance(y, tuple) else y
    w = torch.randn(y._t.shape, generator=torch.Generator().manual_seed(1))
    ag.backward(y, T.wrap(w.clone()))
    xt = x._t.clone().requires_grad_(True)
    pts = [p._t.clone().requires_grad_(True) for p in layer.parameters()]
    yt = torch_fn(xt, *pts)
    yt.backward(w)
    torch.testing.assert_close(y._t, yt.detach(), atol=tol, rtol=tol)
    torch.testing.assert_close(x.grad._t.reshape(xt.shape), xt.grad, atol=tol, rtol=tol)
    for p, pt in zip(layer.parameters(), pts):
        assert p.grad is not None, "missing parameter gradient"
        torch.testing.assert_close(p.grad._t.reshape(pt.shape), pt.grad, atol=tol, rtol=tol)


def gelu_t(x):
    return 0.5 * x * (1 + torch.tanh(0.7978845608 * (x + 0.044715 * x ** 3)))


def test_linear_layernorm_activation_grads():
    _torch_layer_check(lambda: nn.Linear(5, 3), lambda x, w, b: x @ w + b, (4, 5))
    _torch_layer_check(lambda: nn.Linear(5, 3, False), lambda x, w: x @ w, (4, 5))
    _torch_layer_check(lambda: nn.LayerNorm(6),
                       lambda x, g, b: torch.nn.functional.layer_norm(x, (6,), g, b, 1e-5), (3, 6))
    for cls, fn in [(nn.ReLU, torch.relu), (nn.Sigmoid, torch.sigmoid), (nn.Tanh, torch.tanh),
                    (nn.GELU, gelu_t), (nn.SiLU, lambda x: x * torch.sigmoid(x))]:
        _torch_layer_check(cls, fn, (3, 7))


def test_batchnorm_train_eval_and_grads():
    _torch_layer_check(lambda: nn.BatchNorm1d(4),
                       lambda x, g, b: torch.nn.functional.batch_norm(x, None, None, g, b, True, 0.1, 1e-5),
                       (8, 4), tol=1e-3)
    bn = nn.BatchNorm1d(3)
    x = T.new([16, 3]).randn()
    bn(x)
    assert abs(bn.running_mean.get(0) - 0.1 * float(x._t[:, 0].mean())) < 1e-5
    bn.eval()
    y = bn(x)
    ref = (x._t - bn.running_mean._t) / torch.sqrt(bn.running_var._t + 1e-5)
    torch.testing.assert_close(y._t, ref, atol=1e-5, rtol=1e-5)


def test_embedding_positional_dropout():
    lf.manual_seed(3)
    ag.zero_graph()
    emb = nn.Embedding(10, 4)
    ids = vec([1, 3, 3, 9])
    out = emb(ids)
    assert out.shape == [4, 4]
    torch.testing.assert_close(out._t[1], emb.weight._t[3])
    ag.backward(out)
    assert emb.weight.grad._t[3].tolist() == [2, 2, 2, 2] and emb.weight.grad._t[0].abs().sum() == 0
    ag.zero_graph()
    pe = nn.LearnedPE(8, 4)
    x = ag.watch(T.new([6, 4]).randn())
    y = pe(x, 3)
    torch.testing.assert_close(y._t[4], x._t[4] + pe.weight._t[1])
    ag.backward(y)
    assert pe.weight.grad._t[0].tolist() == [2, 2, 2, 2] and pe.weight.grad._t[5].abs().sum() == 0
    sp = nn.SinusoidalPE(16, 4)
    assert abs(sp.pe.get(1 * 4 + 0) - math.sin(1.0)) < 1e-6 and abs(sp.pe.get(1) - 1.0) < 1e-6
    d = nn.Dropout(0.5)
    ones = T.new([10000]).ones()
    rate = float((d(ones)._t == 0).float().mean())
    assert 0.3 < rate < 0.7
    d.eval()
    assert d(ones) is ones


def test_attention_grads_batch_separation_and_causality():
    E, H, S, Bn = 8, 2, 5, 2
    lf.manual_seed(4)
    for cls, causal in [(nn.MultiHeadAttention, False), (nn.FlashMultiHeadAttention, True)]:
        ag.zero_graph()
        attn = cls(E, H)
        x = ag.watch(T.new([Bn * S, E]).randn())
        y = attn(x, seq_len=S)
        w = torch.randn(y._t.shape, generator=torch.Generator().manual_seed(2))
        ag.backward(y, T.wrap(w.clone()))
        xt = x._t.clone().requires_grad_(True)
        ps = [p._t.clone().requires_grad_(True) for p in attn.parameters()]
        wq, wk, wv, wo, bo = ps
        def heads(t):
            return t.reshape(Bn, S, H, E // H).permute(0, 2, 1, 3)
        q, k, v = heads(xt @ wq), heads(xt @ wk), heads(xt @ wv)
        s = q @ k.transpose(-1, -2) / math.sqrt(E // H)
        if causal:
            s = s.masked_fill(torch.triu(torch.ones(S, S, dtype=torch.bool), 1), -math.inf)
        o = (torch.softmax(s, -1) @ v).permute(0, 2, 1, 3).reshape(Bn * S, E)
        yt = o @ wo + bo
        yt.backward(w)
        torch.testing.assert_close(y._t, yt.detach(), atol=1e-4, rtol=1e-4)
        torch.testing.assert_close(x.grad._t, xt.grad, atol=1e-4, rtol=1e-4)
        for p, pt in zip(attn.parameters(), ps):
            torch.testing.assert_close(p.grad._t, pt.grad, atol=1e-4, rtol=1e-4)


def test_transformer_block_gradient_crosses_residuals():
    lf.manual_seed(5)
    ag.zero_graph()
    blk = nn.TransformerBlock(8, 2, 0.0)
    x = ag.watch(T.new([6, 8]).randn())
    y = blk(x, 3)
    ag.backward(y)
    assert x.grad is not None and float(x.grad._t.abs().sum()) > 0
    assert all(p.grad is not None for p in blk.parameters())
    assert len(blk.parameters()) == 2 + 5 + 2 + 2 + 2


def test_conv2d_matches_torch():
    lf.manual_seed(6)
    ag.zero_graph()
    conv = nn.Conv2d(3, 4, 3, 2, 1)
    x = ag.watch(T.new([2 * 3 * 7 * 7]).randn())
    out, oh, ow = conv(x, 2, 7, 7)
    assert (oh, ow) == (4, 4) and out.shape == [2 * 16, 4]
    w = torch.randn(out._t.shape, generator=torch.Generator().manual_seed(3))
    ag.backward(out, T.wrap(w.clone()))
    xt = x._t.reshape(2, 3, 7, 7).clone().requires_grad_(True)
    wt = conv.weight._t.reshape(4, 3, 3, 3).clone().requires_grad_(True)
    bt = conv.bias._t.clone().requires_grad_(True)
    yt = torch.nn.functional.conv2d(xt, wt, bt, 2, 1).permute(0, 2, 3, 1).reshape(-1, 4)
    yt.backward(w)
    torch.testing.assert_close(out._t, yt.detach(), atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(x.grad._t.reshape(2, 3, 7, 7), xt.grad, atol=1e-4, rtol=1e-4)
    torch.testing.assert_close(conv.weight.grad._t.reshape(4, 3, 3, 3), wt.grad, atol=1e-4, rtol=1e-4)
    nchw = nn.to_nchw(out, 2, 4, 16)
    torch.testing.assert_close(nchw._t.reshape(2, 4, 16), yt.detach().reshape(2, 16, 4).transpose(1, 2))


def test_optimizers_and_schedulers():
    x = ag.watch(vec([5.0]))
    opt = lf.optim.Adam([x], 0.1)
    for _ in range(100):
        x.grad = T.mul_scalar(x, 2.0)          # d/dx x^2
        opt.step()
    assert abs(x.get(0)) < 0.5
    w = ag.watch(vec([1.0]))
    ow = lf.optim.AdamW([w], 0.1, None, None, None, 0.1)
    w.grad = vec([0.0])
    ow.step()
    assert w.get(0) < 1.0                       # decays even with zero gradient
    nd = ag.watch(vec([1.0]))
    o2 = lf.optim.AdamW([nd], 0.1, None, None, None, 0.1, [nd])
    nd.grad = vec([0.0])
    o2.step()
    assert nd.get(0) == 1.0
    s = ag.watch(vec([1.0]))
    sgd = lf.optim.SGD([s], 0.1, 0.9)
    s.grad = vec([1.0]); sgd.step()
    s.grad = vec([1.0]); sgd.step()
    assert abs(s.get(0) - (1 - 0.1 - 0.1 * 1.9)) < 1e-6
    opt = lf.optim.Adam([x], 0.1)
    cos = lf.optim.CosineAnnealing(opt, 10)
    lrs = [cos.step() for _ in range(10)]
    assert all(a > b for a, b in zip(lrs, lrs[1:])) and lrs[-1] < 1e-9
    opt = lf.optim.Adam([x], 0.1)
    st = lf.optim.StepLR(opt, 2, 0.5)
    assert abs(st.step() - 0.1) < 1e-12 and abs(st.step() - 0.05) < 1e-12
    opt = lf.optim.Adam([x], 0.1)
    wu = lf.optim.WarmupScheduler(opt, 10)
    assert 0 < wu.step() < 0.1


def _xor_model(hidden):
    return nn.Sequential(nn.Linear(2, hidden), nn.Tanh(), nn.Linear(hidden, 1), nn.Sigmoid())


def test_xor_training_and_checkpoint_roundtrip(tmp_path):
    # config: Linear(2,8)-Tanh-Linear(8,1)-Sigmoid, MSE, Adam lr 0.01, 2000 full-batch steps
    lf.manual_seed(1234)
    model = _xor_model(8)
    crit = nn.MSELoss()
    opt = lf.optim.Adam(model.parameters(), 0.01)
    x = vec([0, 0, 0, 1, 1, 0, 1, 1], [4, 2])
    y = vec([0, 1, 1, 0], [4, 1])
    loss = None
    for _ in range(2000):
        ag.zero_graph()
        model.zero_grad()
        loss = crit(model(x), y)
        ag.backward(loss)
        opt.step()
    assert loss.get(0) < 0.05
    path = str(tmp_path / "xor.bin")
    lf.io.checkpoint.save(model, path)
    lf.manual_seed(99)
    fresh = _xor_model(8)
    lf.io.checkpoint.load(fresh, path)
    torch.testing.assert_close(fresh(x)._t, model(x)._t, atol=1e-5, rtol=0)
    with pytest.raises(ValueError):
        lf.io.checkpoint.load(_xor_model(4), path)


def test_loss_scaling_reaches_parameters():
    lf.manual_seed(7)
    ag.zero_graph()
    lin = nn.Linear(3, 2)
    x = T.new([4, 3]).randn()
    t = T.new([4, 2]).randn()
    loss = nn.MSELoss()(lin(x), t)
    ag.backward(loss)
    base = lin.weight.grad._t.clone()
    ag.zero_graph(); lin.zero_grad()
    scaler = lf.cuda.amp.GradScaler(8.0)
    loss = scaler.scale_loss(nn.MSELoss()(lin(x), t))
    ag.backward(loss)
    torch.testing.assert_close(lin.weight.grad._t, base * 8.0, atol=1e-5, rtol=1e-5)
    opt = lf.optim.SGD(lin.parameters(), 0.1, 0.0)
    before = lin.weight._t.clone()
    scaler.step(opt); scaler.update()
    torch.testing.assert_close(lin.weight._t, before - 0.1 * base, atol=1e-6, rtol=1e-5)
    lin.weight.grad = T.wrap(torch.full_like(base, float("inf")))
    w0 = lin.weight._t.clone()
    scaler.step(opt); scaler.update()
    assert torch.equal(lin.weight._t, w0) and scaler.get_scale() == 4.0
