"""Ported assertions of the reference's test_tensor.lua, test_arithmetic.lua and
test_matmul.lua (test/test_tensor.lua:9-71, test/test_arithmetic.lua:15-96,
test/test_matmul.lua:12-63), run against the Python front end on CPU."""
import math

import luatorch_b200 as lf

T = lf.Tensor


def near(a, b, tol=1e-5):
    assert abs(a - b) < tol, (a, b)


def vec(vals, shape=None):
    return T.from_list(vals, shape or [len(vals)])


def test_creation_shape_numel():
    t = T.new([3, 4])
    assert t.shape == [3, 4] and t.ndim == 2 and t.numel() == 12
    assert t.dtype == "float32" and t.device == "cpu"
    assert str(t) == "Tensor(shape=3x4, dtype=float32, device=cpu)"


def test_fill_zeros_ones_rand():
    t = T.new([2, 3]).fill(7.5)
    for i in range(6):
        near(t.get(i), 7.5)
    t.zeros()
    assert T.sum(t) == 0
    t.ones()
    near(T.sum(t), 6)
    t.rand()
    assert any(t.get(i) != 0 for i in range(6))
    assert 0 <= T.min(t) and T.max(t) < 1
    big = T.new([10000]).randn()
    near(T.mean(big), 0.0, 0.05)


def test_get_set_bounds_and_copy():
    t = T.new([2, 2])
    t.set(3, 4.25)
    near(t.get(3), 4.25)
    assert t.get(99) == 0.0            # out of range: error printed, 0 returned
    t.set(99, 1.0)                     # ignored
    c = t.copy()
    c.set(0, 9.0)
    assert t.get(0) == 0.0 and c.get(0) == 9.0


def test_reshape_shares_storage():
    t = T.new([2, 3])
    r = t.reshape([3, 2])
    r.set(5, 2.0)
    assert t.get(5) == 2.0 and r.shape == [3, 2]
    assert t.reshape([4, 4]) is None


def test_elementwise_known_values():
    a, b = vec([1, 2, 3, 4]), vec([4, 3, 2, 1])
    assert T.add(a, b).tolist() == [5, 5, 5, 5]
    assert T.sub(a, b).tolist() == [-3, -1, 1, 3]
    assert T.mul(a, b).tolist() == [4, 6, 6, 4]
    near(T.div(a, b).get(0), 0.25)
    assert (a + b).tolist() == [5, 5, 5, 5] and (-a).tolist() == [-1, -2, -3, -4]
    assert (a * b).tolist() == [4, 6, 6, 4] and (a - b).get(0) == -3


def test_scalar_unary_reductions():
    a = vec([1, 4, 9, 16])
    assert T.add_scalar(a, 1).tolist() == [2, 5, 10, 17]
    assert T.mul_scalar(a, 2).tolist() == [2, 8, 18, 32]
    assert T.div_scalar(a, 2).tolist() == [0.5, 2, 4.5, 8]
    assert T.pow_scalar(a, 0.5).tolist() == [1, 2, 3, 4]
    assert T.sqrt(a).tolist() == [1, 2, 3, 4]
    assert T.abs(vec([-1, 2, -3])).tolist() == [1, 2, 3]
    near(T.exp(vec([0, 1])).get(1), math.e, 1e-5)
    near(T.log(vec([1, math.e])).get(1), 1.0, 1e-5)
    near(T.sum(a), 30)
    near(T.mean(a), 7.5)
    assert T.max(a) == 16 and T.min(a) == 1


def test_edge_cases_do_not_crash():
    assert T.div(vec([1, 2]), vec([0, 2])).tolist() == [0, 1]      # x/0 -> 0
    assert T.sqrt(vec([-4.0])).get(0) == 0
    assert T.log(vec([0.0])).get(0) == -math.inf
    assert T.add(vec([1, 2]), vec([1, 2, 3])) is None                # size mismatch -> nil


def test_inplace_and_broadcast():
    a = vec([1, 2, 3])
    T.add_(a, vec([1, 1, 1]))
    assert a.tolist() == [2, 3, 4]
    T.sub_(a, vec([1, 1, 1]))
    T.mul_scalar_(a, 3)
    T.add_scalar_(a, 1)
    assert a.tolist() == [4, 7, 10]
    m = vec([1, 2, 3, 4, 5, 6], [2, 3])
    out = T.add_broadcast(m, vec([10, 20, 30]))
    assert out.tolist() == [[11, 22, 33], [14, 25, 36]]
    assert T.add_broadcast_backward(m).tolist() == [5, 7, 9]


def test_matmul_family():
    a = vec([1, 2, 3, 4], [2, 2])
    b = vec([5, 6, 7, 8], [2, 2])
    assert T.matmul(a, b).tolist() == [[19, 22], [43, 50]]
    c = T.matmul(vec([1, 2, 3, 4, 5, 6], [2, 3]), vec([1, 2, 3, 4, 5, 6], [3, 2]))
    assert c.tolist() == [[22, 28], [49, 64]]
    assert T.transpose(vec([1, 2, 3, 4, 5, 6], [2, 3])).tolist() == [[1, 4], [2, 5], [3, 6]]
    near(T.dot(vec([1, 2, 3]), vec([4, 5, 6])), 32)
    assert T.matmul(a, vec([1, 2, 3], [3, 1])) is None
    bm = T.bmm(vec([1, 0, 0, 1, 2, 0, 0, 2], [2, 2, 2]), vec([1, 2, 3, 4, 1, 2, 3, 4], [2, 2, 2]))
    assert bm.tolist() == [[[1, 2], [3, 4]], [[2, 4], [6, 8]]]


def test_activations_softmax_losses():
    x = vec([-1, 0, 2])
    assert T.relu(x).tolist() == [0, 0, 2]
    near(T.sigmoid(x).get(1), 0.5)
    near(T.tanh(x).get(2), math.tanh(2), 1e-6)
    near(T.gelu(x).get(2), 0.5 * 2 * (1 + math.tanh(0.7978845608 * (2 + 0.044715 * 8))), 1e-5)
    near(T.silu(x).get(2), 2 / (1 + math.exp(-2)), 1e-6)
    assert T.gt_scalar(x, 0).tolist() == [0, 0, 1]
    sm = T.softmax(vec([1, 2, 3, 1, 2, 3], [2, 3]))
    near(sum(sm.tolist()[0]), 1.0)
    near(sm.get(2), math.exp(3) / (math.exp(1) + math.exp(2) + math.exp(3)), 1e-6)
    p, t = vec([1, 2, 3, 4]), vec([1, 2, 3, 6])
    near(T.mse_loss(p, t).get(0), 1.0)
    near(T.mae_loss(p, t).get(0), 0.5)
    assert T.mse_loss_backward(p, t).tolist() == [0, 0, 0, -1]
    logits = vec([2, 1, 0, 0, 1, 2], [2, 3])
    labels = vec([0, 2])
    lse = math.log(math.exp(2) + math.exp(1) + 1)
    near(T.cross_entropy_loss(logits, labels).get(0), lse - 2, 1e-5)
    g = T.cross_entropy_loss_backward(logits, labels)
    near(g.get(0), (math.exp(2 - lse) - 1) / 2, 1e-6)
    assert T.cross_entropy_loss(logits, vec([0, 7])) is None


def test_fused_ops_have_cpu_paths():
    x = vec([0.5, -1, 2, 3, 0, 1], [2, 3])
    y = T.fused_layernorm(x, vec([1, 1, 1]), vec([0, 0, 0]))
    near(sum(y.tolist()[0]), 0.0, 1e-5)
    gb = T.fused_gelu_bias(x, vec([1, 1, 1]))
    near(gb.get(1), 0.0, 1e-6)
    q = T.new([2, 4, 8]).randn()
    o = T.flash_attention(q, q, q, 2, 4, 8, True)
    assert o.shape == [2, 4, 8]
    near(o.get(0), q.get(0), 1e-5)     # first causal row attends to itself only
    cols = T.im2col(T.new([1 * 1 * 3 * 3]).ones(), 1, 1, 3, 3, 2, 1, 0)
    assert cols.shape == [4, 4] and T.sum(cols) == 16


def test_functional_ops_layer_on_cpu():
    """lf.ops: the kernel-level functional surface, CPU path against torch."""
    import torch
    import luatorch_b200 as lf
    ops = lf.ops
    g = torch.Generator().manual_seed(3)
    x = torch.randn(6, 16, generator=g)
    gamma, beta = torch.rand(16, generator=g) + 0.5, torch.randn(16, generator=g)
    y, mean, rstd = ops.layernorm(x, gamma, beta, 1e-5)
    torch.testing.assert_close(y, torch.nn.functional.layer_norm(x, (16,), gamma, beta, 1e-5),
                               rtol=1e-5, atol=1e-5)
    bias = torch.randn(16, generator=g)
    torch.testing.assert_close(ops.gelu_bias(x, bias),
                               torch.nn.functional.gelu(x + bias, approximate="tanh"), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(ops.softmax(x), torch.softmax(x, -1))
    labels = torch.randint(0, 16, (6,), generator=g).float()
    loss = ops.cross_entropy(x, labels)
    torch.testing.assert_close(loss.reshape(()), torch.nn.functional.cross_entropy(x, labels.long()))
    dl = ops.cross_entropy_backward(x, labels)
    xr = x.clone().requires_grad_(True)
    torch.nn.functional.cross_entropy(xr, labels.long()).backward()
    torch.testing.assert_close(dl, xr.grad, rtol=1e-5, atol=1e-6)
    a, b = torch.randn(5, 7, generator=g), torch.randn(7, 3, generator=g)
    torch.testing.assert_close(ops.matmul(a, b), a @ b)
    torch.testing.assert_close(ops.column_sum(a), a.sum(0))
    for name in ops.__all__:
        assert callable(getattr(ops, name)), name
