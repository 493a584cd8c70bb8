"""The C ABI of libluatorch.so, exercised through ctypes the way the LuaJIT FFI front end would
(lua/luatorch/tensor.lua:8-179): struct layout, the full symbol list, CPU op values (ported
from test/test_tensor.lua, test_arithmetic.lua, test_matmul.lua) and, on a GPU, the
test/test_cuda.lua checks (round trip, add and matmul against the CPU ops, pool counters)
plus every fused op against the CPU path."""
import ctypes as C
import math
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.environ.get("LUATORCH_LIB") or os.path.join(ROOT, "luatorch_b200", "lib", "libluatorch.so")


class CT(C.Structure):
    _fields_ = [("data", C.POINTER(C.c_float)), ("cuda_data", C.c_void_p), ("shape", C.POINTER(C.c_int64)),
                ("strides", C.POINTER(C.c_int64)), ("ndim", C.c_int), ("numel", C.c_int64),
                ("dtype", C.c_int), ("device", C.c_int), ("requires_grad", C.c_int),
                ("grad", C.c_void_p), ("ref_count", C.c_int)]


TP = C.POINTER(CT)

T_T = ["tensor_copy", "tensor_neg", "tensor_abs", "tensor_sqrt", "tensor_log", "tensor_exp", "tensor_relu",
       "tensor_sigmoid", "tensor_tanh", "tensor_gelu", "tensor_silu", "tensor_softmax", "tensor_transpose",
       "tensor_add_broadcast_backward", "tensor_to_cuda", "tensor_to_cpu", "tensor_to_cuda_async",
       "tensor_to_cpu_async"]
T_TT = ["tensor_add", "tensor_sub", "tensor_mul", "tensor_div", "tensor_add_broadcast", "tensor_matmul",
        "tensor_bmm", "tensor_mse_loss", "tensor_mse_loss_backward", "tensor_mae_loss",
        "tensor_mae_loss_backward", "tensor_cross_entropy_loss", "tensor_cross_entropy_loss_backward"]
T_TF = ["tensor_add_scalar", "tensor_mul_scalar", "tensor_div_scalar", "tensor_pow_scalar", "tensor_gt_scalar"]
F_T = ["tensor_sum", "tensor_mean", "tensor_max", "tensor_min"]
V_TT = ["tensor_add_", "tensor_sub_"]
V_TF = ["tensor_mul_scalar_", "tensor_add_scalar_"]
CUDA_ONLY = ["tensor_matmul_cuda_naive", "tensor_fused_gelu_bias_cuda", "tensor_fused_layernorm_cuda",
             "tensor_fused_adam_cuda", "tensor_flash_attention_cuda", "tensor_has_inf_nan_cuda",
             "tensor_scale_cuda", "tensor_fused_cross_entropy_cuda", "tensor_cast_f32_to_f16_cuda",
             "tensor_cast_f16_to_f32_cuda", "tensor_new_cuda", "tensor_cuda_free", "tensor_sync"]
OTHER = ["tensor_new", "tensor_free", "tensor_fill", "tensor_zeros", "tensor_ones", "tensor_rand", "tensor_randn",
         "tensor_print", "tensor_copy_data", "tensor_get", "tensor_set", "tensor_reshape", "tensor_numel",
         "tensor_im2col", "tensor_dot", "pool_init", "pool_clear", "pool_alloc", "pool_free",
         "pool_allocated_bytes", "pool_cached_bytes", "cuda_memory_allocated", "cuda_memory_cached",
         "luatorch_nccl_get_gpu_count", "luatorch_nccl_init", "luatorch_nccl_allreduce",
         "luatorch_nccl_broadcast", "luatorch_nccl_destroy"]


def _cuda_name(n):
    if n.endswith("_") and not n.endswith("__"):
        return n[:-1] + "_cuda_"
    return n + "_cuda"


@pytest.fixture(scope="module")
def lib():
    assert os.path.exists(LIB), "run python -m luatorch_b200.build"
    L = C.CDLL(LIB)
    for group, res, args in [(T_T, TP, [TP]), (T_TT, TP, [TP, TP]), (T_TF, TP, [TP, C.c_float]),
                             (F_T, C.c_float, [TP]), (V_TT, None, [TP, TP]), (V_TF, None, [TP, C.c_float])]:
        for n in group:
            for name in (n, _cuda_name(n)):
                if hasattr(L, name):
                    getattr(L, name).restype, getattr(L, name).argtypes = res, args
    L.tensor_new.restype, L.tensor_new.argtypes = TP, [C.POINTER(C.c_int64), C.c_int, C.c_int, C.c_int]
    L.tensor_new_cuda.restype, L.tensor_new_cuda.argtypes = TP, [C.POINTER(C.c_int64), C.c_int, C.c_int]
    L.tensor_reshape.restype, L.tensor_reshape.argtypes = TP, [TP, C.POINTER(C.c_int64), C.c_int]
    L.tensor_free.argtypes = [TP]
    L.tensor_get.restype, L.tensor_get.argtypes = C.c_float, [TP, C.c_int64]
    L.tensor_set.argtypes = [TP, C.c_int64, C.c_float]
    L.tensor_fill.argtypes = [TP, C.c_float]
    for n in ("tensor_zeros", "tensor_ones", "tensor_rand", "tensor_randn", "tensor_print"):
        getattr(L, n).argtypes = [TP]
    L.tensor_numel.restype, L.tensor_numel.argtypes = C.c_int64, [TP]
    L.tensor_copy_data.argtypes = [TP, TP]
    L.tensor_dot.restype, L.tensor_dot.argtypes = C.c_float, [TP, TP]
    L.tensor_dot_cuda.restype, L.tensor_dot_cuda.argtypes = C.c_float, [TP, TP]
    L.tensor_im2col.restype, L.tensor_im2col.argtypes = TP, [TP] + [C.c_int] * 7
    L.tensor_fused_gelu_bias_cuda.restype, L.tensor_fused_gelu_bias_cuda.argtypes = TP, [TP, TP]
    L.tensor_fused_layernorm_cuda.restype, L.tensor_fused_layernorm_cuda.argtypes = TP, [TP, TP, TP, C.c_float]
    L.tensor_fused_adam_cuda.argtypes = [TP] * 4 + [C.c_float] * 7
    L.tensor_flash_attention_cuda.restype = TP
    L.tensor_flash_attention_cuda.argtypes = [TP, TP, TP, C.c_int, C.c_int, C.c_int, C.c_int]
    L.tensor_has_inf_nan_cuda.restype, L.tensor_has_inf_nan_cuda.argtypes = C.c_int, [TP]
    L.tensor_scale_cuda.argtypes = [TP, C.c_float]
    L.tensor_fused_cross_entropy_cuda.restype, L.tensor_fused_cross_entropy_cuda.argtypes = TP, [TP, TP]
    L.cuda_memory_allocated.restype = C.c_size_t
    L.cuda_memory_cached.restype = C.c_size_t
    L.luatorch_manual_seed.argtypes = [C.c_uint64]
    return L


def new(L, shape, vals=None):
    arr = (C.c_int64 * len(shape))(*shape)
    t = L.tensor_new(arr, len(shape), 0, 0)
    if vals is not None:
        for i, v in enumerate(vals):
            L.tensor_set(t, i, float(v))
    return t


def values(L, t):
    return [L.tensor_get(t, i) for i in range(t.contents.numel)]


def test_struct_layout_and_symbol_list(lib):
    assert C.sizeof(CT) == 80
    for name, off in [("data", 0), ("cuda_data", 8), ("shape", 16), ("strides", 24), ("ndim", 32), ("numel", 40),
                      ("dtype", 48), ("device", 52), ("requires_grad", 56), ("grad", 64), ("ref_count", 72)]:
        assert getattr(CT, name).offset == off, name
    wanted = set(OTHER + CUDA_ONLY)
    for n in T_T + T_TT + T_TF + F_T + V_TT + V_TF:
        wanted.add(n)
        if not n.startswith(("tensor_to_", "tensor_copy")):
            wanted.add(_cuda_name(n))
    wanted.add("tensor_dot_cuda")
    missing = [n for n in sorted(wanted) if not hasattr(lib, n)]
    assert not missing, missing


def test_cpu_tensor_basics(lib):
    L = lib
    t = new(L, [3, 4])
    assert t.contents.ndim == 2 and t.contents.numel == 12 and t.contents.shape[1] == 4
    assert t.contents.strides[0] == 4 and t.contents.device == 0 and t.contents.ref_count == 1
    L.tensor_fill(t, 7.5)
    assert all(v == 7.5 for v in values(L, t))
    L.tensor_set(t, 3, 1.25)
    assert L.tensor_get(t, 3) == 1.25 and L.tensor_get(t, 99) == 0.0
    c = L.tensor_copy(t)
    L.tensor_set(c, 0, 9.0)
    assert L.tensor_get(t, 0) == 7.5
    L.luatorch_manual_seed(5)
    r = new(L, [10000])
    L.tensor_randn(r)
    assert abs(L.tensor_mean(r)) < 0.05
    L.tensor_rand(r)
    assert 0.0 <= L.tensor_min(r) and L.tensor_max(r) < 1.0
    view = L.tensor_reshape(t, (C.c_int64 * 2)(4, 3), 2)
    L.tensor_set(view, 11, 2.0)
    assert L.tensor_get(t, 11) == 2.0 and t.contents.ref_count == 2
    L.tensor_free(view)                      # storage stays alive: the source still owns it
    assert t.contents.ref_count == 1 and L.tensor_get(t, 11) == 2.0
    assert not L.tensor_reshape(t, (C.c_int64 * 1)(5), 1)
    for x in (t, c, r):
        L.tensor_free(x)


def test_cpu_ops_known_values(lib):
    L = lib
    a, b = new(L, [4], [1, 2, 3, 4]), new(L, [4], [4, 3, 2, 1])
    assert values(L, L.tensor_add(a, b)) == [5, 5, 5, 5]
    assert values(L, L.tensor_mul(a, b)) == [4, 6, 6, 4]
    assert values(L, L.tensor_div(a, new(L, [4], [0, 1, 1, 1])))[0] == 0
    assert not L.tensor_add(a, new(L, [3]))
    assert values(L, L.tensor_sqrt(new(L, [2], [-4, 9]))) == [0, 3]
    assert values(L, L.tensor_log(new(L, [1], [0])))[0] == -math.inf
    assert L.tensor_sum(a) == 10 and L.tensor_mean(a) == 2.5 and L.tensor_max(a) == 4 and L.tensor_min(a) == 1
    L.tensor_add_(a, b)
    assert values(L, a) == [5, 5, 5, 5]
    m = new(L, [2, 2], [1, 2, 3, 4])
    assert values(L, L.tensor_matmul(m, new(L, [2, 2], [5, 6, 7, 8]))) == [19, 22, 43, 50]
    assert values(L, L.tensor_transpose(new(L, [2, 3], [1, 2, 3, 4, 5, 6]))) == [1, 4, 2, 5, 3, 6]
    assert not L.tensor_matmul(m, new(L, [3, 1]))
    assert L.tensor_dot(new(L, [3], [1, 2, 3]), new(L, [3], [4, 5, 6])) == 32
    assert values(L, L.tensor_add_broadcast(new(L, [2, 3], [1, 2, 3, 4, 5, 6]), new(L, [3], [10, 20, 30]))) == [11, 22, 33, 14, 25, 36]
    assert values(L, L.tensor_add_broadcast_backward(new(L, [2, 3], [1, 2, 3, 4, 5, 6]))) == [5, 7, 9]
    sm = values(L, L.tensor_softmax(new(L, [2, 3], [1, 2, 3, 1, 2, 3])))
    assert abs(sum(sm[:3]) - 1) < 1e-6
    logits, labels = new(L, [2, 3], [2, 1, 0, 0, 1, 2]), new(L, [2], [0, 2])
    lse = math.log(math.exp(2) + math.exp(1) + 1)
    assert abs(L.tensor_get(L.tensor_cross_entropy_loss(logits, labels), 0) - (lse - 2)) < 1e-5
    assert not L.tensor_cross_entropy_loss(logits, new(L, [2], [0, 7]))
    assert abs(L.tensor_get(L.tensor_mse_loss(new(L, [2], [1, 3]), new(L, [2], [1, 1])), 0) - 2.0) < 1e-6
    cols = L.tensor_im2col(new(L, [9], [1] * 9), 1, 1, 3, 3, 2, 1, 0)
    assert cols.contents.shape[0] == 4 and cols.contents.shape[1] == 4 and L.tensor_sum(cols) == 16


def _from_np(L, arr):
    import numpy as np
    arr = np.ascontiguousarray(arr, dtype=np.float32)
    t = new(L, list(arr.shape))
    C.memmove(t.contents.data, arr.ctypes.data, arr.nbytes)
    return t


def _to_np(L, t):
    import numpy as np
    assert t, "op returned NULL"
    shape = [t.contents.shape[i] for i in range(t.contents.ndim)]
    out = np.empty(shape, dtype=np.float32)
    C.memmove(out.ctypes.data, t.contents.data, out.nbytes)
    return out


def test_cpu_ops_match_numpy_on_random_shapes(lib):
    """Every CPU op of the C ABI against numpy, over random 1-d / 2-d / 3-d shapes."""
    import numpy as np
    L = lib
    rng = np.random.default_rng(17)
    gelu = lambda x: 0.5 * x * (1 + np.tanh(0.7978845608 * (x + 0.044715 * x ** 3)))
    unary = {"tensor_neg": np.negative, "tensor_abs": np.abs, "tensor_exp": np.exp,
             "tensor_relu": lambda x: np.maximum(x, 0), "tensor_sigmoid": lambda x: 1 / (1 + np.exp(-x)),
             "tensor_tanh": np.tanh, "tensor_gelu": gelu, "tensor_silu": lambda x: x / (1 + np.exp(-x)),
             "tensor_sqrt": lambda x: np.sqrt(np.abs(x)), "tensor_log": lambda x: np.log(np.abs(x) + 1)}
    binary = {"tensor_add": np.add, "tensor_sub": np.subtract, "tensor_mul": np.multiply}
    for trial in range(12):
        shape = [int(d) for d in rng.integers(1, 9, size=int(rng.integers(1, 4)))]
        a, b = rng.standard_normal(shape).astype(np.float32), rng.standard_normal(shape).astype(np.float32)
        ta, tb = _from_np(L, a), _from_np(L, b)
        for name, fn in unary.items():
            src = a
            if name == "tensor_sqrt":
                src = np.abs(a)
            elif name == "tensor_log":
                src = np.abs(a) + 1
            t = _from_np(L, src)
            want = fn(a) if name not in ("tensor_sqrt", "tensor_log") else (np.sqrt(src) if name == "tensor_sqrt" else np.log(src))
            np.testing.assert_allclose(_to_np(L, getattr(L, name)(t)), want, rtol=2e-5, atol=2e-6, err_msg=name)
            L.tensor_free(t)
        for name, fn in binary.items():
            np.testing.assert_allclose(_to_np(L, getattr(L, name)(ta, tb)), fn(a, b), rtol=1e-6, atol=1e-6, err_msg=name)
        np.testing.assert_allclose(_to_np(L, L.tensor_div(ta, _from_np(L, np.abs(b) + 0.5))), a / (np.abs(b) + 0.5), rtol=1e-5)
        np.testing.assert_allclose(_to_np(L, L.tensor_mul_scalar(ta, 2.5)), a * 2.5, rtol=1e-6)
        np.testing.assert_allclose(_to_np(L, L.tensor_add_scalar(ta, -1.25)), a - 1.25, rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(_to_np(L, L.tensor_pow_scalar(_from_np(L, np.abs(a) + 0.1), 1.5)), (np.abs(a) + 0.1) ** 1.5, rtol=1e-5)
        np.testing.assert_array_equal(_to_np(L, L.tensor_gt_scalar(ta, 0.1)), (a > 0.1).astype(np.float32))
        assert abs(L.tensor_sum(ta) - float(a.sum())) < 1e-3 and abs(L.tensor_mean(ta) - float(a.mean())) < 1e-4
        assert L.tensor_max(ta) == float(a.max()) and L.tensor_min(ta) == float(a.min())
        assert abs(L.tensor_get(L.tensor_mse_loss(ta, tb), 0) - float(((a - b) ** 2).mean())) < 1e-4
        assert abs(L.tensor_get(L.tensor_mae_loss(ta, tb), 0) - float(np.abs(a - b).mean())) < 1e-4
        np.testing.assert_allclose(_to_np(L, L.tensor_mse_loss_backward(ta, tb)), 2 * (a - b) / a.size, rtol=1e-5, atol=1e-7)
        # 2-d family
        m, k, n = (int(d) for d in rng.integers(1, 12, size=3))
        x, w, bias = rng.standard_normal((m, k)).astype(np.float32), rng.standard_normal((k, n)).astype(np.float32), rng.standard_normal(n).astype(np.float32)
        tx, tw = _from_np(L, x), _from_np(L, w)
        y = _to_np(L, L.tensor_matmul(tx, tw))
        np.testing.assert_allclose(y, x @ w, rtol=1e-4, atol=1e-5)
        np.testing.assert_allclose(_to_np(L, L.tensor_transpose(tx)), x.T)
        np.testing.assert_allclose(_to_np(L, L.tensor_add_broadcast(_from_np(L, y), _from_np(L, bias))), y + bias, rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(_to_np(L, L.tensor_add_broadcast_backward(tx)), x.sum(0), rtol=1e-5, atol=1e-5)
        e = np.exp(x - x.max(1, keepdims=True))
        np.testing.assert_allclose(_to_np(L, L.tensor_softmax(tx)), e / e.sum(1, keepdims=True), rtol=1e-5, atol=1e-7)
        labels = rng.integers(0, k, size=m)
        lse = np.log(e.sum(1)) + x.max(1)
        want = float((lse - x[np.arange(m), labels]).mean())
        tl = _from_np(L, labels.astype(np.float32))
        assert abs(L.tensor_get(L.tensor_cross_entropy_loss(tx, tl), 0) - want) < 1e-4
        p = e / e.sum(1, keepdims=True)
        p[np.arange(m), labels] -= 1
        np.testing.assert_allclose(_to_np(L, L.tensor_cross_entropy_loss_backward(tx, tl)), p / m, rtol=1e-4, atol=1e-6)
        nb = int(rng.integers(1, 4))
        xa, xb = rng.standard_normal((nb, m, k)).astype(np.float32), rng.standard_normal((nb, k, n)).astype(np.float32)
        np.testing.assert_allclose(_to_np(L, L.tensor_bmm(_from_np(L, xa), _from_np(L, xb))), xa @ xb, rtol=1e-4, atol=1e-5)
        va, vb = rng.standard_normal(k).astype(np.float32), rng.standard_normal(k).astype(np.float32)
        assert abs(L.tensor_dot(_from_np(L, va), _from_np(L, vb)) - float(va @ vb)) < 1e-4


@pytest.mark.gpu
def test_gpu_ops_match_cpu_ops(lib):
    import random
    L = lib
    L.pool_init()
    rnd = random.Random(3)

    def rand(shape):
        n = 1
        for s in shape:
            n *= s
        return new(L, shape, [rnd.uniform(-1, 1) for _ in range(n)])

    def close(gpu_t, cpu_t, tol):
        L.tensor_to_cpu(gpu_t)
        for x, y in zip(values(L, gpu_t), values(L, cpu_t)):
            assert abs(x - y) <= tol * (1 + abs(y)), (x, y)

    a, b = rand([33, 20]), rand([33, 20])
    ga, gb = L.tensor_to_cuda(L.tensor_copy(a)), L.tensor_to_cuda(L.tensor_copy(b))
    assert ga.contents.device == 1 and not ga.contents.data and ga.contents.cuda_data
    rt = L.tensor_to_cpu(L.tensor_to_cuda(L.tensor_copy(a)))
    assert values(L, rt) == values(L, a)                         # H2D / D2H round trip
    close(L.tensor_add_cuda(ga, gb), L.tensor_add(a, b), 1e-6)
    close(L.tensor_mul_cuda(ga, gb), L.tensor_mul(a, b), 1e-6)
    close(L.tensor_gelu_cuda(ga), L.tensor_gelu(a), 1e-5)
    close(L.tensor_softmax_cuda(ga), L.tensor_softmax(a), 1e-5)
    assert abs(L.tensor_sum_cuda(ga) - L.tensor_sum(a)) < 1e-3
    assert L.tensor_max_cuda(ga) == L.tensor_max(a)
    w = rand([20, 17])
    gw = L.tensor_to_cuda(L.tensor_copy(w))
    close(L.tensor_matmul_cuda(ga, gw), L.tensor_matmul(a, w), 1e-3)      # test_cuda.lua tolerance
    close(L.tensor_transpose_cuda(ga), L.tensor_transpose(a), 0)
    bias = rand([20])
    gbias = L.tensor_to_cuda(L.tensor_copy(bias))
    close(L.tensor_add_broadcast_cuda(ga, gbias), L.tensor_add_broadcast(a, bias), 1e-6)
    close(L.tensor_add_broadcast_backward_cuda(ga), L.tensor_add_broadcast_backward(a), 1e-4)
    close(L.tensor_fused_gelu_bias_cuda(ga, gbias), L.tensor_gelu(L.tensor_add_broadcast(a, bias)), 1e-5)
    ones, zeros = new(L, [20], [1] * 20), new(L, [20], [0] * 20)
    ln = L.tensor_fused_layernorm_cuda(ga, L.tensor_to_cuda(ones), L.tensor_to_cuda(zeros), 1e-5)
    L.tensor_to_cpu(ln)
    row = values(L, ln)[:20]
    assert abs(sum(row)) < 1e-4 and abs(sum(v * v for v in row) / 20 - 1) < 1e-2
    labels = new(L, [33], [rnd.randrange(20) for _ in range(33)])
    glabels = L.tensor_to_cuda(L.tensor_copy(labels))
    close(L.tensor_cross_entropy_loss_cuda(ga, glabels), L.tensor_cross_entropy_loss(a, labels), 1e-5)
    close(L.tensor_cross_entropy_loss_backward_cuda(ga, glabels), L.tensor_cross_entropy_loss_backward(a, labels), 1e-5)
    close(L.tensor_mse_loss_cuda(ga, gb), L.tensor_mse_loss(a, b), 1e-5)
    close(L.tensor_mse_loss_backward_cuda(ga, gb), L.tensor_mse_loss_backward(a, b), 1e-6)
    assert L.tensor_has_inf_nan_cuda(ga) == 0
    assert L.cuda_memory_allocated() > 0
    # adam: one step against the reference recurrence
    p, g = rand([50]), rand([50])
    gp, gg = L.tensor_to_cuda(L.tensor_copy(p)), L.tensor_to_cuda(L.tensor_copy(g))
    gm, gv = L.tensor_to_cuda(new(L, [50])), L.tensor_to_cuda(new(L, [50]))
    L.tensor_fused_adam_cuda(gp, gg, gm, gv, 0.01, 0.9, 0.999, 1e-8, 0.1, 0.001, 0.1)
    L.tensor_to_cpu(gp)
    for x, p0, g0 in zip(values(L, gp), values(L, p), values(L, g)):
        m1, v1 = 0.1 * g0, 0.001 * g0 * g0
        ref = p0 * (1 - 0.01 * 0.1) - 0.01 * (m1 / 0.1) / (math.sqrt(v1 / 0.001) + 1e-8)
        assert abs(x - ref) < 1e-5
    # flash attention (head_dim 64 -> tensor-core flash kernel) against a CPU softmax(QK^T)V
    BH, S, D = 2, 128, 64
    q, k, v = rand([BH, S, D]), rand([BH, S, D]), rand([BH, S, D])
    out = L.tensor_flash_attention_cuda(L.tensor_to_cuda(L.tensor_copy(q)), L.tensor_to_cuda(L.tensor_copy(k)),
                                        L.tensor_to_cuda(L.tensor_copy(v)), BH, S, D, 1)
    L.tensor_to_cpu(out)
    qv, kv, vv, ov = values(L, q), values(L, k), values(L, v), values(L, out)
    for (bh, i) in [(0, 0), (1, 5), (1, 127)]:
        sc = [sum(qv[(bh * S + i) * D + d] * kv[(bh * S + j) * D + d] for d in range(D)) / 8.0 for j in range(i + 1)]
        mx = max(sc)
        pr = [math.exp(s - mx) for s in sc]
        z = sum(pr)
        for d in (0, 31, 63):
            ref = sum(pr[j] / z * vv[(bh * S + j) * D + d] for j in range(i + 1))
            assert abs(ov[(bh * S + i) * D + d] - ref) < 2e-2
    L.pool_clear()
