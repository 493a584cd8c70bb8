"""CUDA-graph replay of a training step (luatorch_b200/cuda/graph.py): the replayed step must
train exactly like the eager one, with the step-dependent scalars (learning rate, Adam bias
corrections, dropout offset) read from device memory."""
import pytest
import torch

import luatorch_b200 as lf

pytestmark = pytest.mark.gpu
T, ag, nn = lf.Tensor, lf.autograd, lf.nn


@pytest.fixture(scope="module")
def C():
    from luatorch_b200 import _C
    return _C


def test_dropout_reads_offset_from_device(C):
    x = torch.randn(5000, device="cuda")
    dyn = torch.zeros(1, device="cuda", dtype=torch.int64)
    base = C.dropout(x, 0.3, 77, 1000)
    torch.testing.assert_close(C.dropout_dyn(x, 0.3, 77, 1000, dyn), base, rtol=0, atol=0)
    C.set_step_scalars(None, 0.0, 0.0, 0.0, dyn, 4321)
    assert int(dyn.item()) == 4321
    shifted = C.dropout_dyn(x, 0.3, 77, 1000, dyn)
    torch.testing.assert_close(shifted, C.dropout(x, 0.3, 77, 1000 + 4321), rtol=0, atol=0)
    assert not torch.equal(shifted, base)
    kept = (shifted != 0).float().mean().item()
    assert abs(kept - 0.7) < 0.03


@pytest.mark.parametrize("gdtype", [torch.float32, torch.bfloat16])
def test_optimizers_read_scalars_from_device(C, gdtype):
    n = 4096 + 8
    torch.manual_seed(3)
    p0 = torch.randn(n, device="cuda")
    g = (torch.randn(n, device="cuda") * 0.1).to(gdtype)
    seg_end = torch.tensor([2048, n], device="cuda", dtype=torch.int64)
    seg_wd = torch.tensor([0.1, 0.0], device="cuda")
    lr, bc1, bc2 = 3e-3, 1 - 0.9 ** 4, 1 - 0.95 ** 4
    dyn = torch.zeros(4, device="cuda")
    C.set_step_scalars(dyn, lr, bc1, bc2, None, 0)
    torch.testing.assert_close(dyn[:3].cpu(), torch.tensor([lr, bc1, bc2]))

    def run(use_dyn):
        p, m, v = p0.clone(), torch.full((n,), 0.01, device="cuda"), torch.full((n,), 0.002, device="cuda")
        sh = torch.zeros(n, device="cuda", dtype=torch.bfloat16)
        if use_dyn:   # by-value scalars deliberately wrong: the kernel must take the device ones
            C.adamw_flat_dyn(p, sh, g, m, v, seg_end, seg_wd, 1.0, 0.9, 0.95, 1e-8, 0.5, 0.5, 1.0, None, dyn)
        else:
            C.adamw_flat(p, sh, g, m, v, seg_end, seg_wd, lr, 0.9, 0.95, 1e-8, bc1, bc2, 1.0, None)
        return p, m, v, sh

    for a, b in zip(run(True), run(False)):
        torch.testing.assert_close(a, b, rtol=0, atol=0)

    def run_sgd(use_dyn):
        p, vel = p0.clone(), torch.zeros(n, device="cuda")
        if use_dyn:
            C.sgd_flat_dyn(p, None, g, vel, 1.0, 0.9, False, 1.0, dyn)
        else:
            C.sgd_flat(p, None, g, vel, lr, 0.9, False, 1.0)
        return p, vel

    for a, b in zip(run_sgd(True), run_sgd(False)):
        torch.testing.assert_close(a, b, rtol=0, atol=0)


def _mlp(seed, p_drop):
    lf.manual_seed(seed)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Dropout(p_drop), nn.Linear(256, 10))
    arena = lf.cuda.amp.autocast_bf16(model)
    opt = lf.optim.AdamW(model.parameters(), 1e-3, 0.9, 0.95, 1e-8, 0.05)
    g = torch.Generator().manual_seed(7)
    x = T.wrap(torch.rand(256, 784, generator=g).cuda())
    y = T.wrap(torch.randint(0, 10, (256,), generator=g).float().cuda())
    crit = nn.CrossEntropyLoss()

    def one_step():
        ag.zero_graph()
        arena.zero_grad()
        loss = crit(model(x), y)
        ag.backward(loss)
        opt.step()
        return loss

    return arena, opt, one_step, (x, y)


def test_graphed_step_trains_like_eager():
    warm, steps = 3, 12
    lr_at = lambda k: 1e-3 * (0.9 ** k)          # a schedule: lr changes every step
    arena_e, opt_e, step_e, _ = _mlp(41, 0.0)
    eager = []
    for k in range(warm + steps):
        opt_e.set_lr(lr_at(k))
        eager.append(step_e().item())

    arena_g, opt_g, step_g, inputs = _mlp(41, 0.0)
    # the warm-up steps inside GraphedStep are real steps: give them the first `warm` rates
    calls = {"n": 0}

    def step_with_schedule():
        if calls["n"] < warm:
            opt_g.set_lr(lr_at(calls["n"]))
        calls["n"] += 1
        return step_g()

    graphed = lf.cuda.GraphedStep(step_with_schedule, opt_g, inputs=inputs, warmup=warm)
    assert opt_g.t == warm
    got = []
    for k in range(warm, warm + steps):
        opt_g.set_lr(lr_at(k))
        got.append(graphed().item())
    assert opt_g.t == warm + steps == opt_e.t
    torch.testing.assert_close(torch.tensor(got), torch.tensor(eager[warm:]), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(arena_g.master, arena_e.master, rtol=1e-5, atol=1e-7)
    assert got[-1] < got[0]


def test_graphed_step_with_dropout_and_new_inputs():
    arena, opt, one_step, (x, y) = _mlp(43, 0.2)
    graphed = lf.cuda.GraphedStep(one_step, opt, inputs=(x, y), warmup=2)
    assert graphed._span > 0
    g = torch.Generator().manual_seed(9)
    xs = torch.rand(256, 784, generator=g).pin_memory()
    ys = torch.randint(0, 10, (256,), generator=g).float().pin_memory()
    off_before = lf._backend.rng_state()["offset"]
    losses = [graphed(xs, ys).item() for _ in range(40)]
    torch.testing.assert_close(x._t.cpu(), xs)
    assert lf._backend.rng_state()["offset"] >= off_before + 40 * graphed._span
    assert all(l == l for l in losses)
    assert losses[-1] < 0.7 * losses[0], losses[::8]
    # a frozen learning rate of zero leaves only the masks to differ between two replays
    opt.set_lr(0.0)
    a, b = graphed().item(), graphed().item()
    assert a != b


def _ddp_sgd(seed):
    lf.manual_seed(seed)
    model = nn.Sequential(nn.Linear(64, 128), nn.ReLU(), nn.Linear(128, 16))
    ddp = lf.distributed.DDP(model)
    opt = lf.optim.SGD(ddp.parameters(), 0.05, 0.9)
    ddp.attach(opt)
    g = torch.Generator().manual_seed(8)
    x = T.wrap(torch.rand(128, 64, generator=g).cuda())
    y = T.wrap(torch.randint(0, 16, (128,), generator=g).float().cuda())
    crit = nn.CrossEntropyLoss()

    def one_step():
        ag.zero_graph()
        ddp.zero_grad()
        loss = crit(ddp(x), y)
        ag.backward(loss)
        ddp.sync_gradients()
        opt.step()
        return loss

    return ddp, opt, one_step, (x, y)


def test_graphed_step_with_ddp_wrapper_and_sgd():
    # SGD is not fused into the gradient reduction, so at one rank the wrapper puts nothing on
    # its communication stream; the capture must not wait on that idle stream
    warm, steps = 2, 10
    ddp_e, opt_e, step_e, _ = _ddp_sgd(51)
    for k in range(warm + steps):
        opt_e.set_lr(0.05 / (1 + k))
        last_e = step_e().item()
    ddp_g, opt_g, step_g, inputs = _ddp_sgd(51)
    n = {"k": 0}

    def warm_step():
        if n["k"] < warm:
            opt_g.set_lr(0.05 / (1 + n["k"]))
        n["k"] += 1
        return step_g()

    graphed = lf.cuda.GraphedStep(warm_step, opt_g, inputs=inputs, warmup=warm)
    for k in range(warm, warm + steps):
        opt_g.set_lr(0.05 / (1 + k))
        last_g = graphed().item()
    assert abs(last_g - last_e) <= 1e-5 * max(1.0, abs(last_e)), (last_g, last_e)
    torch.testing.assert_close(ddp_g.arena.master, ddp_e.arena.master, rtol=1e-5, atol=1e-7)


@pytest.mark.gpu
def test_scalar_fetcher_reads_device_scalars_one_step_behind():
    """Every pushed device scalar reaches the host, in order, through pinned memory, and the
    value handed back by push() is the one queued `depth` calls earlier."""
    import luatorch_b200 as lf
    f = lf.cuda.ScalarFetcher(depth=1)
    src = torch.arange(16, device="cuda", dtype=torch.float32) * 0.5
    buf = torch.zeros(1, device="cuda")
    got = []
    for i in range(16):
        buf.copy_(src[i:i + 1])            # the same static buffer every time, as a graph's output
        v = f.push(lf.Tensor.wrap(buf))
        if v is not None:
            got.append(v)
    got += f.drain()
    assert got == [0.5 * i for i in range(16)]
