"""Model-level behaviour on the CPU path: the GPT and MLP of the reference
(lua/luatorch/models/gpt.lua, mlp.lua) - parameter order (the checkpoint ABI), the AdamW
no-decay set, logits shape, sampling, train / eval switches and the module protocol."""
import torch

import luatorch_b200 as lf


def _tiny_gpt(pos="learned", dropout=0.0):
    lf.manual_seed(0)
    return lf.models.GPT(50, 32, 4, 2, 16, dropout, pos=pos)


def test_gpt_parameter_order_and_no_decay_set():
    m = _tiny_gpt()
    ps = m.parameters()
    # token embedding, positions, per block (ln1, attn q/k/v/out(+bias), ln2, ffn1, ffn2), final ln, head
    assert tuple(ps[0]._t.shape) == (50, 32) and tuple(ps[1]._t.shape) == (16, 32)
    assert tuple(ps[-1]._t.shape) == (32, 50)                      # untied head [embed, vocab], no bias
    assert tuple(ps[-3]._t.shape) == (32,) and tuple(ps[-2]._t.shape) == (32,)   # final LayerNorm
    per_block = (len(ps) - 2 - 2 - 1) // 2
    assert per_block == 13
    block0 = [tuple(p._t.shape) for p in ps[2:2 + per_block]]
    assert block0 == [(32,), (32,), (32, 32), (32, 32), (32, 32), (32, 32), (32,), (32,), (32,),
                      (32, 128), (128,), (128, 32), (32,)]
    assert m.num_params() == sum(p._t.numel() for p in ps)
    nd = m.no_decay_params()
    # final LN (2) + per block: ln1 (2), ln2 (2), ffn1 / ffn2 / out_proj biases (3)
    assert len(nd) == 2 + 2 * 7
    assert all(p._t.dim() == 1 for p in nd)
    sinus = _tiny_gpt(pos="sinusoidal")
    assert len(sinus.parameters()) == len(ps) - 1                   # sinusoidal positions have no weight


def test_gpt_forward_shape_loss_decreases_and_modes():
    m = _tiny_gpt(dropout=0.1)
    lf.manual_seed(1)
    tok = torch.randint(0, 50, (2, 9))
    x = lf.Tensor.wrap(tok[:, :-1].float())
    y = lf.Tensor.wrap(tok[:, 1:].reshape(-1).float())
    opt = lf.optim.AdamW(m.parameters(), 3e-3, 0.9, 0.95, 1e-8, 0.1, m.no_decay_params())
    crit = lf.nn.CrossEntropyLoss()
    losses = []
    for _ in range(30):
        lf.autograd.zero_graph()
        for p in m.parameters():
            p.grad = None
        out = m.forward(x)
        assert tuple(out._t.shape) == (16, 50)                       # [batch * seq, vocab]
        loss = crit(out, y)
        lf.autograd.backward(loss)
        opt.step()
        losses.append(float(loss._t.reshape(-1)[0]))
    assert losses[-1] < 0.6 * losses[0]
    m.eval()
    a = m.forward(x)._t.clone()
    b = m.forward(x)._t.clone()
    assert torch.equal(a, b)                                         # dropout off in eval
    m.train()
    assert m.training and all(blk.training for blk in m.blocks)


def test_generate_crops_context_and_respects_top_k():
    m = _tiny_gpt()
    lf.manual_seed(5)
    prompt = lf.Tensor.wrap(torch.tensor([1.0, 2.0, 3.0]))
    out = m.generate(prompt, 30, 0.8, 5)                             # longer than max_seq_len 16
    toks = out._t.tolist()
    assert len(toks) == 33 and toks[:3] == [1.0, 2.0, 3.0]
    assert all(0 <= t < 50 and float(t).is_integer() for t in toks)
    assert m.training                                                # restored after sampling
    again = m.generate([1, 2, 3], 4, 1.0, 1)                         # top-1 = greedy: repeatable
    again2 = m.generate([1, 2, 3], 4, 1.0, 1)
    assert again._t.tolist() == again2._t.tolist()


def test_mlp_and_module_protocol():
    lf.manual_seed(2)
    mlp = lf.models.MLP([8, 16, 4])
    assert mlp.num_params() == 8 * 16 + 16 + 16 * 4 + 4
    assert str(mlp) == "MLP(8 -> 16 -> 4)"
    out = mlp(lf.Tensor.wrap(torch.randn(5, 8)))
    assert tuple(out._t.shape) == (5, 4)
    nn = lf.nn
    a, b = nn.Linear(4, 3), nn.Linear.new(4, 3)                      # nn.X(...) == nn.X.new(...)
    assert type(a) is type(b) and a.num_params() == b.num_params() == 15
    w, bias = a.parameters()
    assert tuple(w._t.shape) == (4, 3) and tuple(bias._t.shape) == (3,)   # weight stored [in, out]
    seq = nn.Sequential(nn.Linear(4, 4), nn.Tanh())
    seq.add(nn.Linear(4, 2))
    assert len(seq.parameters()) == 4 and seq.num_params() == 20 + 10
    seq.zero_grad()
    assert all(p.grad is None for p in seq.parameters())
    assert lf.version == "0.1.0"


def test_graphed_step_needs_a_gpu():
    import pytest
    if torch.cuda.is_available():
        pytest.skip("CPU-only check")
    with pytest.raises(RuntimeError):
        lf.cuda.GraphedStep(lambda: None, optimizer=None)
