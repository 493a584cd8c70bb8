"""Service layers on CPU: checkpoint byte format (golden bytes built by an independent packer
of the format the reference's io/checkpoint.lua writes), training-state sidecars, data
loading, tokenizer file format, logger CSV, config parsing, ONNX export, parameter arena and
optimizer equivalence."""
import io
import json
import os
import struct

import pytest
import torch

import luatorch_b200 as lf

T, ag, nn = lf.Tensor, lf.autograd, lf.nn


def golden_checkpoint(params):
    """Independent packer: int32 n; per param int32 ndim, int32 dtype(0), int64 dims, float32 data."""
    out = bytearray(struct.pack("<i", len(params)))
    for shape, vals in params:
        out += struct.pack("<i", len(shape)) + struct.pack("<i", 0)
        for d in shape:
            out += struct.pack("<q", d)
        out += struct.pack("<%df" % len(vals), *vals)
    return bytes(out)


def test_checkpoint_bytes_are_the_reference_format(tmp_path):
    lf.manual_seed(3)
    model = nn.Sequential(nn.Linear(2, 3), nn.Tanh(), nn.Linear(3, 1, False))
    path = str(tmp_path / "m.bin")
    lf.io.checkpoint.save(model, path)
    expect = golden_checkpoint([(p.shape, p._t.reshape(-1).tolist()) for p in model.parameters()])
    assert open(path, "rb").read() == expect
    assert len(expect) == 4 + (8 + 16 + 24) + (8 + 8 + 12) + (8 + 16 + 12)
    # a file written by the independent packer loads, and saving again is byte-identical
    gold = golden_checkpoint([([2, 3], [1, 2, 3, 4, 5, 6]), ([3], [7, 8, 9]), ([3, 1], [10, 11, 12])])
    p2 = str(tmp_path / "g.bin")
    open(p2, "wb").write(gold)
    lf.io.checkpoint.load(model, p2)
    assert model.layers[0].weight.tolist() == [[1, 2, 3], [4, 5, 6]] and model.layers[2].weight.get(2) == 12
    lf.io.checkpoint.save(model, path)
    assert open(path, "rb").read() == gold
    with pytest.raises(ValueError, match="parameter count mismatch"):
        lf.io.checkpoint.load(nn.Linear(2, 3), p2)
    with pytest.raises(ValueError, match="shape mismatch"):
        lf.io.checkpoint.load(nn.Sequential(nn.Linear(2, 4), nn.Linear(3, 1, False)), p2)
    open(p2, "wb").write(gold[:-5])
    with pytest.raises(IOError):
        lf.io.checkpoint.load(model, p2)


def test_gpt_checkpoint_layout_and_fused_views(tmp_path):
    lf.manual_seed(4)
    m = lf.models.GPT(37, 16, 2, 1, 8, 0.0, pos="learned")
    shapes = [p.shape for p in m.parameters()]
    E, V = 16, 37
    assert shapes == [[V, E], [8, E], [E], [E], [E, E], [E, E], [E, E], [E, E], [E], [E], [E],
                      [E, 4 * E], [4 * E], [4 * E, E], [E], [E], [E], [E, V]]
    path = str(tmp_path / "gpt.bin")
    lf.io.checkpoint.save(m, path)
    lf.manual_seed(5)
    m2 = lf.models.GPT(37, 16, 2, 1, 8, 0.0, pos="learned")
    lf.io.checkpoint.load(m2, path)
    x = T.wrap(torch.randint(0, V, (2, 8)).float())
    with ag.no_grad():
        torch.testing.assert_close(m2(x)._t, m(x)._t)
    # q/k/v are slices of one fused tensor and the head weight is a view of padded storage
    assert m2.blocks[0].attn.q_proj.weight._t.data_ptr() == m2.blocks[0].attn.qkv_weight._t.data_ptr()
    assert m2.head.weight_storage._t.shape[1] == 40


def test_training_state_sidecars_resume_exactly(tmp_path):
    def build():
        lf.manual_seed(6)
        model = nn.Sequential(nn.Linear(4, 8), nn.BatchNorm1d(8), nn.ReLU(), nn.Linear(8, 2))
        opt = lf.optim.AdamW(model.parameters(), 1e-2, 0.9, 0.95, 1e-8, 0.1)
        sched = lf.optim.WarmupScheduler(opt, 3, lf.optim.CosineAnnealing(opt, 10))
        return model, opt, sched

    g = torch.Generator().manual_seed(0)
    xs = [T.wrap(torch.randn(16, 4, generator=g)) for _ in range(6)]
    ys = [T.wrap(torch.randn(16, 2, generator=g)) for _ in range(6)]

    def step(model, opt, sched, i):
        ag.zero_graph(); model.zero_grad()
        loss = nn.MSELoss()(model(xs[i]), ys[i])
        ag.backward(loss); opt.step(); sched.step()
        return loss.item()

    model, opt, sched = build()
    for i in range(3):
        step(model, opt, sched, i)
    path = str(tmp_path / "run.bin")
    lf.io.checkpoint.save(model, path)
    lf.io.checkpoint.save_training_state(path, model, opt, sched, None, step=3)
    tail_a = [step(model, opt, sched, i) for i in range(3, 6)]
    model2, opt2, sched2 = build()
    lf.io.checkpoint.load(model2, path)
    meta = lf.io.checkpoint.load_training_state(path, model2, opt2, sched2)
    assert meta["step"] == 3 and opt2.t == 3
    tail_b = [step(model2, opt2, sched2, i) for i in range(3, 6)]
    assert tail_a == tail_b                       # bitwise identical continuation


def test_dataloader_tokenizer_dataset(tmp_path):
    lf.manual_seed(7)
    data = T.wrap(torch.arange(20, dtype=torch.float32).reshape(10, 2))
    targets = T.wrap(torch.arange(10, dtype=torch.float32))
    dl = lf.data.DataLoader(data, targets, 4, False)
    assert dl.num_batches() == 3 and str(dl) == "DataLoader(samples=10, batch_size=4, batches=3)"
    batches = list(dl.iter())
    assert [b[0].shape for b in batches] == [[4, 2], [4, 2], [2, 2]] and batches[2][1].tolist() == [8, 9]
    seen = sorted(int(v) for b in lf.data.DataLoader(data, targets, 3, True).iter() for v in b[1].tolist())
    assert seen == list(range(10))
    shard = [int(v) for b in lf.data.DataLoader(data, targets, 2, False, rank=1, world_size=2).iter() for v in b[1].tolist()]
    assert shard == [1, 3, 5, 7, 9]
    tok = lf.data.Tokenizer("hello world")
    assert tok.vocab_size == 8 and tok.encode("low") == [tok.char_to_id[ord(c)] for c in "low"]
    assert tok.decode(tok.encode("hello")) == "hello" and tok.decode_tensor(tok.encode_tensor("owl")) == "owl"
    p = str(tmp_path / "vocab.txt")
    tok.save(p)
    lines = open(p).read().split("\n")
    assert lines[0] == "8" and lines[1] == "0 32"            # id 0 is the space (byte 32)
    assert lf.data.Tokenizer.load(p).encode("hello") == tok.encode("hello")
    with pytest.raises(ValueError):
        tok.encode("xyz")
    txt = str(tmp_path / "c.txt")
    open(txt, "w").write("abcdefghij" * 10)
    ds = lf.data.TextDataset(txt, 5, "train", 0.9, verbose=False)
    assert ds.n_samples == 90 - 5 and ds.vocab_size == 10
    a, b = ds.get(2)
    assert a.tolist() == [2, 3, 4, 5, 6] and b.tolist() == [3, 4, 5, 6, 7]
    xb, yb = ds.get_batch(4)
    assert xb.shape == [4, 5] and torch.equal(xb._t[:, 1:], yb._t[:, :-1])
    assert lf.data.TextDataset(txt, 5, "val", 0.9, verbose=False).n_samples == 5


def test_logger_and_config(tmp_path, capsys):
    lg = lf.utils.Logger(2)
    lg.set_epoch(1)
    lg.log(1.0, 0.5, 0.01)
    lg.log(3.0, 0.7, 0.01)
    assert "step      2  epoch   1  loss 2.0000  acc 60.00%  lr 1.00e-02" in capsys.readouterr().out
    p = str(tmp_path / "log.csv")
    lg.save_csv(p)
    assert open(p).read().split("\n")[:2] == ["step,epoch,loss,accuracy,lr", "1,1,1.000000,0.500000,0.01000000"]
    cfg = lf.utils.Config({"lr": 0.1, "layers": 2})
    lua = str(tmp_path / "cfg.lua")
    open(lua, "w").write('-- settings\nreturn {\n  lr = 3e-4, -- rate\n  name = "gpt", use_amp = true,\n  ["top_k"] = 40,\n}\n')
    cfg.load(lua)
    assert cfg.get("lr") == 3e-4 and cfg.get("name") == "gpt" and cfg.get("use_amp") is True
    assert cfg.get("top_k") == 40 and cfg.get("layers") == 2 and cfg.get("missing", 7) == 7
    js = str(tmp_path / "cfg.json")
    open(js, "w").write(json.dumps({"layers": 6}))
    assert cfg.load(js).get("layers") == 6
    cfg.load(str(tmp_path / "nope.lua"))            # missing file keeps defaults
    evil = str(tmp_path / "evil.lua")
    open(evil, "w").write('os.execute("echo pwned")\nreturn { x = os.time() }')
    with pytest.raises(ValueError):
        lf.utils.Config().load(evil)                # config files are parsed, never executed


def test_onnx_export_real_graph(tmp_path):
    lf.manual_seed(8)
    m = lf.models.MLP([4, 8, 3])
    p = str(tmp_path / "m.onnx")
    lf.export.onnx.export(m, T.new([2, 4]), p)
    info = lf.export.onnx.inspect(p)
    assert lf.export.onnx.verify(p)
    assert info["ops"] == ["MatMul", "Add", "Relu", "MatMul", "Add", "Identity"]
    assert info["ir_version"] == 7 and info["opset"] == 13 and info["producer"] == "luatorch"
    assert len([n for n in info["initializers"] if n.startswith("param")]) == 4
    open(p, "wb").write(b"\x00garbage")
    assert not lf.export.onnx.verify(p)


def test_onnx_export_is_numerically_the_model(tmp_path):
    """The stored graph, evaluated with numpy, reproduces the model's forward."""
    import torch
    onnx, nn = lf.export.onnx, lf.nn
    lf.manual_seed(12)
    for pos in ("learned", "sinusoidal"):
        gpt = lf.models.GPT(50, 32, 4, 2, 16, 0.0, pos=pos)
        gpt.eval()
        x = T.wrap(torch.randint(0, 50, (2, 8), generator=torch.Generator().manual_seed(1)).float())
        p = str(tmp_path / ("gpt_%s.onnx" % pos))
        onnx.export(gpt, x, p)
        assert onnx.verify(p, gpt, x)
        g = onnx.load_graph(p)
        assert g["input"] == "input_1" and g["output"] == "output_1"
        assert any(op == "Softmax" and attrs.get("axis") == -1 for op, _, _, attrs in g["nodes"])
    seq = nn.Sequential(nn.Linear(6, 12), nn.GELU(), nn.LayerNorm(12), nn.Linear(12, 8), nn.BatchNorm1d(8),
                        nn.SiLU(), nn.Linear(8, 3), nn.Sigmoid(), nn.Dropout(0.5), nn.Tanh())
    x = T.wrap(torch.randn(16, 6, generator=torch.Generator().manual_seed(2)))
    for _ in range(3):
        seq(x)                                     # BatchNorm running statistics
    seq.eval()
    p = str(tmp_path / "seq.onnx")
    onnx.export(seq, x, p)
    assert onnx.verify(p, seq, x)
    # a different model must fail the numeric check against the same file
    lf.manual_seed(13)
    other = nn.Sequential(nn.Linear(6, 12), nn.GELU(), nn.LayerNorm(12), nn.Linear(12, 8), nn.BatchNorm1d(8),
                          nn.SiLU(), nn.Linear(8, 3), nn.Sigmoid(), nn.Dropout(0.5), nn.Tanh())
    other.eval()
    assert not onnx.verify(p, other, x)


def test_arena_flat_optimizer_matches_per_tensor_optimizer():
    def build():
        lf.manual_seed(9)
        return lf.models.GPT(29, 16, 2, 2, 8, 0.0, pos="learned")

    tok = torch.randint(0, 29, (2, 9), generator=torch.Generator().manual_seed(1))
    x, y = T.wrap(tok[:, :-1].float()), T.wrap(tok[:, 1:].reshape(-1).float())

    def run(model, opt, zero):
        out = []
        for _ in range(4):
            ag.zero_graph(); zero()
            loss = nn.CrossEntropyLoss()(model(x), y)
            ag.backward(loss); opt.step()
            out.append(loss.item())
        return out

    a = build()
    oa = lf.optim.AdamW(a.parameters(), 1e-2, 0.9, 0.95, 1e-8, 0.1, a.no_decay_params())
    la = run(a, oa, a.zero_grad)
    b = build()
    arena = lf.parallel.ParamArena(b.parameters(), device="cpu", compute_dtype=None, grad_dtype=torch.float32)
    ob = lf.optim.AdamW(b.parameters(), 1e-2, 0.9, 0.95, 1e-8, 0.1, b.no_decay_params())
    assert ob.arena is arena and arena.total % 2048 == 0
    lb = run(b, ob, arena.zero_grad)
    assert la == pytest.approx(lb, rel=1e-5)
    for p, q in zip(a.parameters(), b.parameters()):
        torch.testing.assert_close(p._t, q._t, atol=1e-6, rtol=1e-5)
    buckets = arena.buckets(4096)
    assert buckets[0]["end"] == arena.total and buckets[-1]["start"] == 0
    assert all(b1["start"] == b2["end"] for b1, b2 in zip(buckets, buckets[1:]))
    seg_end, seg_wd = ob.segments()
    assert int(seg_end[-1]) == arena.total and sorted(set(round(w, 6) for w in seg_wd.tolist())) == [0.0, 0.1]


def test_xor_latency_benchmark_tool(tmp_path, capsys):
    # examples/benchmark_pytorch.lua: per-step times, percentiles, predictions, CSV
    from luatorch_b200.tools import xor_benchmark as xb
    assert xb.percentile([5.0, 1.0, 3.0, 2.0, 4.0], 0.5) == 3.0
    assert xb.percentile([5.0, 1.0, 3.0, 2.0, 4.0], 0.99) == 5.0
    assert xb.percentile([7.0], 0.5) == 7.0
    csv = tmp_path / "xor.csv"
    ours, theirs = xb.main(["--steps", "400", "--csv", str(csv)])
    out = capsys.readouterr().out
    assert "median per step" in out and "predictions:" in out and "stock torch.nn" in out
    assert ours["steps"] == 400 and ours["final_loss"] < 0.05 and theirs["final_loss"] < 0.05
    assert ours["p50_ms"] <= ours["p95_ms"] <= ours["p99_ms"] <= ours["max_ms"]
    lines = csv.read_text().strip().splitlines()
    assert lines[0] == "step,time_ms,torch_time_ms" and len(lines) == 401


def test_reference_constructor_spelling():
    # every class of the reference is built with X.new(...) (e.g. lua/luatorch/optim/adam.lua:22,
    # lua/luatorch/data/dataloader.lua, lua/luatorch/distributed/ddp.lua)
    p = [lf.Tensor.from_list([1.0, 2.0], [2])]
    opt = lf.optim.Adam.new(p, 0.1)
    assert isinstance(opt, lf.optim.Adam) and opt.lr == 0.1
    assert isinstance(lf.optim.SGD.new(p, 0.1, 0.9), lf.optim.SGD)
    assert isinstance(lf.optim.AdamW.new(p), lf.optim.AdamW)
    assert isinstance(lf.optim.StepLR.new(opt, 2, 0.5), lf.optim.StepLR)
    assert isinstance(lf.optim.CosineAnnealing.new(opt, 10), lf.optim.CosineAnnealing)
    for cls in (lf.optim.WarmupScheduler, lf.data.DataLoader, lf.distributed.DDP, lf.utils.Logger,
                lf.utils.Config, lf.cuda.GradScaler, lf.models.GPT, lf.models.MLP, lf.nn.Linear):
        assert callable(getattr(cls, "new"))


def test_nvtx_ranges_and_comm_fields_in_the_logger(tmp_path, capsys):
    import json
    import torch
    import luatorch_b200 as lf
    nvtx = lf.utils.nvtx
    before = nvtx.pushed
    with nvtx.range("off"):
        pass
    assert nvtx.pushed == before                      # off by default: nothing is opened
    nvtx.enable(True)
    try:
        m = lf.nn.Sequential(lf.nn.Linear(4, 4))
        x, y = lf.Tensor.wrap(torch.randn(2, 4)), lf.Tensor.wrap(torch.randn(2, 4))
        lf.autograd.zero_graph()
        lf.autograd.backward(lf.nn.MSELoss()(m(x), y))
        assert nvtx.pushed == before + 1              # the backward pass is one range
    finally:
        nvtx.enable(False)
    path = str(tmp_path / "log.jsonl")
    lg = lf.utils.Logger(1, jsonl_path=path)
    lg.log_comm({"buckets_ms": [0.1, 0.25], "total_ms": 0.35, "overlap": 0.2857}, {"allocated_mb": 12.0})
    lg.log(1.5, None, 1e-3, tokens=100, step_ms=2.0)
    out = capsys.readouterr().out
    assert "comm 0.350 ms in 2 buckets (29% under backward)" in out and "tok/s 50000" in out
    recs = [json.loads(l) for l in open(path)]
    assert recs[0]["comm"]["buckets_ms"] == [0.1, 0.25] and recs[0]["comm"]["pool"]["allocated_mb"] == 12.0
    assert recs[1]["tokens_per_s"] == 50000.0


def test_scalar_fetcher_returns_values_one_call_behind():
    """CPU fallback of the one-step-behind loss reader: same order, nothing lost."""
    import luatorch_b200 as lf
    f = lf.cuda.ScalarFetcher(depth=2)
    got = [f.push(torch.tensor([float(i)])) for i in range(5)]
    assert got == [None, None, 0.0, 1.0, 2.0]
    assert f.drain() == [3.0, 4.0]
    assert f.drain() == []
    f0 = lf.cuda.ScalarFetcher(depth=0)
    assert f0.push(lf.Tensor.wrap(torch.tensor([7.5]))) == 7.5
