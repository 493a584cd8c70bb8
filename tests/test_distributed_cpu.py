"""Host-side distributed logic with CPU ranks (gloo, world size 2, 127.0.0.1): bucketed
data-parallel training equals single-process training on the concatenated batch, and failure
detection works without any GPU fault (a rank that stops between steps is reported by the
heartbeat before the survivors enter another collective)."""
import os
import subprocess
import sys
import textwrap


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _spawn(body: str, nproc: int, port: int, timeout: int = 180):
    import tempfile
    fd, script = tempfile.mkstemp(suffix="_cpu_rank.py")
    os.close(fd)
    with open(script, "w") as f:
        f.write("import os, sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)


def test_two_cpu_ranks_match_single_process_training():
    r = _spawn("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    assert world == 2
    def build():
        lf.manual_seed(11)
        return lf.nn.Sequential(lf.nn.Linear(6, 16), lf.nn.Tanh(), lf.nn.LayerNorm(16), lf.nn.Linear(16, 3))
    g = torch.Generator().manual_seed(5)
    X = torch.randn(3, 8, 6, generator=g); Y = torch.randn(3, 8, 3, generator=g)
    ddp = lf.distributed.DDP(build(), device="cpu", bucket_mb=0.0001)
    assert len(ddp.buckets) >= 1
    opt = lf.optim.Adam(ddp.parameters(), 1e-2)
    ddp.attach(opt)
    for s in range(3):
        lf.autograd.zero_graph(); ddp.zero_grad()
        xs = lf.Tensor.wrap(X[s, rank * 4:(rank + 1) * 4].clone()); ys = lf.Tensor.wrap(Y[s, rank * 4:(rank + 1) * 4].clone())
        loss = lf.nn.MSELoss()(ddp(xs), ys)
        lf.autograd.backward(loss); ddp.sync_gradients(); opt.step()
    ref = build()
    ropt = lf.optim.Adam(ref.parameters(), 1e-2)
    for s in range(3):
        lf.autograd.zero_graph(); ref.zero_grad()
        loss = lf.nn.MSELoss()(ref(lf.Tensor.wrap(X[s].clone())), lf.Tensor.wrap(Y[s].clone()))
        lf.autograd.backward(loss); ropt.step()
    for p, q in zip(ddp.parameters(), ref.parameters()):
        torch.testing.assert_close(p._t, q._t, atol=1e-5, rtol=1e-4)
    t = lf.Tensor.wrap(torch.full((5,), float(rank)))
    lf.distributed.nccl.allreduce(t)
    assert t.tolist() == [0.5] * 5
    lf.distributed.nccl.broadcast(t, 1)
    dist.barrier()
    if rank == 0: print("CASE_OK")
    lf.distributed.destroy()
    """, 2, 29741)
    assert r.returncode == 0 and "CASE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])


def test_heartbeat_reports_a_rank_that_left_between_steps():
    r = _spawn("""
    import time, torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed.elastic import Heartbeat, RankFailure, StepFailed, run_step_guarded
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, stale_after_s=0.6)
    x = torch.ones(4)
    dist.all_reduce(x)                      # step 0: everybody is here
    hb.check()
    if rank == 2:
        hb.stop()                           # leaves between steps, nothing in flight
        print("RANK2_LEFT", flush=True)
        os._exit(0)
    t0 = time.time()
    failed = None
    while time.time() - t0 < 10:
        try:
            run_step_guarded(lambda: None, step=1, heartbeat=hb)   # host check precedes any collective
        except StepFailed as e:
            failed = e
            break
        time.sleep(0.1)
    assert failed is not None and isinstance(failed.cause, RankFailure) and failed.cause.ranks == [2]
    assert failed.step == 1
    print("DETECTED_BY_%d" % rank, flush=True)
    hb.stop()
    os._exit(0)
    """, 3, 29742, timeout=120)
    out = r.stdout
    assert "RANK2_LEFT" in out and "DETECTED_BY_0" in out and "DETECTED_BY_1" in out, (out[-2000:], r.stderr[-2000:])


def test_resume_with_a_different_world_size(tmp_path):
    import torch
    import luatorch_b200 as lf
    from luatorch_b200.distributed.elastic import resume

    def build():
        lf.manual_seed(21)
        m = lf.nn.Sequential(lf.nn.Linear(4, 8), lf.nn.ReLU(), lf.nn.Linear(8, 2))
        o = lf.optim.AdamW(m.parameters(), 1e-2)
        return m, o, lf.optim.StepLR(o, 2, 0.5), lf.cuda.amp.GradScaler(1024.0)

    m, o, s, sc = build()
    x, y = lf.Tensor.wrap(torch.randn(8, 4)), lf.Tensor.wrap(torch.randn(8, 2))
    for _ in range(3):
        lf.autograd.zero_graph(); m.zero_grad()
        lf.autograd.backward(lf.nn.MSELoss()(m(x), y)); o.step(); s.step()
    path = str(tmp_path / "ck.bin")
    lf.io.checkpoint.save(m, path)
    lf.io.checkpoint.save_training_state(path, m, o, s, sc, step=3)
    m2, o2, s2, sc2, meta = resume(build, path)
    assert meta["step"] == 3 and o2.t == 3 and s2.epoch == 3 and sc2.get_scale() == 1024.0
    torch.testing.assert_close(m2(x)._t, m(x)._t)
    for a, b in zip(o.m, o2.m):
        torch.testing.assert_close(a, b)


def test_state_shards_take_gather_and_optimizer_state_roundtrip_on_gloo_ranks():
    """The bookkeeping of memory-sharded optimizer state, on CPU ranks: each rank keeps slice
    r of every bucket, gather() reassembles the full arrays, an optimizer built on a sharded
    arena allocates 1/world of the moments and its state_dict / load_state_dict round-trip."""
    r = _spawn("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.parallel.arena import ParamArena, StateShards, bucket_align_for
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    assert world == 3 and bucket_align_for(3) == 6144 and bucket_align_for(8) == 2048
    lf.manual_seed(3)
    model = lf.nn.Sequential(lf.nn.Linear(40, 70), lf.nn.Tanh(), lf.nn.Linear(70, 9))
    arena = ParamArena(model.parameters(), device="cpu", compute_dtype=torch.bfloat16,
                       grad_dtype=torch.float32, bucket_align=bucket_align_for(world))
    buckets = arena.buckets(2048)
    assert all((b["end"] - b["start"]) % (8 * world) == 0 for b in buckets)
    full = arena.master.clone()
    shards = StateShards(buckets, rank, world)
    assert shards.numel * world == arena.total
    mine = shards.take(full)
    back = shards.gather(mine, arena.total)
    assert torch.equal(back, full)
    arena.shard_state(shards)
    assert arena.master is None and arena.master_shard.numel() == shards.numel
    w0 = model.layers[0].weight
    assert w0._t.dtype == torch.bfloat16          # values read from the bf16 shadow meanwhile
    opt = lf.optim.AdamW(model.parameters(), 1e-2)
    assert opt.arena is arena and opt.m_flat.numel() == shards.numel
    opt.m_flat.copy_(torch.arange(shards.numel, dtype=torch.float32) + 1000 * rank)
    opt.v_flat.fill_(float(rank + 1))
    opt.t = 5
    sd = opt.state_dict()                          # collective: full moments on every rank
    assert sum(t.numel() for t in sd["m"]) == sum(u.numel() for u in arena.units)
    opt2 = lf.optim.AdamW(model.parameters(), 1e-2)
    opt2.load_state_dict(sd)
    # arena padding between tensors is not part of a checkpoint; everything else is
    keep = torch.zeros(arena.total, dtype=torch.bool)
    for u, o in zip(arena.units, arena.offsets):
        keep[o:o + u.numel()] = True
    k = shards.take(keep)
    assert torch.equal(opt2.m_flat[k], opt.m_flat[k]) and torch.equal(opt2.v_flat[k], opt.v_flat[k])
    assert opt2.t == 5
    arena.materialize_master()
    assert torch.equal(arena.master, full) and w0._t.dtype == torch.float32
    arena.master[arena.offsets[0]] = 42.0
    arena.release_master(write_back=True)
    arena.materialize_master()
    assert arena.master[arena.offsets[0]].item() == 42.0
    try:
        opt.step(); raise SystemExit("step() on sharded state must refuse")
    except RuntimeError:
        pass
    dist.barrier()
    if rank == 0: print("CASE_OK")
    lf.distributed.destroy()
    """, 3, 29743)
    assert r.returncode == 0 and "CASE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])


def test_gradient_accumulation_with_no_sync_and_second_backward_guard():
    r = _spawn("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    lf.distributed.init()
    rank, world = lf.distributed.rank(), lf.distributed.world_size()
    def build():
        lf.manual_seed(11)
        return lf.nn.Sequential(lf.nn.Linear(6, 16), lf.nn.Tanh(), lf.nn.Linear(16, 3))
    g = torch.Generator().manual_seed(9)
    X = torch.randn(2, 8, 6, generator=g); Y = torch.randn(2, 8, 3, generator=g)   # 2 micro-batches
    ddp = lf.distributed.DDP(build(), device="cpu", bucket_mb=0.0001)
    opt = lf.optim.SGD(ddp.parameters(), 0.1, 0.0)
    ddp.attach(opt)
    crit = lf.nn.MSELoss()
    def micro(i):
        lf.autograd.zero_graph()
        xs = lf.Tensor.wrap(X[i, rank * 4:(rank + 1) * 4].clone()); ys = lf.Tensor.wrap(Y[i, rank * 4:(rank + 1) * 4].clone())
        lf.autograd.backward(crit(ddp(xs), ys))
    ddp.zero_grad()
    with ddp.no_sync():
        micro(0)                       # accumulates locally, nothing is reduced or applied
    micro(1)                           # reduces and applies the sum of both micro-batches
    ddp.sync_gradients(); opt.step()
    ref = build()
    ropt = lf.optim.SGD(ref.parameters(), 0.1, 0.0)
    lf.autograd.zero_graph(); ref.zero_grad()
    for i in range(2):
        lf.autograd.zero_graph()
        lf.autograd.backward(crit(ref(lf.Tensor.wrap(X[i].clone())), lf.Tensor.wrap(Y[i].clone())))
    ropt.step()
    for p, q in zip(ddp.parameters(), ref.parameters()):
        torch.testing.assert_close(p._t, q._t, atol=1e-5, rtol=1e-4)
    # a second backward without zero_grad() or no_sync() is refused instead of silently dropped
    try:
        micro(0)
        raise SystemExit("second backward must raise")
    except RuntimeError as e:
        assert "no_sync" in str(e)
    dist.barrier()
    if rank == 0: print("CASE_OK")
    lf.distributed.destroy()
    """, 2, 29744)
    assert r.returncode == 0 and "CASE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])


def test_collective_checkpoint_roundtrip_on_cpu_ranks(tmp_path):
    path = str(tmp_path / "ddp.bin")
    r = _spawn("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    lf.distributed.init()
    rank = lf.distributed.rank()
    PATH = %r
    def build():
        lf.manual_seed(4)
        m = lf.nn.Sequential(lf.nn.Linear(5, 12), lf.nn.ReLU(), lf.nn.Linear(12, 2))
        d = lf.distributed.DDP(m, device="cpu")
        o = lf.optim.AdamW(d.parameters(), 1e-2); d.attach(o)
        return m, d, o
    m, d, o = build()
    x, y = lf.Tensor.wrap(torch.randn(8, 5)), lf.Tensor.wrap(torch.randn(8, 2))
    for _ in range(2):
        lf.autograd.zero_graph(); d.zero_grad()
        lf.autograd.backward(lf.nn.MSELoss()(d(x), y)); d.sync_gradients(); o.step()
    d.save_checkpoint(PATH, o, None, None, step=2)
    m2, d2, o2 = build()
    meta = d2.load_checkpoint(PATH, o2)
    assert meta["step"] == 2 and o2.t == 2
    for p, q in zip(m.parameters(), m2.parameters()):
        assert torch.equal(p._t, q._t)
    for a, b in zip(o.m, o2.m):
        assert torch.equal(a, b)
    dist.barrier()
    if rank == 0: print("CASE_OK")
    lf.distributed.destroy()
    """ % path, 2, 29745)
    assert r.returncode == 0 and "CASE_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
