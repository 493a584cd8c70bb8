"""Multi-GPU checks of the peer-memory collectives and the fused all-reduce + AdamW kernels.

Each test launches one process per GPU (2 ranks) with torch.distributed.run on 127.0.0.1 and
compares against the process group's NCCL all_reduce plus the reference AdamW arithmetic.
The reference project has no distributed tests at all."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(body: str, nproc: int = 2, timeout: int = 240, multicast: bool = False, port: int = 29731):
    """Run `body` as `nproc` ranks, one per GPU.  NCCL's NVLS is always off; the symmetric
    buffers are bound to an NVLink multicast object only for the cases that test the
    multimem path (`multicast=True`)."""
    import tempfile
    fd, script = tempfile.mkstemp(suffix="_mg_case.py")
    os.close(fd)
    with open(script, "w") as f:
        f.write("import os, sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    if not multicast:
        env["TORCH_SYMM_MEM_DISABLE_MULTICAST"] = "1"
        env["LT_NVLS"] = "0"
    if nproc == 1:
        cmd = [sys.executable, script]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
               "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    assert r.returncode == 0, (r.stdout[-3000:], r.stderr[-3000:])
    assert "CASE_OK" in r.stdout, r.stdout[-3000:]
    return r.stdout


def test_peer_allreduce_and_broadcast():
    _run("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed import comm, nccl
    comm.init()
    r, w = comm.rank(), comm.world_size()
    buf = comm.SymmetricBuffer(1 << 22, required=True)
    assert buf.peer_mapped
    for dtype in (torch.float32, torch.bfloat16):
        torch.manual_seed(100 + r)
        x = torch.randn(100003, device="cuda").to(dtype)
        ref = x.float().clone()
        dist.all_reduce(ref); ref /= w
        comm.allreduce_mean_(x, buf)
        torch.cuda.synchronize()
        comm.check_status()
        torch.testing.assert_close(x.float(), ref, atol=2e-2 if dtype == torch.bfloat16 else 1e-5, rtol=1e-2)
    t = torch.full((5000,), float(r + 1), device="cuda")
    comm.broadcast_(t, 1, buf)
    torch.cuda.synchronize()
    assert torch.all(t == 2.0)
    a = lf.Tensor.wrap(torch.full((1000,), float(r), device="cuda"))
    nccl.allreduce(a)
    torch.cuda.synchronize()
    assert abs(a.get(0) - (w - 1) / 2) < 1e-6
    comm.check_status()
    dist.barrier()
    if r == 0: print("CASE_OK")
    comm.destroy()
    """)


_FUSED_CASE = """
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed import comm
    comm.init()
    r, w = comm.rank(), comm.world_size()
    NVLS = %(nvls)s
    def full_master(ddp):
        a = ddp.arena
        if a.state_shards is not None:
            ddp.gather_master(); m = a.master.clone(); ddp.release_master(); return m
        if ddp.mode == "sharded":
            ddp.gather_master()
        return a.master.clone()
    cases = [("sharded", True, "adamw"), ("sharded", False, "adamw"), ("replicated", False, "adamw"),
             ("nccl", False, "adamw"), ("sharded", True, "sgd"), ("replicated", False, "sgd"),
             ("sharded", True, "sgd_nesterov")]
    for mode, shard_state, okind in cases:
        lf.manual_seed(7)
        model = lf.nn.Sequential(lf.nn.Linear(64, 256), lf.nn.GELU(), lf.nn.LayerNorm(256), lf.nn.Linear(256, 32))
        ddp = lf.distributed.DDP(model, mode=mode, bucket_mb=0.02, shard_state=shard_state, nvls=NVLS)
        assert ddp.mode == mode, (ddp.mode, mode)
        assert ddp.nvls == (NVLS and mode == "sharded"), (ddp.nvls, NVLS, mode)
        assert (ddp.arena.state_shards is not None) == (mode == "sharded" and shard_state)
        a = ddp.arena
        if okind == "adamw":
            opt = lf.optim.AdamW(ddp.parameters(), 1e-2, 0.9, 0.95, 1e-8, 0.1, [model.layers[2].gamma])
            if a.state_shards is not None:
                assert opt.m_flat.numel() * w == a.total and a.master is None   # 1/world of the state
        else:
            opt = lf.optim.SGD(ddp.parameters(), 0.05, 0.9, okind == "sgd_nesterov")
        ddp.attach(opt)
        master0 = full_master(ddp)
        m_ref = torch.zeros_like(master0); v_ref = torch.zeros_like(master0)
        wd = torch.zeros_like(master0)
        if okind == "adamw":
            seg_end, seg_wd = opt.segments()
            prev = 0
            for e, d in zip(seg_end.tolist(), seg_wd.tolist()):
                wd[prev:e] = d; prev = e
        p_ref = master0.clone()
        crit = lf.nn.MSELoss()
        for step in range(1, 4):
            torch.manual_seed(1000 * step + r)
            x = lf.Tensor.wrap(torch.randn(32, 64, device="cuda"))
            y = lf.Tensor.wrap(torch.randn(32, 32, device="cuda"))
            lf.autograd.zero_graph(); ddp.zero_grad()
            loss = crit(ddp(x), y)
            lf.autograd.backward(loss)
            torch.cuda.synchronize()
            g = a.grad.float().clone()            # local gradient before the reduction
            dist.all_reduce(g); g /= w
            g = g.bfloat16().float() if mode == "nccl" else g
            ddp.sync_gradients(); opt.step()
            torch.cuda.synchronize()
            ddp.check()
            master = full_master(ddp)
            if okind == "adamw":
                bc1, bc2 = 1 - 0.9 ** step, 1 - 0.95 ** step
                p_ref = p_ref * (1 - 1e-2 * wd)
                m_ref = 0.9 * m_ref + 0.1 * g
                v_ref = 0.95 * v_ref + 0.05 * g * g
                p_ref = p_ref - 1e-2 * (m_ref / bc1) / ((v_ref / bc2).sqrt() + 1e-8)
            else:
                m_ref = 0.9 * m_ref + g
                p_ref = p_ref - 0.05 * ((0.9 * m_ref + g) if okind == "sgd_nesterov" else m_ref)
            # the forward of the next step reads the shadow: it must equal bf16(master) everywhere
            torch.testing.assert_close(a.shadow.float(), master.bfloat16().float(), atol=0, rtol=0)
            # parameters follow the reference recurrence driven by the averaged gradient
            err = (master - p_ref).abs().max().item()
            assert err < 2e-3, (mode, okind, step, err)
            p_ref = master.clone()                # follow the kernel's state for the next step
        # replicas identical across ranks
        chk = a.shadow.float().clone()
        dist.all_reduce(chk, op=dist.ReduceOp.MAX)
        assert torch.equal(chk, a.shadow.float()), mode
        dist.barrier()
    if r == 0: print("CASE_OK")
    comm.destroy()
"""


def test_fused_allreduce_optimizer_modes_match_reference_math():
    """AdamW and SGD-momentum bodies, sharded (state in 1/world of the memory or full length),
    replicated and process-group modes, plain peer loads and stores."""
    _run(_FUSED_CASE % {"nvls": "False"}, timeout=400)


def test_fused_allreduce_optimizer_nvls_multimem():
    """The same cases with the sharded kernel reading through multimem.ld_reduce and
    publishing through multimem.st (buffers bound to an NVLink multicast object)."""
    _run(_FUSED_CASE % {"nvls": "True"}, timeout=400, multicast=True)


def test_sharded_training_state_saves_and_resumes_bit_identically():
    """3 steps with memory-sharded optimizer state -> save_checkpoint -> fresh processes
    load_checkpoint -> the next 3 steps equal an uninterrupted 6-step run bit for bit."""
    import tempfile
    d = tempfile.mkdtemp()
    body = """
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed import comm
    comm.init()
    r, w = comm.rank(), comm.world_size()
    PHASE, PATH = %(phase)r, %(path)r
    def build():
        lf.manual_seed(11)
        model = lf.nn.Sequential(lf.nn.Linear(64, 256), lf.nn.GELU(), lf.nn.LayerNorm(256), lf.nn.Linear(256, 32))
        ddp = lf.distributed.DDP(model, mode="sharded", bucket_mb=0.02)
        opt = lf.optim.AdamW(ddp.parameters(), 1e-2, 0.9, 0.95, 1e-8, 0.1, [model.layers[2].gamma])
        ddp.attach(opt)
        sched = lf.optim.StepLR(opt, 2, 0.5)
        return model, ddp, opt, sched
    crit = lf.nn.MSELoss()
    def step(ddp, opt, sched, i):
        torch.manual_seed(1000 * i + r)
        x = lf.Tensor.wrap(torch.randn(32, 64, device="cuda"))
        y = lf.Tensor.wrap(torch.randn(32, 32, device="cuda"))
        lf.autograd.zero_graph(); ddp.zero_grad()
        loss = crit(ddp(x), y)
        lf.autograd.backward(loss)
        ddp.sync_gradients(); opt.step(); sched.step()
        torch.cuda.synchronize(); ddp.check()
    model, ddp, opt, sched = build()
    assert ddp.arena.state_shards is not None
    if PHASE == "first":
        for i in range(1, 4): step(ddp, opt, sched, i)
        ddp.save_checkpoint(PATH, opt, sched, None, step=3)
        for i in range(4, 7): step(ddp, opt, sched, i)          # the uninterrupted run goes on
        ddp.gather_master()
        if r == 0:
            torch.save({"master": ddp.arena.master.cpu(), "shadow": ddp.arena.shadow.cpu()}, PATH + ".expect")
        ddp.release_master()
        sd = opt.state_dict()
        if r == 0: torch.save(sd, PATH + ".expect_opt")
    else:
        meta = ddp.load_checkpoint(PATH, opt, sched, None)
        assert meta["step"] == 3 and opt.t == 3
        for i in range(4, 7): step(ddp, opt, sched, i)
        ddp.gather_master()
        exp = torch.load(PATH + ".expect")
        assert torch.equal(ddp.arena.master.cpu(), exp["master"]), "fp32 master differs after resume"
        assert torch.equal(ddp.arena.shadow.cpu(), exp["shadow"])
        ddp.release_master()
        sd, exp_sd = opt.state_dict(), torch.load(PATH + ".expect_opt")
        for k in ("m", "v"):
            for x_, y_ in zip(sd[k], exp_sd[k]):
                assert torch.equal(x_, y_), "moment %%s differs after resume" %% k
    dist.barrier()
    if r == 0: print("CASE_OK")
    comm.destroy()
    """
    path = os.path.join(d, "ckpt.bin")
    _run(body % {"phase": "first", "path": path})
    assert os.path.exists(path) and os.path.exists(path + ".opt.bin")
    _run(body % {"phase": "resume", "path": path}, port=29733)


def test_graph_replay_on_two_ranks_matches_eager():
    """The captured step (with the fused collectives numbering themselves on the device)
    replays on both ranks and trains exactly like the eager loop."""
    _run("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed import comm
    comm.init()
    r, w = comm.rank(), comm.world_size()
    results = {}
    for use_graph in (False, True):
        for mode, okind in (("replicated", "adam"), ("sharded", "sgd")):
            lf.manual_seed(5)
            model = lf.nn.Sequential(lf.nn.Linear(64, 128), lf.nn.ReLU(), lf.nn.Linear(128, 16))
            ddp = lf.distributed.DDP(model, mode=mode, bucket_mb=0.02)
            opt = lf.optim.Adam(ddp.parameters(), 1e-2) if okind == "adam" else lf.optim.SGD(ddp.parameters(), 0.05, 0.9)
            ddp.attach(opt)
            sched = lf.optim.StepLR(opt, 3, 0.5)
            crit = lf.nn.MSELoss()
            torch.manual_seed(50 + r)
            x = lf.Tensor.wrap(torch.randn(32, 64, device="cuda"))
            y = lf.Tensor.wrap(torch.randn(32, 16, device="cuda"))
            def one_step():
                lf.autograd.zero_graph(); ddp.zero_grad()
                loss = crit(ddp(x), y)
                lf.autograd.backward(loss)
                ddp.sync_gradients(); opt.step()
                return loss
            runner = lf.cuda.GraphedStep(one_step, opt, inputs=(x, y), warmup=2) if use_graph else None
            if not use_graph:
                for _ in range(2): one_step(); sched.step()      # same number of real steps as the warm-up
            else:
                for _ in range(2): sched.step()
            losses = []
            for i in range(8):
                torch.manual_seed(900 + 10 * i + r)
                xb, yb = torch.randn(32, 64, device="cuda"), torch.randn(32, 16, device="cuda")
                if runner is not None:
                    loss = runner(lf.Tensor.wrap(xb), lf.Tensor.wrap(yb))
                else:
                    x._t.copy_(xb); y._t.copy_(yb)
                    loss = one_step()
                sched.step()
                losses.append(loss.item())
            torch.cuda.synchronize(); ddp.check()
            results[(use_graph, mode)] = (losses, ddp.arena.shadow.float().clone())
            dist.barrier()
    for mode in ("replicated", "sharded"):
        le, se = results[(False, mode)]
        lg, sg = results[(True, mode)]
        assert max(abs(a - b) for a, b in zip(le, lg)) < 1e-4, (mode, le, lg)
        torch.testing.assert_close(sg, se, rtol=0, atol=1e-2)
        assert le[-1] == le[-1]
    if r == 0: print("CASE_OK")
    comm.destroy()
    """, timeout=400)


def test_c_abi_collectives_wait_for_default_stream_producers():
    """luatorch_nccl_allreduce / broadcast (one process drives both devices, as the reference's
    wrapper does) called right after asynchronous default-stream work that produces their
    buffers: the collective must see the finished values.  Also an unaligned float*."""
    _run("""
    import ctypes, torch
    assert torch.cuda.device_count() >= 2
    lib = ctypes.CDLL(os.path.join(%(root)r, "luatorch_b200", "lib", "libluatorch.so"))
    lib.luatorch_nccl_init.restype = ctypes.c_int
    lib.luatorch_nccl_allreduce.restype = ctypes.c_int
    lib.luatorch_nccl_allreduce.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_int]
    lib.luatorch_nccl_broadcast.restype = ctypes.c_int
    lib.luatorch_nccl_broadcast.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_int64, ctypes.c_int, ctypes.c_int]
    assert lib.luatorch_nccl_get_gpu_count() >= 2
    assert lib.luatorch_nccl_init(2) == 0
    n = 1 << 20
    bufs, big = [], []
    for d in range(2):
        with torch.cuda.device(d):
            bufs.append(torch.zeros(n + 8, device="cuda:%%d" %% d))
            big.append(torch.randn(4096, 4096, device="cuda:%%d" %% d))
    def table(ts):
        arr = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in ts])
        return arr
    for trial in range(3):
        for off in (0, 1):                            # 1: a float* that is 4 bytes off a 16-byte boundary
            views = [b[off:off + n] for b in bufs]
            for d in range(2):
                with torch.cuda.device(d):            # default stream: a long producer, then the fill
                    for _ in range(20):
                        big[d] = (big[d] @ big[d]).clamp_(-1, 1)
                    views[d].fill_(float(d + 1 + trial))
            assert lib.luatorch_nccl_allreduce(table(views), n, 2) == 0
            for d in range(2):
                got = views[d].cpu()
                assert torch.all(got == 1.5 + trial), (trial, off, d, got[:4])
    views = [b[:n] for b in bufs]
    for d in range(2):
        with torch.cuda.device(d):
            for _ in range(20):
                big[d] = (big[d] @ big[d]).clamp_(-1, 1)
            views[d].fill_(float(10 + d))
    assert lib.luatorch_nccl_broadcast(table(views), n, 1, 2) == 0
    assert torch.all(views[0].cpu() == 11.0) and torch.all(views[1].cpu() == 11.0)
    lib.luatorch_nccl_destroy()
    print("CASE_OK")
    """ % {"root": ROOT}, nproc=1)


def test_gather_matmul_fused_allgather_gemm():
    """Row shards of the weight live on the ranks; the GEMM gathers them itself."""
    _run("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed import comm
    comm.init()
    r, w = comm.rank(), comm.world_size()
    for (M, K, N, gelu) in [(1024, 768, 3072, True), (8192, 768, 768, False), (512, 2048, 1024, False)]:
        torch.manual_seed(5)                       # same full weight on every rank
        full = (torch.randn(K, N, device="cuda") * 0.05).bfloat16()
        bias = torch.randn(N, device="cuda").bfloat16()
        torch.manual_seed(100 + r)                 # own activations
        x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        sw = comm.ShardedWeight(K, N)
        for it in range(3):                        # repeated calls reuse pads and flags
            sw.weight.zero_()
            sw.shard.copy_(full[r * (K // w):(r + 1) * (K // w)])
            torch.cuda.synchronize(); dist.barrier()
            y = comm.gather_matmul(x, sw, bias, gelu)
            torch.cuda.synchronize()
            comm.check_status()
            assert torch.equal(sw.weight, full), "local copy incomplete after the gather"
            ref = x.float() @ full.float() + bias.float()
            if gelu:
                ref = 0.5 * ref * (1 + torch.tanh(0.7978845608 * (ref + 0.044715 * ref ** 3)))
            torch.testing.assert_close(y.float(), ref, atol=0.08, rtol=0.03)
            dist.barrier()
    from luatorch_b200 import _C
    assert _C.gemm_device_error() == 0
    if r == 0: print("CASE_OK")
    comm.destroy()
    """)


def test_rank_leaving_between_steps_is_seen_on_the_host_before_the_next_launch():
    """Two GPU ranks train with the fused kernels; rank 1 then stops between steps with nothing
    in flight.  Rank 0 learns of it from the heartbeat on the host and never launches the next
    collective (no device-side fault or hang is involved; NVLS is off, plain peer loads)."""
    _run("""
    import time, torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed import comm
    from luatorch_b200.distributed.elastic import Heartbeat, RankFailure, StepFailed, run_step_guarded
    comm.init()
    r, w = comm.rank(), comm.world_size()
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, r, w, interval_s=0.05, stale_after_s=0.8)
    lf.manual_seed(3)
    model = lf.nn.Sequential(lf.nn.Linear(64, 128), lf.nn.GELU(), lf.nn.Linear(128, 16))
    ddp = lf.distributed.DDP(model, mode="sharded", bucket_mb=0.02, nvls=False)
    assert not ddp.nvls and ddp.grad_buf.multicast_ptr == 0    # plain peer loads, no multicast binding
    opt = lf.optim.AdamW(ddp.parameters(), 1e-2)
    ddp.attach(opt)
    crit = lf.nn.MSELoss()
    x = lf.Tensor.wrap(torch.randn(32, 64, device="cuda"))
    y = lf.Tensor.wrap(torch.randn(32, 16, device="cuda"))
    launched = [0]
    def step():
        launched[0] += 1
        lf.autograd.zero_graph(); ddp.zero_grad()
        loss = crit(ddp(x), y)
        lf.autograd.backward(loss)
        ddp.sync_gradients(); opt.step()
        torch.cuda.synchronize()
        ddp.check()
    for s_ in range(2):                       # both ranks present
        run_step_guarded(step, s_, hb)
    dist.barrier()
    torch.cuda.synchronize()                  # nothing of this rank is in flight any more
    if r == 1:
        hb.stop()                             # the rank "leaves": its heartbeat stops
        store.wait(["lt_test_done"])          # stay alive (and silent) until rank 0 has noticed
    else:
        t0, failed = time.time(), None
        while time.time() - t0 < 15:
            try:
                run_step_guarded(lambda: None, 2, hb)   # the host check precedes every launch
            except StepFailed as e:
                failed = e
                break
            time.sleep(0.1)
        assert failed is not None and isinstance(failed.cause, RankFailure) and failed.cause.ranks == [1]
        assert launched[0] == 2               # no third step was launched
        store.set("lt_test_done", "1")
        print("CASE_OK")
    hb.stop()
    comm.destroy()
    """)
