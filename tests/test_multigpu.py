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


def _run(body: str, nproc: int = 2, timeout: int = 240):
    import tempfile
    fd, script = tempfile.mkstemp(suffix="_mg_case.py")
    os.close(fd)
    with open(script, "w") as f:
        f.write("import os, sys\nsys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(body))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(nproc),
           "--master-addr", "127.0.0.1", "--master-port", "29731", script]
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


def test_fused_allreduce_adamw_modes_match_reference_math():
    _run("""
    import torch, torch.distributed as dist
    import luatorch_b200 as lf
    from luatorch_b200.distributed import comm
    comm.init()
    r, w = comm.rank(), comm.world_size()
    for mode in ("sharded", "replicated", "nccl"):
        lf.manual_seed(7)
        model = lf.nn.Sequential(lf.nn.Linear(64, 256), lf.nn.GELU(), lf.nn.LayerNorm(256), lf.nn.Linear(256, 32))
        ddp = lf.distributed.DDP(model, mode=mode, bucket_mb=0.02)
        assert ddp.mode == mode, (ddp.mode, mode)
        opt = lf.optim.AdamW(ddp.parameters(), 1e-2, 0.9, 0.95, 1e-8, 0.1, [model.layers[2].gamma])
        ddp.attach(opt)
        a = ddp.arena
        master0 = a.master.clone()
        m_ref = torch.zeros_like(master0); v_ref = torch.zeros_like(master0)
        seg_end, seg_wd = opt.segments()
        wd = torch.zeros_like(master0); prev = 0
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
            if mode == "sharded":
                ddp.gather_master()
            bc1, bc2 = 1 - 0.9 ** step, 1 - 0.95 ** step
            p_ref = p_ref * (1 - 1e-2 * wd)
            m_ref = 0.9 * m_ref + 0.1 * g
            v_ref = 0.95 * v_ref + 0.05 * g * g
            p_ref = p_ref - 1e-2 * (m_ref / bc1) / ((v_ref / bc2).sqrt() + 1e-8)
            # the forward of the next step reads the shadow: it must equal bf16(master) everywhere
            torch.testing.assert_close(a.shadow.float(), a.master.bfloat16().float(), atol=0, rtol=0)
            # parameters follow the reference recurrence driven by the averaged gradient
            # (tolerance: the next step's gradients are computed from bf16 weights that differ
            # by rounding between the two paths only through p itself)
            err = (a.master - p_ref).abs().max().item()
            assert err < 2e-3, (mode, step, err)
            p_ref = a.master.clone()              # follow the kernel's state for the next step
        # replicas identical across ranks
        chk = a.shadow.float().clone()
        dist.all_reduce(chk, op=dist.ReduceOp.MAX)
        assert torch.equal(chk, a.shadow.float()), mode
        dist.barrier()
    if r == 0: print("CASE_OK")
    comm.destroy()
    """)


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
    ddp = lf.distributed.DDP(model, mode="sharded", bucket_mb=0.02)
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
