"""Roofline of the fused all-reduce + AdamW kernels against the NVLink bound and against NCCL.

    python -m torch.distributed.run --nproc-per-node N -m luatorch_b200.tools.comm_benchmark

For each bucket size it times (CUDA events, max over ranks, after warm-up)
  fused-sharded     one launch: reduce-scatter over peer memory + shard AdamW + bf16 parameter
                    all-gather by peer stores
  fused-replicated  one launch: every rank reduces the whole bucket and updates its replica
  nccl + adamw      ncclAllReduce on the bf16 gradients, then the flat AdamW launch
and reports the achieved fraction of the roofline: the slower of (bytes that must ENTER a GPU
over NVLink / 770 GB/s per direction, the measured peer-copy rate of this machine class) and
(local HBM traffic of the AdamW update / measured copy bandwidth).

It then times the all-gather fused into the GEMM (`gather_matmul`: weight row shards pulled
over NVLink by the kernel that multiplies them) against the unfused pair (process-group
all_gather, then the same GEMM); roofline = the slower of FLOPs / measured bf16 GEMM peak and
remote shard bytes / 770 GB/s.
"""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
NVLINK_NOMINAL_BPS = 900e9     # NVLink 5: per direction per GPU


def measure_peer_copy(buf, rank, world, nbytes=256 << 20, iters=10):
    """Bytes per second one GPU pulls from ONE peer with this package's copy kernel (every rank
    reads its right-hand neighbour at the same time): the measured link rate the rooflines
    below are quoted against, next to the nominal 900 GB/s."""
    from luatorch_b200 import _backend as B
    from luatorch_b200.distributed import comm
    C = B.ext()
    nbytes = min(nbytes, buf.nbytes)
    status = comm.status_buffer()
    best = 0.0
    for root in range(min(world, 2)):
        def fn():
            C.peer_broadcast(buf.ptrs, buf.signal_ptrs, rank, world, root, 0, nbytes, 0, status)
        for _ in range(2):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        best = max(best, nbytes / (float(t.item()) * 1e-3))
    return best


def main():
    from luatorch_b200 import _backend as B
    from luatorch_b200.distributed import comm
    comm.init()
    rank, world = comm.rank(), comm.world_size()
    C = B.ext()
    hbm = 6.65e12
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        hbm = json.load(open(p))["hbm_gbs"] * 1e9
    sizes_mb = [1, 8, 32, 128, 311]
    n_max = max(sizes_mb) * 1024 * 1024 // 2
    grad_buf = comm.SymmetricBuffer(n_max * 2)
    shadow_buf = comm.SymmetricBuffer(n_max * 2)
    master = torch.randn(n_max, device="cuda")
    m = torch.zeros(n_max, device="cuda")
    v = torch.zeros(n_max, device="cuda")
    grad = grad_buf.typed(torch.bfloat16)[:n_max]
    shadow = shadow_buf.typed(torch.bfloat16)[:n_max]
    grad.copy_(torch.randn(n_max, device="cuda") * 0.01)
    seg_end = torch.tensor([n_max], device="cuda", dtype=torch.int64)
    seg_wd = torch.tensor([0.1], device="cuda")
    status = comm.status_buffer()
    blocks = int(os.environ.get("LT_COMM_BLOCKS", "0"))   # 0 = the kernel's default
    grad_mc = grad_buf.multicast_ptr + comm.SIGNAL_PAD_BYTES if grad_buf.multicast_ptr else 0
    shadow_mc = shadow_buf.multicast_ptr + comm.SIGNAL_PAD_BYTES if shadow_buf.multicast_ptr else 0

    def timed(fn, iters=10, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # with every rank reading from one root, the root's outgoing link carries world - 1 streams:
    # a reader's share is the per-direction link rate divided by the readers
    copy_bps = measure_peer_copy(grad_buf, rank, world) * max(1, world - 1)
    NVLINK_BPS = copy_bps
    if rank == 0:
        print("world %d; peer copy measured %.0f GB/s out of one GPU (nominal %.0f); HBM %.0f GB/s; multicast %s"
              % (world, copy_bps / 1e9, NVLINK_NOMINAL_BPS / 1e9, hbm / 1e9, "yes" if grad_mc else "no"))
    for mb in sizes_mb:
        n = mb * 1024 * 1024 // 2 // (8 * world) * (8 * world)
        nbytes = n * 2

        def fused(mode, nvls=False):
            C.allreduce_adamw(grad_buf.ptrs, grad_buf.signal_ptrs, rank, world, 0, n, master, shadow_buf.ptrs, m, v,
                              seg_end, seg_wd, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.05, 1.0 / world, 0, mode,
                              blocks, status, -1, 0, 0.0, False, grad_mc if nvls else 0,
                              shadow_mc if nvls else 0, None, None)

        def nccl_path():
            g = grad[:n]
            dist.all_reduce(g)
            C.adamw_flat(master[:n], shadow[:n], g, m[:n], v[:n], seg_end, seg_wd, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.05,
                         1.0 / world, None)

        rows = []
        cases = [
            # bytes ENTERING a GPU over NVLink: a two-shot all-reduce brings in (W-1)/W of the
            # bucket as read responses of the reduce-scatter and another (W-1)/W as the peers'
            # all-gather stores; the one-shot form reads the whole bucket from every peer
            ("fused-sharded", lambda: fused(1), 2.0 * nbytes * (world - 1) / world, n / world * 26.0 + nbytes / world * 2),
            ("fused-replicated", lambda: fused(0), nbytes * (world - 1), n * 26.0 + nbytes),
            ("nccl + adamw", nccl_path, 2.0 * nbytes * (world - 1) / world, n * 28.0),
        ]
        if grad_mc:
            # in-switch reduction: a GPU receives its reduced slice once and every peer's
            # published slice once, and sends each of its gradient bytes once
            cases.insert(1, ("fused-sharded-nvls", lambda: fused(1, True), 1.0 * nbytes,
                             n / world * 26.0 + nbytes / world * 2))
        for name, fn, link_bytes, hbm_bytes in cases:
            ms = timed(fn)
            bound_s = max(link_bytes / NVLINK_BPS, hbm_bytes / hbm)
            bound_n = max(link_bytes / NVLINK_NOMINAL_BPS, hbm_bytes / hbm)
            rows.append((name, ms, bound_s * 1e3 / ms if ms > 0 else 0.0, bound_n * 1e3 / ms if ms > 0 else 0.0))
        comm.check_status()
        if rank == 0:
            print("bucket %4d MB (bf16 grads): " % mb + "  ".join(
                "%s %.3f ms (%.0f%% of measured-link roofline, %.0f%% of 900 GB/s)" % (a, b, 100 * c, 100 * d)
                for a, b, c, d in rows), flush=True)
    # ---- all-gather fused into the consuming GEMM
    peak = 1.59e15
    if os.path.exists(p):
        peak = json.load(open(p))["bf16_tflops"] * 1e12
    for (M, K, N) in [(8192, 768, 3072), (8192, 2048, 8192), (8192, 3072, 768), (8192, 768, 50264)]:
        if K % world:
            continue
        sw = comm.ShardedWeight(K, N)
        sw.weight.copy_((torch.randn(K, N, device="cuda") * 0.02).bfloat16())
        x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
        y = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        parts = torch.empty(K, N, device="cuda", dtype=torch.bfloat16)

        def fused_gemm():
            comm.gather_matmul(x, sw)

        def unfused():
            dist.all_gather_into_tensor(parts, sw.shard.contiguous())
            C.gemm(x, parts, y, M, N, K, K, N, N, False, True, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, False, None, 0, None, 0,
                   None, None, 0, 0)

        def local_only():
            C.gemm(x, parts, y, M, N, K, K, N, N, False, True, 1, 1, 0, 0, 0, 0, 0, 0, 1.0, False, None, 0, None, 0,
                   None, None, 0, 0)

        t_f, t_u, t_l = timed(fused_gemm), timed(unfused), timed(local_only)
        comm.check_status()
        bound = max(2.0 * M * N * K / peak, K * N * 2.0 * (world - 1) / world / NVLINK_BPS)
        if rank == 0:
            print("gather+GEMM [%d,%d]x[%d,%d]: fused %.3f ms (%.0f%% of roofline)  all_gather + GEMM %.3f ms  "
                  "GEMM alone %.3f ms" % (M, K, K, N, t_f, 100 * bound * 1e3 / t_f, t_u, t_l), flush=True)
        del sw
    dist.barrier()
    comm.destroy()


if __name__ == "__main__":
    main()
