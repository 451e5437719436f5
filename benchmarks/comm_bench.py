"""Fused compute+collective kernels vs their NCCL + cuBLAS baselines, with roofline fractions.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 benchmarks/comm_bench.py

Each JSON line (rank 0): op, shape, fused ms, baseline ms (both device-timed with CUDA events, max over
ranks, L2 flushed before every iteration), and the fraction of the roofline
``max(FLOPs / measured GEMM peak, bytes over NVLink / 770 GB/s per direction)``.
"""

from __future__ import annotations

import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from titan_b200.utils.device import measured_peaks  # noqa: E402

LINK_GBS = 770.0


def main():
    only = sys.argv[sys.argv.index("--only") + 1] if "--only" in sys.argv else ""  # substring filter on op labels
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    from titan_b200.ops import _lib, fused_comm

    group = dist.group.WORLD
    peaks = measured_peaks()
    tf_peak = peaks["bf16_tflops"] if peaks else 1590.0
    tag = "of measured" if peaks else "of fallback"
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def timeit(fn, iters=10, warmup=3):
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        ts = []
        for _ in range(iters):
            flush.zero_()
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            t = torch.tensor([a.elapsed_time(b)], device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ts.append(float(t))
        ts.sort()
        return ts[len(ts) // 2]

    def emit(**kw):
        if rank == 0:
            print(json.dumps(kw), flush=True)

    def want(label):
        return only in label

    dt = torch.bfloat16
    # ---- sequence-parallel all-gather → GEMM (column-parallel), 70B-like: A_shard [S/tp, 8192]
    for label, m_total, K, N in [("sp_ag_gemm 70B qkv", 8192, 8192, 10240 // world if world <= 8 else 1280),
                                 ("sp_ag_gemm 70B w13", 8192, 8192, 57344 // world),
                                 ("sp_ag_gemm 8B w13", 8192, 4096, 28672 // world)]:
        if not want(label):
            continue
        N = max(256, N // 256 * 256)
        m_shard = m_total // world
        a = torch.randn(m_shard, K, device="cuda", dtype=dt)
        b = torch.randn(N, K, device="cuda", dtype=dt) * 0.02
        fused = timeit(lambda: fused_comm.all_gather_matmul(a, b, group))
        base = timeit(lambda: fused_comm.all_gather_matmul_baseline(a, b, group))
        flops = 2.0 * m_total * N * K
        link_bytes = (world - 1) * m_shard * K * 2
        roof_ms = max(flops / (tf_peak * 1e9), link_bytes / (LINK_GBS * 1e6))
        emit(op=label, world=world, M=m_total, N=N, K=K, fused_ms=fused, nccl_cublas_ms=base,
             speedup=base / fused, roofline_ms=roof_ms, frac_of_roofline=roof_ms / fused, peak=tag)

    # ---- FSDP weight gather fused into the first GEMM: x [8192, 4096] · gather(W_shard)ᵀ
    for label, M, K, N in [("fsdp_ag_gemm 8B qkv", 8192, 4096, 6144), ("fsdp_ag_gemm 8B w13", 8192, 4096, 28672)]:
        n_shard = N // world // 256 * 256
        if n_shard == 0 or not want(label):
            continue
        x = torch.randn(M, K, device="cuda", dtype=dt)
        w = torch.randn(n_shard, K, device="cuda", dtype=dt) * 0.02
        fused = timeit(lambda: fused_comm.all_gather_weight_matmul(x, w, group))

        def base_fn():
            full = torch.empty(world * n_shard, K, device="cuda", dtype=dt)
            dist.all_gather_into_tensor(full, w, group=group)
            return x @ full.t()

        base = timeit(base_fn)
        flops = 2.0 * M * n_shard * world * K
        link_bytes = (world - 1) * n_shard * K * 2
        roof_ms = max(flops / (tf_peak * 1e9), link_bytes / (LINK_GBS * 1e6))
        emit(op=label, world=world, M=M, N=n_shard * world, K=K, fused_ms=fused, nccl_cublas_ms=base,
             speedup=base / fused, roofline_ms=roof_ms, frac_of_roofline=roof_ms / fused, peak=tag)

    # ---- row-parallel GEMM → reduce-scatter: A [8192, K/tp], B [8192, K/tp]
    for label, M, N, Kfull in [("gemm_rs 70B wo", 8192, 8192, 8192), ("gemm_rs 70B w2", 8192, 8192, 28672)]:
        if not want(label):
            continue
        K = Kfull // world // 64 * 64
        a = torch.randn(M, K, device="cuda", dtype=dt)
        b = torch.randn(N, K, device="cuda", dtype=dt) * 0.02
        fused = timeit(lambda: fused_comm.matmul_reduce_scatter(a, b, group))
        base = timeit(lambda: fused_comm.matmul_reduce_scatter_baseline(a, b, group))
        flops = 2.0 * M * N * K
        link_bytes = (world - 1) * (M // world) * N * 2
        roof_ms = max(flops / (tf_peak * 1e9), link_bytes / (LINK_GBS * 1e6))
        emit(op=label, world=world, M=M, N=N, K=K, fused_ms=fused, nccl_cublas_ms=base, speedup=base / fused,
             roofline_ms=roof_ms, frac_of_roofline=roof_ms / fused, peak=tag)

    # ---- Ulysses: projection + head->sequence exchange, and exchange + output projection.
    # Llama-8B-like attention over a sequence split `world` ways (32 heads x 128, dim 4096, 8192 local tokens)
    from titan_b200.ops import ulysses_fused as uf

    for label, s_loc, dim, nq in [("ulysses_proj_a2a 8B wq", 8192, 4096, 4096),
                                  ("ulysses_a2a_proj 8B wo", 8192, 4096, 4096)]:
        if not want(label) or nq % (64 * world):
            continue
        w = torch.randn(nq, dim, device="cuda", dtype=dt) * 0.02 if "wq" in label else \
            torch.randn(dim, nq, device="cuda", dtype=dt) * 0.02
        if "wq" in label:
            x = torch.randn(s_loc, dim, device="cuda", dtype=dt)
            fused = timeit(lambda: uf._scatter(x, w, s_loc, group, False))
            base = timeit(lambda: uf.proj_all_to_all_baseline(x, w, s_loc, group))
        else:
            o = torch.randn(s_loc * world, nq // world, device="cuda", dtype=dt)
            fused = timeit(lambda: uf._gather(o, w, s_loc, group, False))
            base = timeit(lambda: uf.all_to_all_proj_baseline(o, w, s_loc, group))
        flops = 2.0 * s_loc * dim * nq
        link_bytes = (world - 1) * s_loc * (nq // world) * 2
        roof_ms = max(flops / (tf_peak * 1e9), link_bytes / (LINK_GBS * 1e6))
        emit(op=label, world=world, M=s_loc, N=nq if "wq" in label else dim, K=dim if "wq" in label else nq,
             fused_ms=fused, nccl_cublas_ms=base, speedup=base / fused, roofline_ms=roof_ms,
             frac_of_roofline=roof_ms / fused, peak=tag)

    # ---- gradient bucket: bf16 → fp32 reduce-scatter with scale (one Llama-8B layer = 218 M params)
    if want("castscale_reduce_scatter 8B layer"):
        n = 218_112_000 // (world * 8) * (world * 8)
        bucket = torch.randn(n, device="cuda").to(dt)
        fused = timeit(lambda: fused_comm.castscale_reduce_scatter(bucket, 1.0 / world, torch.float32, group))
        base = timeit(lambda: fused_comm.castscale_reduce_scatter_baseline(bucket, 1.0 / world, torch.float32, group))
        link_bytes = (world - 1) * (n // world) * 2
        roof_ms = link_bytes / (LINK_GBS * 1e6)
        emit(op="castscale_reduce_scatter 8B layer", world=world, numel=n, fused_ms=fused, nccl_ms=base,
             speedup=base / fused, roofline_ms=roof_ms, frac_of_roofline=roof_ms / fused,
             note="fused moves bf16 over the link and accumulates fp32; NCCL path casts to fp32 first")
    torch.cuda.synchronize()
    _lib.shared_status().raise_if_set("comm bench")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
