"""Per-kernel timings against the library baseline and the measured roofline.

    python benchmarks/kernel_bench.py [--only gemm,rmsnorm,...] [--iters 20]

Each line is JSON: kernel, shape, our time, baseline (PyTorch / cuBLAS) time, achieved TFLOP/s or
GB/s, and the fraction of the measured peak (cuBLAS bf16 burst throughput / copy bandwidth from
MEASURED_PEAKS.json when present, else the stated fallback).  Timing: CUDA events on the launching
stream, 5 warm-up iterations, an L2 flush (write of a 256 MB buffer) before every timed iteration.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from titan_b200.utils.device import measured_peaks  # noqa: E402

_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device="cuda")
    _FLUSH.zero_()


def timeit(fn, iters=20, warmup=5):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush_l2()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    return times[len(times) // 2]  # median, ms


def peaks():
    p = measured_peaks()
    if p:
        return p["bf16_tflops"], p["hbm_gbs"], "of measured"
    return 1590.0, 6650.0, "of fallback"


def emit(**kw):
    print(json.dumps(kw), flush=True)


def timeit_interleaved(fns: dict, iters=20, warmup=3):
    """Median time of each callable, measured round-robin (A, B, C, A, B, C, ...) so that slow drifts of the GPU's
    clocks under its power cap hit every candidate alike; L2 flushed before every timed call."""
    for _ in range(warmup):
        for fn in fns.values():
            fn()
    torch.cuda.synchronize()
    times = {k: [] for k in fns}
    for _ in range(iters):
        for k, fn in fns.items():
            flush_l2()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            times[k].append(a.elapsed_time(b))
    return {k: sorted(v)[len(v) // 2] for k, v in times.items()}


GEMM_SHAPES = [  # (M, N, K, a_mn, b_mn, label): forward, input-gradient and weight-gradient products
    (8192, 4096, 4096, 0, 0, "llama8b wq/wo fwd"),
    (8192, 1024, 4096, 0, 0, "llama8b wk/wv fwd"),
    (8192, 6144, 4096, 0, 0, "llama8b qkv fwd (fused)"),
    (8192, 14336, 4096, 0, 0, "llama8b w1/w3 fwd"),
    (8192, 28672, 4096, 0, 0, "llama8b w13 fwd (fused)"),
    (8192, 4096, 14336, 0, 0, "llama8b w2 fwd"),
    (8192, 4096, 4096, 0, 1, "llama8b wq/wo dgrad"),
    (8192, 4096, 1024, 0, 1, "llama8b wk/wv dgrad"),
    (8192, 4096, 6144, 0, 1, "llama8b qkv dgrad (fused)"),
    (8192, 4096, 14336, 0, 1, "llama8b w1/w3 dgrad"),
    (8192, 4096, 28672, 0, 1, "llama8b w13 dgrad (fused)"),
    (8192, 14336, 4096, 0, 1, "llama8b w2 dgrad"),
    (4096, 4096, 8192, 1, 1, "llama8b wq/wo wgrad"),
    (1024, 4096, 8192, 1, 1, "llama8b wk/wv wgrad"),
    (6144, 4096, 8192, 1, 1, "llama8b qkv wgrad (fused)"),
    (14336, 4096, 8192, 1, 1, "llama8b w1/w3 wgrad"),
    (28672, 4096, 8192, 1, 1, "llama8b w13 wgrad (fused)"),
    (4096, 14336, 8192, 1, 1, "llama8b w2 wgrad"),
    (8192, 128256, 4096, 0, 0, "llama8b output fwd"),
    (8192, 4096, 128256, 0, 1, "llama8b output dgrad"),
    (128256, 4096, 8192, 1, 1, "llama8b output wgrad"),
    (8192, 5120, 8192, 0, 0, "llama70b-tp2 qkv fwd"),
    (8192, 8192, 4096, 0, 0, "llama70b-tp2 wo fwd"),
    (8192, 14336, 8192, 0, 0, "llama70b-tp2 w1/w3 fwd"),
    (8192, 8192, 14336, 0, 0, "llama70b-tp2 w2 fwd"),
    (8192, 8192, 14336, 0, 1, "llama70b-tp2 w1/w3 dgrad"),
    (14336, 8192, 8192, 1, 1, "llama70b-tp2 w1/w3 wgrad"),
    (8192, 14336, 8192, 1, 1, "llama70b-tp2 w2 wgrad"),
]


def bench_gemm(iters, shapes=None):
    from titan_b200.ops.gemm import gemm

    tf_peak, _, tag = peaks()
    for M, N, K, a_mn, b_mn, label in (shapes or GEMM_SHAPES):
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        t = timeit_interleaved({
            "ours": lambda: gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out),
            "cublas": lambda: torch.matmul(A, B, out=out),
            "single": lambda: gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out, policy="single"),
        }, iters)
        fl = 2.0 * M * N * K
        emit(kernel="gemm_tcgen05", label=label, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, ms=t["ours"],
             cublas_ms=t["cublas"], single_cta_ms=t["single"], tflops=fl / t["ours"] / 1e9,
             cublas_tflops=fl / t["cublas"] / 1e9, frac_of_peak=fl / t["ours"] / 1e9 / tf_peak, peak=tag,
             speedup_vs_cublas=t["cublas"] / t["ours"], timing="round-robin medians, L2 flushed before every call")
        del a, b, out


def bench_gemm_sustained(rounds=6, block_ms=250.0, shapes=None):
    """GEMM throughput under the power cap, the regime of a training step: each candidate runs back to back for
    ``block_ms`` (no L2 flush, no pauses), candidates alternate block by block for ``rounds`` rounds, and the
    medians of the block rates are reported.  A burst timing flatters whichever kernel runs on a cool chip."""
    from titan_b200.ops.gemm import gemm

    _, _, tag = peaks()
    p = measured_peaks()
    sustained_peak = p["bf16_tflops_sustained"] if p and "bf16_tflops_sustained" in p else 1400.0
    pick = shapes or [sh for sh in GEMM_SHAPES if "70b" not in sh[5]]
    for M, N, K, a_mn, b_mn, label in pick:
        a = torch.randn((K, M) if a_mn else (M, K), device="cuda", dtype=torch.bfloat16)
        b = torch.randn((K, N) if b_mn else (N, K), device="cuda", dtype=torch.bfloat16)
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        A = a.t() if a_mn else a
        B = b if b_mn else b.t()
        fns = {"ours": lambda: gemm(a, b, a_mn=bool(a_mn), b_mn=bool(b_mn), out=out),
               "cublas": lambda: torch.matmul(A, B, out=out)}
        fl = 2.0 * M * N * K
        reps = {}
        for k, fn in fns.items():
            for _ in range(3):
                fn()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            reps[k] = max(3, int(block_ms / max(e0.elapsed_time(e1), 1e-3)))
        rates = {k: [] for k in fns}
        for _ in range(rounds):
            for k, fn in fns.items():
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps[k]):
                    fn()
                e1.record()
                torch.cuda.synchronize()
                rates[k].append(fl * reps[k] / e0.elapsed_time(e1) / 1e9)
        med = {k: sorted(v)[len(v) // 2] for k, v in rates.items()}
        emit(kernel="gemm_tcgen05_sustained", label=label, M=M, N=N, K=K, a_mn=a_mn, b_mn=b_mn, tflops=med["ours"],
             cublas_tflops=med["cublas"], speedup_vs_cublas=med["ours"] / med["cublas"],
             frac_of_sustained_peak=med["ours"] / sustained_peak, peak="of measured (sustained cuBLAS bf16)",
             timing=f"{rounds} alternating blocks of {block_ms:.0f} ms per candidate, medians")
        del a, b, out


def bench_elementwise(iters):
    from titan_b200.ops.cross_entropy import cross_entropy_sum
    from titan_b200.ops.norm import rms_norm_bwd, rms_norm_fwd
    from titan_b200.ops.rope import rope_apply
    from titan_b200.ops.swiglu import swiglu
    from titan_b200.models.common import rope as rope_ref

    _, bw_peak, tag = peaks()
    rows, dim = 8192, 4096
    x = torch.randn(rows, dim, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(dim, device="cuda", dtype=torch.bfloat16)
    g = torch.randn_like(x)
    ours = timeit(lambda: rms_norm_fwd(x, w, 1e-5), iters)
    base = timeit(lambda: torch.nn.functional.rms_norm(x, (dim,), w, 1e-5), iters)
    byt = 2 * x.numel() * 2
    emit(kernel="rmsnorm_fwd", shape=[rows, dim], ms=ours, torch_ms=base, gbs=byt / ours / 1e6,
         frac_of_peak=byt / ours / 1e6 / bw_peak, peak=tag)
    _, rstd = rms_norm_fwd(x, w, 1e-5)
    ours = timeit(lambda: rms_norm_bwd(g, x, w, rstd), iters)
    byt = 3 * x.numel() * 2
    emit(kernel="rmsnorm_bwd", shape=[rows, dim], ms=ours, gbs=byt / ours / 1e6,
         frac_of_peak=byt / ours / 1e6 / bw_peak, peak=tag)

    q = torch.randn(1, 8192, 32, 128, device="cuda", dtype=torch.bfloat16)
    cache = rope_ref.precompute_freqs_cis(128, 8192, 500000.0).cuda()
    ours = timeit(lambda: rope_apply(q, cache), iters)
    base = timeit(lambda: rope_ref.apply_rotary_emb_single_complex(q, cache), iters)
    byt = 2 * q.numel() * 2
    emit(kernel="rope", shape=list(q.shape), ms=ours, torch_ms=base, gbs=byt / ours / 1e6,
         frac_of_peak=byt / ours / 1e6 / bw_peak, peak=tag)

    a = torch.randn(8192, 14336, device="cuda", dtype=torch.bfloat16)
    b = torch.randn_like(a)
    ours = timeit(lambda: swiglu(a, b), iters)
    base = timeit(lambda: torch.nn.functional.silu(a) * b, iters)
    byt = 3 * a.numel() * 2
    emit(kernel="swiglu_fwd", shape=list(a.shape), ms=ours, torch_ms=base, gbs=byt / ours / 1e6,
         frac_of_peak=byt / ours / 1e6 / bw_peak, peak=tag)

    T, V = 8192, 128256
    logits = torch.randn(T, V, device="cuda", dtype=torch.bfloat16)
    labels = torch.randint(0, V, (T,), device="cuda")
    ours = timeit(lambda: cross_entropy_sum(logits, labels), max(5, iters // 4))
    byt = logits.numel() * 2
    emit(kernel="cross_entropy_fwd", shape=[T, V], ms=ours, gbs=byt / ours / 1e6,
         frac_of_peak=byt / ours / 1e6 / bw_peak, peak=tag)
    del logits

    from titan_b200.optim.fused_adamw import adamw_multi_tensor

    n = 256 * 1024 * 1024
    p = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    gr = torch.randn(n, device="cuda", dtype=torch.bfloat16)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    ours = timeit(lambda: adamw_multi_tensor([p], [gr], [m], [v], lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,
                                             weight_decay=0.1, step=3), max(5, iters // 4))
    # library baseline: torch's fused AdamW wants one dtype for params and state, so it runs on bf16 state
    mb, vb, st = m.bfloat16(), v.bfloat16(), torch.tensor(3.0, device="cuda")
    base = timeit(lambda: torch._fused_adamw_([p], [gr], [mb], [vb], [], [st], lr=1e-3, beta1=0.9, beta2=0.95,
                                              weight_decay=0.1, eps=1e-8, amsgrad=False, maximize=False),
                  max(5, iters // 4))
    byt = n * (2 + 2 + 4 + 4 + 2 + 4 + 4)
    emit(kernel="adamw_multi", numel=n, ms=ours, torch_ms=base, gbs=byt / ours / 1e6,
         frac_of_peak=byt / ours / 1e6 / bw_peak, peak=tag)


def bench_indexer(iters):
    """Lightning-indexer scoring + top-k (64 heads of dim 128): the kernel that keeps the query block in shared
    memory against the generic tiled GEMM's indexer mode, at a cached and at a long key stream."""
    from titan_b200.ops import dsa

    tf_peak, _, tag = peaks()
    for S, T in ((4096, 16384), (8192, 32768)):
        q = torch.randn(1, S, 64, 128, device="cuda", dtype=torch.bfloat16)
        k = torch.randn(1, T, 1, 128, device="cuda", dtype=torch.bfloat16)
        w = torch.rand(1, S, 64, device="cuda")
        off = T - S
        rec = dict(kernel="indexer_scores_topk", S=S, T=T, heads=64, topk=2048)
        for name, flag in (("resident", True), ("tiled", False)):
            dsa.RESIDENT_SCORING = flag
            rec[f"{name}_ms"] = timeit(lambda: dsa.lightning_indexer_topk(q, w, k, 2048, off), iters)
        dsa.RESIDENT_SCORING = True
        visible = S * (off + (S + 1) / 2)                     # causal (query, key) pairs
        fl = 2.0 * visible * 64 * 128
        rec["resident_tflops_causal"] = fl / rec["resident_ms"] / 1e9
        rec["frac_of_peak"] = rec["resident_tflops_causal"] / tf_peak
        rec["peak"] = tag
        emit(**rec)
        del q, k, w


def bench_moe(iters):
    """Router top-k, routing plan, permute and combine at DeepSeek-16B-like sizes (32768 tokens, dim 2048, 64 experts,
    top-6): CUDA-event time and achieved bytes per kernel."""
    from titan_b200.ops.moe import combine, make_plan, permute, router_topk

    _, bw_peak, tag = peaks()
    T_, D, E, k = 32768, 2048, 64, 6
    x = torch.randn(T_, D, device="cuda", dtype=torch.bfloat16)
    logits = torch.randn(T_, E, device="cuda")
    gate, idx, _ = router_topk(logits, k, score_func="softmax")
    plan = make_plan(idx, E)
    buf = permute(x, plan)
    gw = gate.to(torch.bfloat16)
    ms = timeit(lambda: router_topk(logits, k, score_func="softmax"), iters)
    emit(kernel="router_topk", shape=[T_, E, k], ms=ms)
    ms = timeit(lambda: make_plan(idx, E), iters)
    emit(kernel="moe_plan", pairs=T_ * k, ms=ms)
    byt = x.numel() * 2 * (1 + k)
    ms = timeit(lambda: permute(x, plan), iters)
    emit(kernel="moe_permute", shape=[T_, D, k], ms=ms, gbs=byt / ms / 1e6, frac_of_peak=byt / ms / 1e6 / bw_peak, peak=tag)
    ms = timeit(lambda: combine(buf, plan, T_, gw), iters)
    emit(kernel="moe_combine", shape=[T_, D, k], ms=ms, gbs=byt / ms / 1e6, frac_of_peak=byt / ms / 1e6 / bw_peak, peak=tag)


def bench_attention(iters):
    """Causal GQA attention forward, Llama-3 8B shape: the tcgen05 kernel against the library backends."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    from titan_b200.ops.flash_attention import _FlashFn

    tf_peak, _, tag = peaks()
    B, S, H, HK, D = 1, 8192, 32, 8, 128
    q = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    k = torch.randn(B, S, HK, D, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    v = torch.randn(B, S, HK, D, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    fl = 4.0 * B * H * S * S * D / 2
    from titan_b200.ops.flash_attention import _flash_fwd_launch as _fwd

    ours = timeit(lambda: _fwd(q, k, v, D ** -0.5), iters)   # the launch itself: no Python dispatcher in the timed gap
    rec = dict(kernel="flash_fwd_tcgen05", shape=[B, H, HK, S, D], ms=ours, tflops=fl / ours / 1e9,
               frac_of_peak=fl / ours / 1e9 / tf_peak, peak=tag)
    for name, be in (("cudnn", SDPBackend.CUDNN_ATTENTION), ("flash2", SDPBackend.FLASH_ATTENTION)):
        try:
            with sdpa_kernel(be):
                ms = timeit(lambda: F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True), iters)
            rec[f"{name}_ms"], rec[f"{name}_tflops"] = ms, fl / ms / 1e9
        except RuntimeError as e:  # backend not available for this shape
            rec[f"{name}_error"] = str(e)[:80]
    emit(**rec)

    # backward: the tcgen05 kernel (dK / dV in tensor memory, dQ by vector reductions) against the library backends
    from titan_b200.ops.flash_attention import _flash_bwd_launch, _flash_fwd_launch

    g = torch.randn(B, S, H, D, device="cuda", dtype=torch.bfloat16).transpose(1, 2)
    out, lse = _flash_fwd_launch(q, k, v, D ** -0.5)
    ours = timeit(lambda: _flash_bwd_launch(q, k, v, out, lse, g, D ** -0.5), iters)
    rec = dict(kernel="flash_bwd_tcgen05", shape=[B, H, HK, S, D], ms=ours, tflops=2.5 * fl / ours / 1e9,
               frac_of_peak=2.5 * fl / ours / 1e9 / tf_peak, peak=tag)
    for name, be in (("cudnn", SDPBackend.CUDNN_ATTENTION), ("flash2", SDPBackend.FLASH_ATTENTION)):
        try:
            ql, kl, vl = (t.detach().clone().requires_grad_() for t in (q, k, v))
            with sdpa_kernel(be):
                o = F.scaled_dot_product_attention(ql, kl, vl, is_causal=True, enable_gqa=True)
                ms = timeit(lambda: torch.autograd.grad(o, (ql, kl, vl), g, retain_graph=True), iters)
            rec[f"{name}_ms"], rec[f"{name}_tflops"] = ms, 2.5 * fl / ms / 1e9
        except RuntimeError as e:
            rec[f"{name}_error"] = str(e)[:80]
    emit(**rec)

    # packed documents (8 documents of 1024 tokens in one 8192-token row): one launch each way against the
    # per-document loop over the library attention
    from titan_b200.models.common.varlen_attention import VarlenMetadata
    from titan_b200.ops.flash_attention import flash_attention

    meta = VarlenMetadata([list(range(0, S + 1, 1024))], 1024)
    ss = meta.seq_start("cuda")

    def ours_fb():
        ql, kl, vl = (t.detach().requires_grad_() for t in (q, k, v))
        flash_attention(ql, kl, vl, seq_start=ss).backward(g)

    def loop_fb():
        ql, kl, vl = (t.detach().requires_grad_() for t in (q, k, v))
        docs = [F.scaled_dot_product_attention(ql[:, :, a:a + 1024], kl[:, :, a:a + 1024], vl[:, :, a:a + 1024],
                                               is_causal=True, enable_gqa=True) for a in range(0, S, 1024)]
        torch.cat(docs, dim=2).backward(g)

    emit(kernel="flash_packed_docs_fwd_bwd", shape=[B, H, HK, S, D], docs=8, ms=timeit(ours_fb, iters),
         library_loop_ms=timeit(loop_fb, iters))


def bench_lowp(iters):
    """Block-scaled MXFP8 GEMM (operands already quantised) against the library bf16 GEMM of the same shape, and the
    whole quantise + GEMM product against it."""
    from titan_b200.lowp.mx import mx_quantize
    from titan_b200.ops.mxfp8_gemm import mxfp8_gemm, pack_scale_atoms

    tf_peak, _, tag = peaks()
    for M, N, K in [(8192, 4096, 4096), (8192, 14336, 4096), (8192, 4096, 14336), (16384, 8192, 8192)]:
        a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        b = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
        aq, sa = mx_quantize(a, -1)
        bq, sb = mx_quantize(b, -1)
        pa, pb = pack_scale_atoms(sa), pack_scale_atoms(sb)
        fl = 2.0 * M * N * K
        gemm_ms = timeit(lambda: mxfp8_gemm(aq, pa, bq, pb, packed=True), iters)
        t128 = timeit(lambda: mxfp8_gemm(aq, pa, bq, pb, packed=True, tile_n=128), iters)
        t256 = timeit(lambda: mxfp8_gemm(aq, pa, bq, pb, packed=True, tile_n=256), iters)

        def whole():
            q1, s1 = mx_quantize(a, -1)
            q2, s2 = mx_quantize(b, -1)
            return mxfp8_gemm(q1, s1, q2, s2)

        whole_ms = timeit(whole, iters)
        lib_ms = timeit(lambda: a @ b.t(), iters)
        emit(kernel="mxfp8_gemm_block_scaled", shape=[M, N, K], ms=gemm_ms, tflops=fl / gemm_ms / 1e9,
             tile128_ms=t128, tile256_ms=t256,
             with_quantise_ms=whole_ms, with_quantise_tflops=fl / whole_ms / 1e9, cublas_bf16_ms=lib_ms,
             cublas_bf16_tflops=fl / lib_ms / 1e9, vs_bf16_peak=fl / gemm_ms / 1e9 / tf_peak, peak=tag)
    # the quantisers: one pass that writes both views against the two single-axis passes plus the bf16 transpose they need
    from titan_b200.lowp.mx import mx_quantize_dual
    from titan_b200.lowp.mx_linear import mx_linear

    _, bw_peak, _ = peaks()
    for R, C in [(8192, 4096), (8192, 14336)]:
        x = torch.randn(R, C, device="cuda", dtype=torch.bfloat16)
        dual_ms = timeit(lambda: mx_quantize_dual(x), iters)
        row_ms = timeit(lambda: mx_quantize(x, -1), iters)
        t_ms = timeit(lambda: mx_quantize(x.t().contiguous(), -1), iters)
        nbytes = R * C * (2 + 2 * (1 + 1 / 32))
        emit(kernel="mx_quantize_dual", shape=[R, C], ms=dual_ms, gbs=nbytes / dual_ms / 1e6,
             frac_of_copy_bw=nbytes / dual_ms / 1e6 / bw_peak, separate_passes_ms=row_ms + t_ms, peak=tag)
    for T_, N, K in [(8192, 4096, 4096), (8192, 14336, 4096)]:
        x = torch.randn(T_, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        w = (torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02).requires_grad_()
        g = torch.randn(T_, N, device="cuda", dtype=torch.bfloat16)

        def step(lin):
            x.grad = w.grad = None
            lin(x, w).backward(g)

        mx_ms = timeit(lambda: step(mx_linear), iters)
        bf_ms = timeit(lambda: step(torch.nn.functional.linear), iters)
        emit(kernel="mx_linear_fwd_bwd", shape=[T_, N, K], ms=mx_ms, tflops=6.0 * T_ * N * K / mx_ms / 1e9,
             bf16_linear_ms=bf_ms, bf16_linear_tflops=6.0 * T_ * N * K / bf_ms / 1e9, speedup=bf_ms / mx_ms)


    # grouped experts (DeepSeek 16B shapes: 49152 routed rows, 8 local experts): one grouped block-scaled launch per
    # product against the bf16 grouped GEMM of the padded path
    from titan_b200.lowp.mx_linear import mx_grouped_mm
    from titan_b200.ops.moe import grouped_linear

    E, rows = 8, 49152
    offs = torch.full((E,), rows // E, device="cuda", dtype=torch.int32).cumsum(0).to(torch.int32)
    for N, K in [(2816, 2048), (2048, 1408)]:
        x = torch.randn(rows, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
        w = (torch.randn(E, N, K, device="cuda", dtype=torch.bfloat16) * 0.02).requires_grad_()
        g = torch.randn(rows, N, device="cuda", dtype=torch.bfloat16)

        def gstep(fn):
            x.grad = w.grad = None
            fn().backward(g)

        mx_ms = timeit(lambda: gstep(lambda: mx_grouped_mm(x, w, offs, aligned=True)), iters)
        bf_ms = timeit(lambda: gstep(lambda: grouped_linear(x, w, offs)), iters)
        fl = 6.0 * rows * N * K
        emit(kernel="mx_grouped_mm_fwd_bwd", shape=[rows, E, N, K], ms=mx_ms, tflops=fl / mx_ms / 1e9,
             bf16_grouped_ms=bf_ms, bf16_grouped_tflops=fl / bf_ms / 1e9, speedup=bf_ms / mx_ms)


def bench_sparse(iters):
    """Kernels of the dense form of sparse attention: masked softmax (forward / backward) and the indexer-score
    backward, with the bytes they must move against the measured copy bandwidth."""
    from titan_b200.ops.masked_softmax import masked_softmax

    _, bw_peak, tag = peaks()
    H, Sc, T = 16, 512, 8192
    s_ = torch.randn(H, Sc, T, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    allowed = torch.rand(Sc, T, device="cuda") < 0.25
    sink = torch.zeros(H, device="cuda")
    g = torch.randn(H, Sc, T, device="cuda", dtype=torch.bfloat16)
    fwd = timeit(lambda: masked_softmax(s_.detach(), allowed, 1.0, sink), iters)
    p_ = masked_softmax(s_, allowed, 1.0, sink)

    def bwd_only():
        s_.grad = None
        p_.backward(g, retain_graph=True)

    bwd = timeit(bwd_only, iters)
    n = H * Sc * T
    emit(kernel="masked_softmax_fwd", shape=[H, Sc, T], ms=fwd, gbs=(4 * n + Sc * T) / fwd / 1e6,
         frac_of_copy_bw=(4 * n + Sc * T) / fwd / 1e6 / bw_peak, peak=tag)
    emit(kernel="masked_softmax_bwd", shape=[H, Sc, T], ms=bwd, gbs=6 * n / bwd / 1e6,
         frac_of_copy_bw=6 * n / bwd / 1e6 / bw_peak, peak=tag, note="includes the autograd wrapper and the sink reduction")


def bench_sparse_mla(iters):
    """Sparse MLA (DeepSeek sparse attention core): the tcgen05 kernel on gathered key tiles against the dense-masked
    form (one GEMM over all keys + masked softmax + one GEMM) at growing key streams, forward only and forward +
    backward.  16 heads, 576-dim latent keys, 512-dim values, top-2048 keys per query."""
    from titan_b200.ops.dsa import _sparse_chunk
    from titan_b200.ops.sparse_mla import sparse_mla, sparse_mla_forward

    tf_peak, _, tag = peaks()
    H, dq, dv, K = 16, 576, 512, 2048
    for S, T in ((4096, 8192), (4096, 32768), (4096, 131072)):
        g = torch.Generator(device="cuda").manual_seed(0)
        q = (torch.randn(S, H, dq, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
        kv = (torch.randn(T, dq, device="cuda", generator=g) * 0.3).to(torch.bfloat16)
        idx = torch.randint(0, T, (S, K), device="cuda", generator=g, dtype=torch.int32)
        scale = dq ** -0.5
        fwd = timeit(lambda: sparse_mla_forward(q, kv, idx, scale, dv), iters)
        q1, kv1 = q.clone().requires_grad_(), kv.clone().requires_grad_()
        go = torch.randn(S, H, dv, device="cuda", dtype=torch.bfloat16)

        def fb():
            q1.grad = kv1.grad = None
            out, _, _ = sparse_mla(q1, kv1, idx, scale, dv, None, 256)
            out.backward(go)

        fwdbwd = timeit(fb, max(3, iters // 4))
        useful = 2.0 * S * H * K * (dq + dv)   # QK^T over the selected keys + PV
        rec = dict(kernel="sparse_mla_fwd", S=S, T=T, H=H, topk=K, ms=fwd, fwd_bwd_ms=fwdbwd,
                   useful_tflops=useful / fwd / 1e9, frac_of_peak=useful / fwd / 1e9 / tf_peak, peak=tag,
                   gathered_gbs=S * K * (dq + dv) * 2 / fwd / 1e6,
                   note="two passes over the keys: full rows for the logits, the value columns again for P V")
        if T <= 32768:   # the dense-masked form needs [H, chunk, T] logits: only short streams
            qh = q.transpose(0, 1).contiguous()
            v = kv[:, :dv].contiguous()

            def dense():
                for s0 in range(0, S, 256):
                    _sparse_chunk(qh[:, s0:s0 + 256], kv, v, idx[s0:s0 + 256], scale, True)

            rec["dense_masked_ms"] = timeit(dense, max(3, iters // 4))
            rec["speedup_vs_dense_masked"] = rec["dense_masked_ms"] / fwd
        emit(**rec)
        del q, kv, idx


def profile_case(name: str, launches: int = 3) -> None:
    """One small workload (inputs larger than L2, well under 1 GB on the device), launched a few times: the
    target of a profiler capture.  Prints nothing but the case name; timings come from the bench modes."""
    dev, bf = "cuda", torch.bfloat16
    if name == "gemm":
        from titan_b200.ops.gemm import gemm

        a, b = torch.randn(8192, 4096, device=dev, dtype=bf), torch.randn(4096, 4096, device=dev, dtype=bf)
        out = torch.empty(8192, 4096, device=dev, dtype=bf)
        fn = lambda: gemm(a, b, out=out)  # noqa: E731
    elif name == "gemm_wgrad":
        from titan_b200.ops.gemm import gemm

        a, b = torch.randn(8192, 14336, device=dev, dtype=bf), torch.randn(8192, 4096, device=dev, dtype=bf)
        out = torch.empty(14336, 4096, device=dev, dtype=bf)
        fn = lambda: gemm(a, b, a_mn=True, b_mn=True, out=out)  # noqa: E731
    elif name == "sparse_mla":
        from titan_b200.ops.sparse_mla import sparse_mla_forward

        q = (torch.randn(1024, 16, 576, device=dev) * 0.3).to(bf)
        kv = (torch.randn(131072, 576, device=dev) * 0.3).to(bf)      # 151 MB of latent keys: larger than L2
        idx = torch.randint(0, 131072, (1024, 2048), device=dev, dtype=torch.int32)
        fn = lambda: sparse_mla_forward(q, kv, idx, 576 ** -0.5, 512)  # noqa: E731
    elif name == "sparse_mla_bwd":
        from titan_b200.ops.sparse_mla import sparse_mla_backward

        q = (torch.randn(1024, 16, 576, device=dev) * 0.3).to(bf)
        kv = (torch.randn(131072, 576, device=dev) * 0.3).to(bf)
        idx = torch.randint(0, 131072, (1024, 2048), device=dev, dtype=torch.int32)
        go = (torch.randn(1024, 16, 512, device=dev) * 0.3).to(bf)
        lse = torch.full((1024, 16), 8.0, device=dev)
        delta = torch.zeros(1024, 16, device=dev)
        fn = lambda: sparse_mla_backward(q, kv, idx, go, lse, delta, 576 ** -0.5, 512)  # noqa: E731
    elif name == "indexer_sel_bwd":
        from titan_b200.ops.dsa import _indexer_selected_backward

        q = (torch.randn(1, 2048, 64, 128, device=dev) * 0.3).to(bf)
        k = (torch.randn(1, 131072, 1, 128, device=dev) * 0.3).to(bf)
        w = torch.rand(1, 2048, 64, device=dev)
        idx = torch.randint(0, 131072, (1, 2048, 2048), device=dev, dtype=torch.int32)
        g = torch.randn(1, 2048, 2048, device=dev)
        fn = lambda: _indexer_selected_backward(q, w, k, idx, g)  # noqa: E731
    elif name == "rope":
        from titan_b200.models.common import rope as rope_ref
        from titan_b200.ops.rope import rope_apply

        q = torch.randn(2, 8192, 32, 128, device=dev, dtype=bf)     # 134 MB
        cache = rope_ref.precompute_freqs_cis(128, 8192, 500000.0).cuda()
        fn = lambda: rope_apply(q, cache)  # noqa: E731
    elif name == "swiglu":
        from titan_b200.ops.swiglu import swiglu

        a = torch.randn(8192, 14336, device=dev, dtype=bf, requires_grad=True)   # 235 MB each
        b = torch.randn(8192, 14336, device=dev, dtype=bf, requires_grad=True)
        g = torch.randn(8192, 14336, device=dev, dtype=bf)

        def fn():
            a.grad = b.grad = None
            swiglu(a, b).backward(g)
    elif name == "cross_entropy":
        from titan_b200.ops.cross_entropy import cross_entropy_sum

        logits = torch.randn(2048, 128256, device=dev, dtype=bf, requires_grad=True)   # 525 MB
        labels = torch.randint(0, 128256, (2048,), device=dev)

        def fn():
            logits.grad = None
            cross_entropy_sum(logits, labels).backward()
    elif name == "adamw":
        from titan_b200.optim.fused_adamw import adamw_multi_tensor

        n = 64 * 1024 * 1024
        p_, gr = torch.randn(n, device=dev, dtype=bf), torch.randn(n, device=dev, dtype=bf)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        fn = lambda: adamw_multi_tensor([p_], [gr], [m], [v], lr=1e-3, beta1=0.9, beta2=0.95, eps=1e-8,  # noqa: E731
                                        weight_decay=0.1, step=3)
    elif name == "moe_route_permute_combine":
        from titan_b200.ops.moe import combine, make_plan, permute, router_topk

        T_, D, E, k = 32768, 2048, 64, 6                           # x 134 MB; routed copies 805 MB
        x = torch.randn(T_, D, device=dev, dtype=bf)
        logits = torch.randn(T_, E, device=dev)

        def fn():
            gate, idx, _ = router_topk(logits, k, score_func="softmax")
            plan = make_plan(idx, E)
            buf = permute(x, plan)
            combine(buf, plan, T_, gate.to(bf))
    elif name == "grouped_gemm":
        from titan_b200.ops.moe import grouped_linear

        E, rows, D, Hd = 8, 4096, 2048, 1408
        x = torch.randn(E * rows, D, device=dev, dtype=bf)
        w = torch.randn(E, Hd, D, device=dev, dtype=bf) * 0.02
        offs = (torch.arange(1, E + 1, device=dev, dtype=torch.int32) * rows)
        fn = lambda: grouped_linear(x, w, offs)  # noqa: E731
    elif name == "mhc":
        from titan_b200.ops.mhc_cuda import mhc_post, mhc_pre

        T_, D = 8192, 2048                                          # streams [T, 4, D] bf16 = 134 MB
        x = torch.randn(T_, 4, D, device=dev, dtype=bf, requires_grad=True)
        hfn = (torch.randn(24, 4 * D, device=dev) * 0.05).requires_grad_()
        hs = (torch.randn(3, device=dev) * 0.5 + 1.0).requires_grad_()
        hb = (torch.randn(24, device=dev) * 0.3).requires_grad_()
        g = torch.randn(T_, 4, D, device=dev, dtype=bf)

        def fn():
            x.grad = hfn.grad = hs.grad = hb.grad = None
            y, post, comb = mhc_pre(x, hfn, hs, hb, 20, 1e-6, 1e-6)
            mhc_post(y, x, post, comb).backward(g)
    elif name == "compressor_pool":
        from titan_b200.ops.compressor_pool import compressor_pool

        B_, S_, d = 2, 16384, 512                                   # ratio 4 with overlap: width 1024, 134 MB per input
        kv = torch.randn(B_, S_, 2 * d, device=dev, requires_grad=True)
        score = torch.randn(B_, S_, 2 * d, device=dev, requires_grad=True)
        ape = torch.randn(4, 2 * d, device=dev, requires_grad=True)
        g = torch.randn(B_, S_ // 4, d, device=dev)

        def fn():
            kv.grad = score.grad = ape.grad = None
            compressor_pool(kv, score, ape, 4, d, True).backward(g)
    elif name == "rmsnorm_bwd":
        from titan_b200.ops.norm import rms_norm

        x = torch.randn(16384, 4096, device=dev, dtype=bf, requires_grad=True)
        w = torch.ones(4096, device=dev, dtype=bf, requires_grad=True)
        g = torch.randn(16384, 4096, device=dev, dtype=bf)

        def fn():
            x.grad = w.grad = None
            rms_norm(x, w, 1e-6).backward(g)
    elif name == "indexer_topk":
        from titan_b200.ops.dsa import lightning_indexer_topk

        q = torch.randn(1, 4096, 64, 128, device=dev, dtype=bf)
        k = torch.randn(1, 16384, 1, 128, device=dev, dtype=bf)
        w = torch.rand(1, 4096, 64, device=dev)
        fn = lambda: lightning_indexer_topk(q, w, k, 2048, 16384 - 4096)  # noqa: E731
    elif name == "flash_fwd":
        from titan_b200.ops.flash_attention import _FlashFn

        q = torch.randn(1, 8192, 32, 128, device=dev, dtype=bf).transpose(1, 2)
        k = torch.randn(1, 8192, 8, 128, device=dev, dtype=bf).transpose(1, 2)
        v = torch.randn(1, 8192, 8, 128, device=dev, dtype=bf).transpose(1, 2)
        fn = lambda: _FlashFn.apply(q, k, v, 128 ** -0.5, None)  # noqa: E731
    elif name == "flash_bwd":
        from titan_b200.ops.flash_attention import _flash_bwd_launch, _flash_fwd_launch

        q = torch.randn(1, 8192, 32, 128, device=dev, dtype=bf).transpose(1, 2)
        k = torch.randn(1, 8192, 8, 128, device=dev, dtype=bf).transpose(1, 2)
        v = torch.randn(1, 8192, 8, 128, device=dev, dtype=bf).transpose(1, 2)
        g = torch.randn(1, 8192, 32, 128, device=dev, dtype=bf).transpose(1, 2)
        out, lse = _flash_fwd_launch(q, k, v, 128 ** -0.5)
        fn = lambda: _flash_bwd_launch(q, k, v, out, lse, g, 128 ** -0.5)  # noqa: E731
    elif name == "mxfp8_gemm":
        from titan_b200.ops.mxfp8_gemm import mxfp8_gemm, pack_scale_atoms

        aq = torch.randn(8192, 4096, device=dev).to(torch.float8_e4m3fn)
        bq = torch.randn(4096, 4096, device=dev).to(torch.float8_e4m3fn)
        pa = pack_scale_atoms(torch.randint(120, 134, (8192, 128), dtype=torch.uint8, device=dev))
        pb = pack_scale_atoms(torch.randint(120, 134, (4096, 128), dtype=torch.uint8, device=dev))
        fn = lambda: mxfp8_gemm(aq, pa, bq, pb, packed=True)  # noqa: E731
    elif name == "masked_softmax":
        from titan_b200.ops.masked_softmax import masked_softmax

        # 16 heads x 512 queries x 8192 keys in bf16 (134 MB of logits: larger than L2), a quarter of the keys allowed
        s_ = torch.randn(16, 512, 8192, device=dev, dtype=bf, requires_grad=True)
        allowed = torch.rand(512, 8192, device=dev) < 0.25
        sink = torch.zeros(16, device=dev)
        g = torch.randn(16, 512, 8192, device=dev, dtype=bf)

        def fn():
            s_.grad = None
            masked_softmax(s_, allowed, 1.0, sink).backward(g)
    elif name == "indexer_relu_bwd":
        import ctypes

        from titan_b200.ops import _lib

        P, I, LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        _lib.declare("tb_indexer_relu_bwd", [P, P, P, P, P, LL, I, I, I, P])
        sc, heads, keys = 128, 64, 8192  # x: 128 x 64 x 8192 bf16 = 134 MB
        x = torch.randn(sc * heads, keys, device=dev, dtype=bf)
        dscore = torch.randn(sc, keys, device=dev)
        w = torch.rand(sc * heads, device=dev)
        dx, dw = torch.empty_like(x), torch.empty(sc * heads, device=dev)

        def fn():
            rc = _lib.lib().tb_indexer_relu_bwd(x.data_ptr(), dscore.data_ptr(), w.data_ptr(), dx.data_ptr(),
                                                dw.data_ptr(), sc * heads, heads, keys, 1, _lib.stream_ptr())
            _lib.check(rc, "indexer_relu_bwd")
    elif name == "mx_quantize_dual":
        from titan_b200.lowp.mx import mx_quantize_dual

        x = torch.randn(16384, 4096, device=dev, dtype=bf)  # 134 MB in, 138 MB out

        def fn():
            mx_quantize_dual(x)
    else:
        raise SystemExit(f"unknown profile case {name!r}")
    for _ in range(launches):
        fn()
    torch.cuda.synchronize()
    print(json.dumps({"profile_case": name, "launches": launches}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="gemm,elementwise")
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--profile-case", default=None,
                    help="run one small case a few times and exit (see `profile_case` for the names)")
    args = ap.parse_args()
    if args.profile_case:
        profile_case(args.profile_case)
        return
    which = set(args.only.split(","))
    if "gemm" in which:
        bench_gemm(args.iters)
    if "gemm_sustained" in which:
        bench_gemm_sustained()
    if "sparse_mla" in which:
        bench_sparse_mla(args.iters)
    if "moe" in which:
        bench_moe(args.iters)
    if "indexer" in which:
        bench_indexer(args.iters)
    if "elementwise" in which:
        bench_elementwise(args.iters)
    if "attention" in which:
        bench_attention(args.iters)
    if "lowp" in which:
        bench_lowp(args.iters)
    if "sparse" in which:
        bench_sparse(args.iters)


if __name__ == "__main__":
    main()
