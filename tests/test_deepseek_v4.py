"""DeepSeek-V4 on CPU: index sets, compressor, hyper-connections, fused sparse path vs the dense oracle, MoE routing,
state-dict mapping, and a two-step trainer run.

Models what the reference covers in tests/unit_tests/models/test_deepseek_v4_{moe,rope_cache,state_dict_adapter,
parallelize_static,pp_static}.py and tests/unit_tests/converters/test_mhc*.py.
"""

import pytest
import torch

from titan_b200.models.deepseek_v4 import DeepSeekV4Model, deepseekv4_configs
from titan_b200.models.deepseek_v4.layers import (
    Compressor,
    compress_visible_idxs,
    li_compute,
    sparse_attention_dense,
    window_topk_idxs,
)
from titan_b200.ops import mhc
from titan_b200.ops.smla import li_select, smla_attention


def _cfg(**kw):
    cfg = deepseekv4_configs["smoketest"]()
    cfg.max_seq_len = 256
    for k, v in kw.items():
        setattr(cfg, k, v)
    return cfg


def test_window_and_compress_index_sets():
    w = window_topk_idxs(4, 6)
    assert w.shape == (6, 4)
    assert w[0].tolist() == [0, -1, -1, -1]
    assert w[5].tolist() == [2, 3, 4, 5]
    c = compress_visible_idxs(4, 8, offset=8)
    assert c.shape == (8, 2)
    assert c[2].tolist() == [-1, -1]  # block 0 closes at token 3
    assert c[3].tolist() == [8, -1]
    assert c[7].tolist() == [8, 9]


def test_sinkhorn_is_doubly_stochastic_and_hc_roundtrip_shapes():
    torch.manual_seed(0)
    mixes = torch.randn(5, 24)
    pre, post, comb = mhc.hc_split_sinkhorn(mixes, torch.tensor([1.0, 1.0, 1.0]), torch.zeros(24), 4, 20, 1e-6)
    assert pre.shape == (5, 4) and post.shape == (5, 4) and comb.shape == (5, 4, 4)
    assert torch.allclose(comb.sum(-1), torch.ones(5, 4), atol=1e-3)
    assert torch.allclose(comb.sum(-2), torch.ones(5, 4), atol=1e-3)
    assert (post > 0).all() and (post < 2).all()
    x = torch.randn(2, 3, 4, 16)
    fn = torch.randn(24, 64) * 0.1
    y, post, comb = mhc.hc_pre(x, fn, torch.ones(3), torch.zeros(24))
    assert y.shape == (2, 3, 16)
    out = mhc.hc_post(y, x, post, comb)
    assert out.shape == x.shape
    # out[n] = post[n]·y + Σ_m comb[m, n]·x[m]
    ref = post[..., None] * y[..., None, :] + torch.einsum("bsmn,bsmd->bsnd", comb, x)
    assert torch.allclose(out, ref, atol=1e-5)


def test_compressor_overlap_pools_previous_block():
    cfg = _cfg()
    comp = Compressor(cfg, 4, 32)
    comp.init_states()
    # first compressed key only sees block 0's second-half projections: the slots of the (missing) previous block
    # carry -inf gates and must get zero weight
    kv = torch.randn(1, 8, 64)
    score = torch.zeros(1, 8, 64)
    with torch.no_grad():
        comp.ape.zero_()
    pooled = comp.pool(kv, score)
    assert pooled.shape == (1, 2, 32)
    assert torch.allclose(pooled[0, 0], kv[0, :4, 32:].mean(0), atol=1e-6)
    expect = torch.cat([kv[0, :4, :32], kv[0, 4:, 32:]], 0).mean(0)
    assert torch.allclose(pooled[0, 1], expect, atol=1e-6)


@pytest.mark.parametrize("ratio", [1, 4, 16])
def test_fused_sparse_attention_matches_dense_oracle(ratio):
    torch.manual_seed(1)
    B, S, H, hd, window = 2, 64, 4, 32, 8
    q = torch.randn(B, S, H, hd, requires_grad=True)
    kv = torch.randn(B, S, hd, requires_grad=True)
    sink = torch.randn(H, requires_grad=True)
    kvc = torch.randn(B, S // ratio, hd, requires_grad=True) if ratio > 1 else None
    idx = None
    if ratio == 4:
        qi, ki, w = torch.randn(B, S, 2, 16), torch.randn(B, S // 4, 16), torch.rand(B, S, 2)
        idx, _ = li_compute(qi, ki, w, 4, 5, S)
    out_ref, probs = sparse_attention_dense(q, kv, sink, kvc, idx, window, ratio, hd ** -0.5)
    g = torch.randn_like(out_ref)
    grads_ref = torch.autograd.grad(out_ref, [t for t in (q, kv, sink, kvc) if t is not None], g)
    out, dist = smla_attention(q, kv, sink, kvc, idx, window, ratio, hd ** -0.5, want_dist=True, chunk=16)
    grads = torch.autograd.grad(out, [t for t in (q, kv, sink, kvc) if t is not None], g)
    assert torch.allclose(out, out_ref, atol=1e-5)
    for a, b in zip(grads, grads_ref):
        assert torch.allclose(a, b, atol=1e-4)
    if ratio == 4:
        cmp = probs[..., S:].sum(1) / H
        ref_dist = torch.gather(cmp, -1, (idx - S).clamp(min=0)).masked_fill(idx < 0, 0.0)
        assert torch.allclose(dist, ref_dist, atol=1e-6)


def test_li_select_matches_eager_selection():
    torch.manual_seed(2)
    B, S, Hi, Di = 2, 64, 4, 16
    qi, ki, w = torch.randn(B, S, Hi, Di), torch.randn(B, S // 4, Di), torch.rand(B, S, Hi)
    idx_ref, val_ref = li_compute(qi, ki, w, 4, 6, S)
    idx, val = li_select(qi, ki, w, 4, 6, S)
    assert torch.equal(idx.sort(-1).values, idx_ref.sort(-1).values)
    ok = idx_ref >= 0
    assert torch.allclose(val.sort(-1).values[ok.sort(-1).values], val_ref.sort(-1).values[ok.sort(-1).values],
                          atol=1e-5)


def test_model_forward_backward_with_and_without_fused_core():
    torch.manual_seed(0)
    cfg = _cfg(num_mtp_modules=1)
    model = DeepSeekV4Model(cfg)
    model.init_states()
    tok = torch.randint(0, cfg.vocab_size, (2, 129))
    cfg.max_seq_len = 128
    outs = model(tok)
    assert [tuple(o.shape) for o in outs] == [(2, 128, cfg.vocab_size)] * 2
    from titan_b200.converters.smla import SMLAConverter

    SMLAConverter().convert(model)
    outs_f = model(tok)
    for a, b in zip(outs, outs_f):
        assert torch.allclose(a, b, atol=2e-4), (a - b).abs().max()
    sum(o.float().logsumexp(-1).mean() for o in outs_f).backward()
    missing = [n for n, p in model.named_parameters() if p.grad is None]
    assert missing == []
    # the indexer is trained by its KL loss only
    g = model.layers["2"].attention.pre_attention.indexer.wq_b.weight.grad
    assert g.abs().sum() > 0


def test_hash_layers_route_by_token_id_and_have_no_bias():
    cfg = _cfg()
    model = DeepSeekV4Model(cfg)
    model.init_states()
    moe0, moe1 = model.layers["0"].moe, model.layers["1"].moe
    assert moe0.router.hash and moe0.expert_bias is None
    assert not moe1.router.hash and moe1.expert_bias is not None
    x = torch.randn(6, cfg.dim)
    ids = torch.tensor([5, 9, 5, 9, 5, 9])
    _, sel, _ = moe0.router(x, None, ids)
    assert torch.equal(sel[0], sel[2]) and torch.equal(sel[1], sel[3])


def test_state_dict_adapter_roundtrip():
    from titan_b200.models.deepseek_v4.state_dict_adapter import DeepSeekV4StateDictAdapter

    cfg = _cfg(num_mtp_modules=1)
    model = DeepSeekV4Model(cfg)
    model.init_states()
    sd = {k: v for k, v in model.state_dict().items()}
    ad = DeepSeekV4StateDictAdapter(cfg)
    hf = ad.to_hf(sd)
    assert "embed.weight" in hf and "head.weight" in hf and "hc_head_fn" in hf
    assert "layers.2.attn.compressor.ape" in hf and "layers.3.attn.compressor.wkv.weight" in hf
    assert "layers.2.attn.indexer.compressor.ape" in hf
    assert "layers.0.ffn.gate.tid2eid" in hf and hf["layers.0.ffn.gate.tid2eid"].dtype == torch.float32
    assert "layers.1.ffn.gate.bias" in hf and "layers.0.ffn.gate.bias" not in hf
    assert "layers.1.ffn.experts.7.w2.weight" in hf
    assert "mtp.0.e_proj.weight" in hf and "mtp.0.norm.weight" in hf and "mtp.0.hc_head_scale" in hf
    back = ad.from_hf(hf)
    assert set(back) == set(sd)
    for k in sd:
        assert torch.equal(back[k].to(sd[k].dtype), sd[k]), k


def _launch(args, nproc, port, timeout=900):
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, PYTHONPATH=root, OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), "-m", "titan_b200.entry", *args]
    res = subprocess.run(cmd, cwd=root, env=env, capture_output=True, text=True, timeout=timeout)
    log = res.stdout + res.stderr
    assert res.returncode == 0, log[-4000:]
    return log


def _losses(log):
    import re

    return [float(m) for m in re.findall(r"r0\] .*? step:\s+\d+\s+loss:\s+([0-9.]+|nan|inf)", log)]


_BASE = ["--module", "deepseek_v4", "--config", "deepseek_v4_smoketest", "--training.seq_len", "128",
         "--comm.backend", "gloo", "--training.local_batch_size", "2"]


def _step_line(log, step):
    import re

    m = re.search(rf"r0\] .*? step:\s+{step}\s+loss:\s+([0-9.]+)\s+grad_norm:\s+([0-9.]+)", log)
    assert m, log[-3000:]
    return float(m.group(1)), float(m.group(2))


def test_trainer_tp2_and_fsdp2_reproduce_the_single_rank_step(tmp_path):
    """One rank trains 2 steps and checkpoints after step 1.  A tensor-parallel pair resumes from that checkpoint
    (resharded load) and must reproduce step 2: same loss and same gradient norm."""
    folder = str(tmp_path / "run")
    common = [*_BASE, "--job.dump_folder", folder, "--checkpoint.enable", "--checkpoint.interval", "1",
              "--training.steps", "2"]
    ref = _step_line(_launch(common, 1, 29560), 2)
    tp = _step_line(_launch([*common, "--checkpoint.load_step", "1", "--parallelism.data_parallel_shard_degree", "1",
                             "--parallelism.tensor_parallel_degree", "2"], 2, 29561), 2)
    assert abs(tp[0] - ref[0]) < 2e-3 and abs(tp[1] - ref[1]) < 2e-3 * max(ref[1], 1.0), (tp, ref)


def test_trainer_fsdp2_three_steps(tmp_path):
    log = _launch([*_BASE, "--job.dump_folder", str(tmp_path / "fsdp"), "--training.local_batch_size", "1",
                   "--parallelism.data_parallel_shard_degree", "2", "--training.steps", "3"], 2, 29562)
    fsdp = _losses(log)
    assert len(fsdp) == 3 and all(x == x and x < 20 for x in fsdp), log[-2000:]


@pytest.mark.gpu
def test_li_select_kernels_match_eager_selection_on_gpu():
    """Compressed keys (ratio 4): tcgen05 scoring + radix top-k must pick the same key set as the dense oracle."""
    torch.manual_seed(3)
    dev = "cuda"
    B, S, Hi, Di, k = 2, 2048, 64, 128, 128
    qi = torch.randn(B, S, Hi, Di, device=dev, dtype=torch.bfloat16)
    ki = torch.randn(B, S // 4, Di, device=dev, dtype=torch.bfloat16)
    w = torch.rand(B, S, Hi, device=dev, dtype=torch.bfloat16)
    idx_ref, _ = li_compute(qi.float(), ki.float(), w.float(), 4, k, S)
    idx, val = li_select(qi, ki, w, 4, k, S)
    assert idx.shape == idx_ref.shape
    # same number of valid slots per query; the sets agree except for near-ties of bf16 vs fp32 scoring
    assert torch.equal((idx >= 0).sum(-1), (idx_ref >= 0).sum(-1))
    same = 0
    total = 0
    for b in range(B):
        for s in range(0, S, 97):
            a = set(idx[b, s][idx[b, s] >= 0].tolist())
            r = set(idx_ref[b, s][idx_ref[b, s] >= 0].tolist())
            same += len(a & r)
            total += len(r)
            assert all(S <= t < S + (s + 1) // 4 for t in a)
    assert same >= 0.97 * total


@pytest.mark.gpu
def test_v4_model_bf16_step_on_gpu_with_fused_paths():
    torch.manual_seed(0)
    cfg = _cfg(num_mtp_modules=1)
    cfg.max_seq_len = 256
    with torch.device("cuda"):
        model = DeepSeekV4Model(cfg)
    model.init_states(buffer_device=torch.device("cuda"))
    tok = torch.randint(0, cfg.vocab_size, (2, 257), device="cuda")
    ref = [o.float() for o in model(tok)]
    from titan_b200.converters.smla import SMLAConverter

    SMLAConverter().convert(model)
    outs = model(tok)
    for a, b in zip(ref, outs):
        assert torch.allclose(a, b.float(), atol=5e-3, rtol=5e-3), (a - b.float()).abs().max()
    model.bfloat16()
    outs = model(tok)
    loss = sum(o.float().logsumexp(-1).mean() for o in outs)
    loss.backward()
    assert torch.isfinite(loss)
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


def test_sparse_attention_dense_mask_and_gather_paths_agree():
    """The selected compressed keys are attended either through one masked GEMM (short streams) or through a row gather
    whose backward is a scatter-add (long streams): same output, same gradients."""
    from titan_b200.ops import smla

    torch.manual_seed(3)
    B, S, H, hd, ratio, k = 1, 64, 2, 16, 4, 6
    Tc = S // ratio
    mk = lambda *s: torch.randn(*s, dtype=torch.float64)
    q, kv, kvc, sink = mk(B, S, H, hd), mk(B, S, hd), mk(B, Tc, hd), mk(H)
    # per query: k distinct visible compressed keys (or -1 where fewer are visible)
    idx = torch.full((B, S, k), -1, dtype=torch.long)
    for s in range(S):
        vis = (s + 1) // ratio
        pick = torch.randperm(vis)[:k] if vis else torch.empty(0, dtype=torch.long)
        idx[0, s, : pick.numel()] = pick + S
    results = []
    saved = smla.DENSE_RATIO
    for dense_ratio in (4, 0):
        smla.DENSE_RATIO = dense_ratio
        try:
            leaves = [t.clone().requires_grad_(True) for t in (q, kv, kvc)]
            out, dist = smla.smla_attention(leaves[0], leaves[1], sink, leaves[2], idx, 8, ratio, hd ** -0.5,
                                            want_dist=True, chunk=16)
            out.square().sum().backward()
            results.append((out.detach(), dist, [t.grad for t in leaves]))
        finally:
            smla.DENSE_RATIO = saved
    (o1, d1, g1), (o2, d2, g2) = results
    torch.testing.assert_close(o1, o2)
    torch.testing.assert_close(d1, d2)
    for a, b in zip(g1, g2):  # the gather path accumulates its scatter-add in fp32
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("with_idx", [True, False])
def test_fused_chunk_path_matches_dense_oracle_on_gpu(with_idx):
    """bf16 on CUDA takes the one-GEMM / masked-softmax-with-sink / one-GEMM path: against the fp32 dense oracle,
    outputs, the indexer's teacher distribution and all gradients (queries, keys, compressed keys, sink)."""
    from titan_b200.ops import smla

    torch.manual_seed(7)
    B, S, H, hd, ratio, k, window = 1, 256, 4, 64, 4, 16, 32
    Tc = S // ratio
    dev = "cuda"
    q = torch.randn(B, S, H, hd, device=dev) * 0.5
    kv = torch.randn(B, S, hd, device=dev) * 0.5
    kvc = torch.randn(B, Tc, hd, device=dev) * 0.5
    sink = torch.randn(H, device=dev)
    idx = None
    if with_idx:
        idx = torch.full((B, S, k), -1, dtype=torch.long, device=dev)
        for s in range(S):
            vis = (s + 1) // ratio
            pick = torch.randperm(vis, device=dev)[:k]
            idx[0, s, : pick.numel()] = pick + S
    scale = hd ** -0.5
    ref_leaves = [t.clone().requires_grad_(True) for t in (q, kv, kvc, sink)]
    ref, probs = sparse_attention_dense(ref_leaves[0], ref_leaves[1], ref_leaves[3], ref_leaves[2], idx, window, ratio,
                                        scale)
    leaves = [t.to(torch.bfloat16).requires_grad_(True) for t in (q, kv, kvc)] + [sink.clone().requires_grad_(True)]
    out, dist = smla.smla_attention(leaves[0], leaves[1], leaves[3], leaves[2], idx, window, ratio, scale,
                                    want_dist=with_idx)
    torch.testing.assert_close(out.float(), ref, rtol=5e-2, atol=3e-2)
    if with_idx:
        cmp = probs[..., S:].detach().sum(dim=1) / H
        want = torch.gather(cmp, -1, (idx - S).clamp(min=0)).masked_fill(idx < 0, 0.0)
        torch.testing.assert_close(dist, want, rtol=5e-2, atol=2e-2)
    g = torch.randn_like(ref)
    ref.backward(g)
    out.backward(g.to(out.dtype))
    for a, b, name in zip(leaves, ref_leaves, ("dq", "dkv", "dkvc", "dsink")):
        torch.testing.assert_close(a.grad.float(), b.grad.float(), rtol=8e-2, atol=6e-2,
                                   msg=lambda m, n=name: f"{n}: {m}")


@pytest.mark.gpu
def test_gathered_tile_kernel_path_matches_dense_oracle_on_gpu():
    """Head dim 128 with a long compressed stream goes to the tensor-core gathered-tile kernel: window keys and selected
    compressed keys are listed per query in one key buffer.  Outputs, teacher distribution and gradients against the
    fp32 dense oracle."""
    from titan_b200.ops import smla

    torch.manual_seed(11)
    B, S, H, hd, ratio, k, window = 2, 384, 16, 128, 4, 24, 32
    Tc = S // ratio
    dev = "cuda"
    q = torch.randn(B, S, H, hd, device=dev) * 0.5
    kv = torch.randn(B, S, hd, device=dev) * 0.5
    kvc = torch.randn(B, Tc, hd, device=dev) * 0.5
    sink = torch.randn(H, device=dev)
    idx = torch.full((B, S, k), -1, dtype=torch.long, device=dev)
    for b in range(B):
        for s in range(S):
            vis = (s + 1) // ratio
            pick = torch.randperm(vis, device=dev)[:k]
            idx[b, s, : pick.numel()] = pick + S
    scale = hd ** -0.5
    ref_leaves = [t.clone().requires_grad_(True) for t in (q, kv, kvc, sink)]
    ref, probs = sparse_attention_dense(ref_leaves[0], ref_leaves[1], ref_leaves[3], ref_leaves[2], idx, window, ratio,
                                        scale)
    leaves = [t.to(torch.bfloat16).requires_grad_(True) for t in (q, kv, kvc)] + [sink.clone().requires_grad_(True)]
    saved = smla.KERNEL_RATIO
    smla.KERNEL_RATIO = 0
    try:
        assert smla._kernel_takes(leaves[0], leaves[2], idx, window, ratio)
        out, dist = smla.smla_attention(leaves[0], leaves[1], leaves[3], leaves[2], idx, window, ratio, scale,
                                        want_dist=True)
    finally:
        smla.KERNEL_RATIO = saved
    torch.testing.assert_close(out.float(), ref, rtol=5e-2, atol=3e-2)
    cmp = probs[..., S:].detach().sum(dim=1) / H
    want = torch.gather(cmp, -1, (idx - S).clamp(min=0)).masked_fill(idx < 0, 0.0)
    torch.testing.assert_close(dist, want, rtol=5e-2, atol=2e-2)
    g = torch.randn_like(ref)
    ref.backward(g)
    out.backward(g.to(out.dtype))
    for a, b_, name in zip(leaves, ref_leaves, ("dq", "dkv", "dkvc", "dsink")):
        torch.testing.assert_close(a.grad.float(), b_.grad.float(), rtol=8e-2, atol=6e-2,
                                   msg=lambda m, n=name: f"{n}: {m}")


def test_kernel_path_key_lists_match_the_dense_oracle_on_cpu(monkeypatch):
    """The key lists handed to the gathered-tile kernel (window of raw keys, then the selected compressed keys, as rows
    of one buffer, padded to 128) with the kernel replaced by its fp32 gather oracle: same output and teacher
    distribution as the dense statement of the attention."""
    from titan_b200.ops import smla, sparse_mla as sm

    def oracle(q, kv, idx, scale, dv, sink=None, chunk=128):
        out, lse, teacher = sm.sparse_mla_forward_ref(q, kv, idx, scale, dv, sink)
        return out, teacher, lse

    monkeypatch.setattr(sm, "sparse_mla", oracle)
    monkeypatch.setattr(smla, "_kernel_takes", lambda *a, **k: True)
    torch.manual_seed(2)
    B, S, H, hd, ratio, k, window = 2, 96, 4, 32, 4, 8, 16
    Tc = S // ratio
    mk = lambda *s: torch.randn(*s, dtype=torch.float64) * 0.5  # noqa: E731
    q, kv, kvc, sink = mk(B, S, H, hd), mk(B, S, hd), mk(B, Tc, hd), mk(H)
    idx = torch.full((B, S, k), -1, dtype=torch.long)
    for b in range(B):
        for s in range(S):
            vis = (s + 1) // ratio
            pick = torch.randperm(vis)[:k]
            idx[b, s, : pick.numel()] = pick + S
    scale = hd ** -0.5
    ref, probs = sparse_attention_dense(q, kv, sink, kvc, idx, window, ratio, scale)
    out, dist = smla.smla_attention(q, kv, sink, kvc, idx, window, ratio, scale, want_dist=True)
    torch.testing.assert_close(out, ref.to(out.dtype), rtol=1e-4, atol=1e-6)   # the oracle works in fp32
    cmp = probs[..., S:].sum(dim=1) / H
    want = torch.gather(cmp, -1, (idx - S).clamp(min=0)).masked_fill(idx < 0, 0.0)
    torch.testing.assert_close(dist, want.to(dist.dtype), rtol=1e-4, atol=1e-6)


def test_compile_plan_reproduces_the_eager_steps_under_fsdp(tmp_path):
    """`--compile.enable` compiles the projections around the attention cores and the router / shared experts in
    place (the cores and the routed experts stay eager): two FSDP ranks must log the losses of the eager run, and the
    checkpoint keeps its parameter names."""
    common = [*_BASE, "--training.steps", "2", "--metrics.log_freq", "1", "--debug.seed", "0"]
    eager = _launch([*common, "--job.dump_folder", str(tmp_path / "eager")], 2, 29566)
    comp = _launch([*common, "--job.dump_folder", str(tmp_path / "compiled"), "--compile.enable",
                    "--compile.backend", "aot_eager"], 2, 29567)
    assert "compiled" in comp and "DeepSeek-V4 submodules" in comp
    a, b = _losses(eager), _losses(comp)
    assert len(a) == 2 and len(b) == 2
    assert all(abs(x - y) < 1e-3 for x, y in zip(a, b)), (a, b)


def test_compile_plan_skips_cores_experts_and_norms():
    from types import SimpleNamespace

    from titan_b200.models.deepseek_v4.parallelize import apply_compile
    from titan_b200.protocols.model_spec import get_model_spec

    spec = get_model_spec("deepseek_v4", "smoketest")
    with torch.device("meta"):
        model = spec.model.build()
    compiled = []
    import torch.nn as nn

    real = nn.Module.compile
    nn.Module.compile = lambda self, *a, **k: compiled.append(self)
    try:
        n = apply_compile(model, SimpleNamespace(backend="eager"))
        n_tnd = apply_compile(model, SimpleNamespace(backend="eager"), use_global_tnd=True)
    finally:
        nn.Module.compile = real
    names = {type(m).__name__ for m in compiled}
    assert n == len(compiled) - n_tnd and n > n_tnd > 0
    assert "InnerAttention" not in names and not any("Experts" in t and "Shared" not in t for t in names), names
    assert not any("norm" in t.lower() for t in names), names
    assert {"PreAttention", "PostAttention"} <= names
