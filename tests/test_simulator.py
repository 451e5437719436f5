"""Memory simulator against peaks measured on B200s (`torch.cuda.max_memory_allocated` of the benchmark runs).

Measured, Llama-3 8B, seq 8192, local batch 1, bf16 weights + fp32 AdamW state, FSDP2 keeping the gathered weights
between forward and backward: without recomputation 112.0 / 89.9 / 70.8 / 61.5 GiB on 1 / 2 / 4 / 8 GPUs; with
selective checkpointing (every contraction kept) 103.0 GiB on one GPU.  The estimate has to land within 10 %."""

import pytest
import torch

MEASURED_GIB = {
    ("llama3_8b_noac", 1): 112.0,
    ("llama3_8b_noac", 2): 89.9,
    ("llama3_8b_noac", 4): 70.8,
    ("llama3_8b_noac", 8): 61.5,
    ("llama3_8b", 1): 103.0,
}


@pytest.mark.parametrize("recipe,world", sorted(MEASURED_GIB))
def test_estimate_matches_measured_peak(recipe, world):
    from titan_b200.config.manager import resolve_recipe
    from titan_b200.simulator.memory import estimate

    cfg = resolve_recipe("llama3", recipe)
    cfg.parallelism.fsdp_reduce_scatter = "nccl"   # the measured runs used the stock reduce-scatter
    rep = estimate(cfg, world)
    got = rep.bytes_total / 2 ** 30
    want = MEASURED_GIB[(recipe, world)]
    assert abs(got / want - 1) < 0.10, (got, want, rep.summary())
    assert rep.fits
    assert not any("closed-form" in n for n in rep.notes), rep.notes   # the converted model ran on meta tensors


def _v32_sparse(seq_len, cp):
    def edit(cfg):
        cfg.training.seq_len = seq_len
        cfg.parallelism.context_parallel_degree = cp
        cfg.parallelism.data_parallel_shard_degree = -1
    return edit


def _llama_selective_without_swiglu_keep(cfg):
    cfg.activation_checkpoint.selective_keep_swiglu = False


def _v4_mini_as_benchmarked(cfg):
    from titan_b200.protocols.converter import ConverterConfig

    cfg.training.seq_len, cfg.training.local_batch_size, cfg.training.dtype = 3840, 1, "bfloat16"
    cfg.model_converters.converters = [ConverterConfig(name=n, options={}) for n in (
        "b200_rms_norm", "b200_rope", "b200_moe_dispatch", "b200_gmm", "b200_smla", "b200_mhc_pre", "b200_mhc_post")]


# (module, recipe, edit, world) -> GiB measured by `torch.cuda.max_memory_allocated` in benchmark runs on B200s.
# MoE, sparse-attention, hyper-connection and MXFP8 models run their kernel code paths on meta tensors (no launches),
# fused expert parallelism sizes its buffers for the capacity factor, library optimizers keep bf16 moments.
MEASURED_MORE = [
    ("deepseek_v32", "deepseek_v32_sparse_cp8", _v32_sparse(8192, 1), 1, 91.9),
    ("deepseek_v32", "deepseek_v32_sparse_cp8", _v32_sparse(32768, 1), 1, 166.5),
    ("deepseek_v32", "deepseek_v32_sparse_cp8", _v32_sparse(65536, 2), 2, 133.7),
    ("deepseek_v32", "deepseek_v32_sparse_cp8", _v32_sparse(131072, 4), 4, 117.2),
    ("deepseek_v3", "deepseek_v3_16b_ep8", None, 8, 81.5),
    ("deepseek_v4", "debug_deepseek_v4_single_node_1b", _v4_mini_as_benchmarked, 1, 18.7),
    ("llama3", "llama3_8b", None, 1, 110.0),
    ("llama3", "llama3_8b", _llama_selective_without_swiglu_keep, 2, 80.5),
    ("llama3", "llama3_8b", _llama_selective_without_swiglu_keep, 4, 61.8),
    ("llama3", "llama3_8b", _llama_selective_without_swiglu_keep, 8, 52.5),
    ("llama3", "llama3_8b_mxfp8", None, 1, 110.8),
    ("llama3", "llama3_8b_baseline", None, 1, 81.8),
]


@pytest.mark.parametrize("module,recipe,edit,world,want", MEASURED_MORE,
                         ids=[f"{r}-{getattr(e, '__name__', 'as_is') if e else 'as_is'}-{w}gpu-{g}GiB"
                              for _, r, e, w, g in MEASURED_MORE])
def test_estimate_matches_measured_peak_of_other_models(module, recipe, edit, world, want):
    from titan_b200.config.manager import resolve_recipe
    from titan_b200.simulator.memory import estimate

    cfg = resolve_recipe(module, recipe)
    if edit is not None:
        edit(cfg)
    rep = estimate(cfg, world)
    got = rep.bytes_total / 2 ** 30
    assert abs(got / want - 1) < 0.08, (got, want, rep.summary())
    assert not any("closed-form" in n for n in rep.notes), rep.notes


def test_no_launch_mode_restores_the_library_and_keeps_declarations():
    from titan_b200.ops import _lib

    with _lib.no_launch():
        assert _lib.launches_disabled() and _lib.stream_ptr() == 0
        assert _lib.lib().tb_anything(1, 2, 3) == 0
        _lib.declare("tb_example_entry", [])          # remembered, applied when the real library is next used
        assert _lib.on_device(torch.empty(1, device="meta"))
    assert not _lib.launches_disabled()
    assert not _lib.on_device(torch.empty(1, device="meta"))
    assert "tb_example_entry" in _lib._PENDING_DECLARATIONS
    _lib._PENDING_DECLARATIONS.pop("tb_example_entry")


def test_tracker_gives_value_dependent_ops_a_shape_on_meta_tensors():
    from titan_b200.simulator.memory import MetaMemoryTracker

    idx = torch.empty(64, dtype=torch.int64, device="meta")
    with MetaMemoryTracker() as tr:
        counts = torch.bincount(idx, minlength=8)
        hist = torch.histc(torch.empty(64, device="meta"), bins=16, min=0, max=15)
        where = torch.nonzero(torch.empty(4, 5, device="meta"))
        assert counts.shape == (8,) and hist.shape == (16,) and where.shape == (20, 2)   # nonzero: upper bound
        assert tr.current == 8 * 8 + 16 * 4 + 20 * 2 * 8
    with pytest.raises(NotImplementedError), MetaMemoryTracker():
        torch.empty(3, device="meta").tolist()   # a host read has no stand-in: callers must not need the values


def test_peak_is_not_activations_plus_gradients():
    """On one GPU the peak sits at the start of backward: hardly any gradient exists there."""
    from titan_b200.config.manager import resolve_recipe
    from titan_b200.simulator.memory import estimate

    rep = estimate(resolve_recipe("llama3", "llama3_8b_noac"), 1)
    assert rep.bytes_grads_at_peak < 0.1 * rep.bytes_grads
    assert rep.bytes_total < rep.bytes_params + rep.bytes_grads + rep.bytes_optimizer_device + rep.bytes_activations


def test_tracker_ignores_views_of_outside_storages():
    from titan_b200.simulator.memory import MetaMemoryTracker

    w = torch.empty(1024, 1024, device="meta")
    x = torch.empty(8, 1024, device="meta")
    with MetaMemoryTracker() as tr:
        y = x @ w.t()          # the transpose is a view of `w`: nothing new but `y`
        assert tr.current == y.numel() * 4
        tr.reweight(y, 0.25)
        assert tr.current == y.numel()


@pytest.mark.gpu
def test_estimate_against_a_real_run(cuda_device, tmp_path):
    """Two steps of a 1B-parameter Llama on the device; the estimate must be within 10 % of the allocator's peak."""
    from titan_b200.config.manager import resolve_recipe
    from titan_b200.simulator.memory import estimate

    cfg = resolve_recipe("llama3", "llama3_8b")
    cfg.model.overrides = {"n_layers": 4, "vocab_size": 32000}
    cfg.training.seq_len = 4096
    cfg.training.steps = 2
    cfg.metrics.log_freq = 1
    cfg.checkpoint.enable = False
    cfg.job.dump_folder = str(tmp_path)
    est = estimate(cfg, 1).bytes_total
    torch.cuda.reset_peak_memory_stats()
    base = torch.cuda.memory_allocated()
    trainer = cfg.build()
    try:
        trainer.train()
        peak = torch.cuda.max_memory_allocated() - base
    finally:
        trainer.close()
    assert abs(est / peak - 1) < 0.10, (est / 2 ** 30, peak / 2 ** 30)
