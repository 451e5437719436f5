"""`torch.ops.titan_b200.*`: fake kernels give the right shapes on the meta device, selective activation
checkpointing keeps the contraction ops, and (GPU) a converted block neither recomputes its GEMMs under selective
checkpointing nor breaks `torch.compile(fullgraph=True)`."""

import pytest
import torch


def test_fake_kernels_give_shapes_on_meta():
    from titan_b200.ops.registry import ops

    bf = torch.bfloat16
    a, b = torch.empty(64, 32, device="meta", dtype=bf), torch.empty(48, 32, device="meta", dtype=bf)
    assert ops.gemm(a, b).shape == (64, 48) and ops.gemm(a, b).dtype == bf
    assert ops.gemm(a, a, True, True, True).shape == (32, 32) and ops.gemm(a, a, True, True, True).dtype == torch.float32
    x, w = torch.empty(4, 8, 16, device="meta", dtype=bf), torch.empty(16, device="meta", dtype=bf)
    y, rstd = ops.rms_norm_fwd(x, w, 1e-5)
    assert y.shape == x.shape and rstd.shape == (32,) and rstd.dtype == torch.float32
    dx, dw = ops.rms_norm_bwd(y, x, w, rstd)
    assert dx.shape == x.shape and dw.shape == w.shape
    g = torch.empty(32, 24, device="meta", dtype=bf)
    assert ops.swiglu_fwd(g, g, None, 32, 24, 24, 0.0).shape == (32, 24)
    assert ops.swiglu_fwd(g, None, None, 32, 12, 24, 0.0).shape == (32, 12)
    dg, du, ds = ops.swiglu_bwd(g, g, g, None, 32, 24, 24, 0.0)
    assert dg.shape == g.shape and du.shape == g.shape and ds.numel() == 0
    q = torch.empty(2, 16, 4, 8, device="meta", dtype=bf)
    assert ops.rope(q, torch.empty(16, 4, 2, device="meta"), None, True, False).shape == q.shape
    logits, labels = torch.empty(32, 100, device="meta", dtype=bf), torch.empty(32, device="meta", dtype=torch.int64)
    loss, lse = ops.cross_entropy_fwd(logits, labels, -100)
    assert loss.shape == (32,) and lse.shape == (32,)
    offs = torch.empty(4, device="meta", dtype=torch.int32)
    assert ops.grouped_gemm_m(a, torch.empty(4, 48, 32, device="meta", dtype=bf), offs, 48, False).shape == (64, 48)
    assert ops.grouped_gemm_k(a, a, offs, 4).shape == (4, 32, 32)
    qh = torch.empty(1, 8, 256, 128, device="meta", dtype=bf)
    kh = torch.empty(1, 2, 256, 128, device="meta", dtype=bf)
    o, l = ops.flash_attention_fwd(qh, kh, kh, 0.1)
    assert o.shape == qh.shape and l.shape == (1, 8, 256)


def test_contraction_ops_are_on_the_selective_checkpoint_save_list():
    from titan_b200.ops.registry import CONTRACTION_OPS
    from titan_b200.parallel.activation_checkpoint import sac_save_ops

    assert set(CONTRACTION_OPS) <= sac_save_ops()


@pytest.mark.gpu
def test_selective_checkpointing_keeps_tcgen05_gemm_outputs(cuda_device):
    """Forward + backward of a checkpointed feed-forward block: 3 linears x (fwd, dgrad, wgrad) = 9 GEMM launches;
    a recomputed forward would add 3 more."""
    from titan_b200.config.configs import ActivationCheckpointConfig
    from titan_b200.converters.linear import TcLinear
    from titan_b200.models.common.layers import FeedForward
    from titan_b200.ops import _lib
    from titan_b200.parallel.activation_checkpoint import apply_ac

    torch.manual_seed(0)
    ff = FeedForward(dim=256, hidden_dim=512).to(device="cuda", dtype=torch.bfloat16)
    for m in ff.modules():
        if type(m).__name__ == "Linear":
            m.__class__ = TcLinear
    ref = FeedForward(dim=256, hidden_dim=512).to(device="cuda", dtype=torch.bfloat16)
    ref.load_state_dict(ff.state_dict())
    holder = torch.nn.Module()
    holder.layers = torch.nn.ModuleDict({"0": ff})
    apply_ac(holder, ActivationCheckpointConfig(mode="selective", selective_ac_option="op_save_all_mm"))
    x = torch.randn(2, 128, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    before = _lib.launch_count()
    y = holder.layers["0"](x)
    y.float().pow(2).sum().backward()
    torch.cuda.synchronize()
    launches = _lib.launch_count() - before
    yr = ref(xr)
    yr.float().pow(2).sum().backward()
    torch.testing.assert_close(y.float(), yr.float(), rtol=3e-2, atol=3e-2)
    torch.testing.assert_close(x.grad.float(), xr.grad.float(), rtol=5e-2, atol=5e-1)
    assert launches == 9, launches


@pytest.mark.gpu
def test_converted_ops_compile_fullgraph(cuda_device):
    from titan_b200.ops.gemm import linear
    from titan_b200.ops.norm import rms_norm
    from titan_b200.ops.swiglu import swiglu

    torch.manual_seed(0)
    w1 = (torch.randn(512, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    w3 = (torch.randn(512, 256, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    nw = torch.ones(256, device="cuda", dtype=torch.bfloat16, requires_grad=True)

    def f(x):
        h = rms_norm(x, nw, 1e-5)
        return swiglu(linear(h, w1), linear(h, w3))

    x = torch.randn(256, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    eager = f(x)
    compiled = torch.compile(f, fullgraph=True)(x)
    torch.testing.assert_close(compiled.float(), eager.float(), rtol=2e-2, atol=2e-2)
    compiled.float().sum().backward()
    assert x.grad is not None and w1.grad is not None and torch.isfinite(x.grad.float()).all()


def test_ops_go_through_the_dispatcher_only_when_somebody_watches():
    """`ops.<name>` calls the launcher directly for eager CUDA tensors and the dispatcher operator under a dispatch
    mode (selective checkpointing, fake tensors) or for meta tensors."""
    import torch
    from torch.utils._python_dispatch import TorchDispatchMode

    from titan_b200.ops import registry

    class Watch(TorchDispatchMode):
        def __torch_dispatch__(self, func, types, args=(), kwargs=None):
            return func(*args, **(kwargs or {}))

    meta = torch.empty(4, 8, device="meta")
    assert registry._nobody_watches((meta,)) is False          # meta tensors need the fake kernel
    assert registry._nobody_watches((3, None)) is False        # no tensor in front: nothing to launch on
    with Watch():
        assert registry._nobody_watches((meta,)) is False
    assert registry.ops.gemm.default is torch.ops.titan_b200.gemm.default
    assert registry.ops.swiglu_fwd.op is torch.ops.titan_b200.swiglu_fwd


def test_selective_checkpointing_keeps_swiglu_only_where_a_recipe_asks():
    from titan_b200.config.manager import resolve_recipe
    from titan_b200.ops import registry
    from titan_b200.parallel.activation_checkpoint import sac_save_ops

    assert registry.SWIGLU_OPS[0] not in sac_save_ops()        # not global: MoE blocks hold capacity-sized buffers
    assert resolve_recipe("llama3", "llama3_8b").activation_checkpoint.selective_keep_swiglu
    assert not resolve_recipe("deepseek_v32", "deepseek_v32_sparse_cp8").activation_checkpoint.selective_keep_swiglu
    for op in (registry.ops.gemm.default, registry.ops.sparse_mla_fwd.default, registry.ops.indexer_topk.default,
               registry.ops.mx_linear_fwd.default):
        assert op in sac_save_ops()
