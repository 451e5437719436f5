"""Low-precision training on CPU: MX numerics, MX linear / grouped autograd against fp32 (SQNR floors), the MXFP8
converter, parameter-level QAT (prepare / convert), and — on a GPU — the MX kernels against the PyTorch statement.

SQNR floors follow the reference's experimental tests (experiments/ao_npu/tests/test_training.py:33-50):
fp8 row-wise weight fake-quant ≥ 30 / 30 / 22 dB (out / input grad / param grad), block-fp8 + MX ≥ 12 / 12 / 8 dB.
"""

import pytest
import torch
import torch.nn as nn

from titan_b200.lowp.mx import (
    mx_dequantize_ref,
    mx_fake_quantize,
    mx_quantize,
    mx_quantize_dual,
    mx_quantize_ref,
    sqnr,
)
from titan_b200.lowp.mx_converter import MXFP8Converter, MXFP8ConverterConfig
from titan_b200.lowp.mx_linear import mx_grouped_mm, mx_linear
from titan_b200.lowp.qat import (
    ParamSwapConfig,
    QuantizeConfig,
    block_fp8_fake_quantize,
    fp8_rowwise_fake_quantize,
    mxfp4_fake_quantize,
    quantize_params,
)


def test_mx_scale_rules_and_roundtrip():
    x = torch.zeros(2, 64)
    x[0, :32] = torch.linspace(-448, 448, 32)      # amax 448 → exponent 0 under rceil
    x[0, 32:] = torch.linspace(-1, 1, 32) * 449     # just above → exponent 1
    x[1, :32] = 0.0                                  # empty block
    x[1, 32:] = torch.randn(32) * 1e-3
    q, s = mx_quantize_ref(x, -1, "rceil")
    assert s[0].tolist() == [127, 128] and s[1, 0] == 0
    back = mx_dequantize_ref(q, s, -1, torch.float32)
    assert torch.equal(back[0, :32].abs().max(), torch.tensor(448.0)) and back[1, :32].abs().sum() == 0
    # floor rule: floor(log2(448)) - 8 = 0; values stay within e4m3 after clipping
    qf, sf = mx_quantize_ref(x, -1, "floor")
    assert sf[0, 0] == 127
    # axis -2 quantises down the rows
    y = torch.randn(64, 16)
    q2, s2 = mx_quantize_ref(y, -2)
    assert q2.shape == (64, 16) and s2.shape == (2, 16)
    assert sqnr(y, mx_dequantize_ref(q2, s2, -2, torch.float32)) > 25
    assert torch.equal(mx_quantize(y, -2)[1], s2)


def test_mx_linear_gradients_meet_sqnr_floors():
    torch.manual_seed(0)
    x = torch.randn(96, 128, requires_grad=True)
    w = (torch.randn(64, 128) * 0.05).requires_grad_()
    g = torch.randn(96, 64)
    y = mx_linear(x, w)
    y.backward(g)
    xr, wr = x.detach().clone().requires_grad_(), w.detach().clone().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g)
    assert sqnr(yr, y) > 25 and sqnr(xr.grad, x.grad) > 25 and sqnr(wr.grad, w.grad) > 25
    # the quantise-once form (every dim a multiple of 32) computes exactly what three separately quantised GEMMs do
    fq = lambda t, ax: mx_fake_quantize(t.detach(), ax)  # noqa: E731
    assert torch.allclose(y, fq(x, -1) @ fq(w, -1).t(), atol=1e-5)
    assert torch.allclose(x.grad, fq(g, -1) @ fq(w, -2), atol=1e-5)
    assert torch.allclose(w.grad, fq(g, -2).t() @ fq(x, -2), atol=1e-4)
    # ragged dims are padded inside the op
    x2 = torch.randn(5, 40, requires_grad=True)
    w2 = torch.randn(7, 40, requires_grad=True)
    mx_linear(x2, w2).sum().backward()
    assert x2.grad.shape == x2.shape and w2.grad.shape == w2.shape


def test_mx_grouped_mm_matches_per_expert_linears():
    torch.manual_seed(1)
    x = torch.randn(64, 64, requires_grad=True)
    w = (torch.randn(3, 32, 64) * 0.1).requires_grad_()
    offs = torch.tensor([32, 32, 64], dtype=torch.int32)  # expert 1 is empty
    out = mx_grouped_mm(x, w, offs)
    out.sum().backward()
    ref0, ref2 = mx_linear(x[:32].detach(), w[0].detach()), mx_linear(x[32:].detach(), w[2].detach())
    assert torch.allclose(out[:32], ref0, atol=1e-5) and torch.allclose(out[32:], ref2, atol=1e-5)
    assert w.grad[1].abs().sum() == 0 and w.grad[0].abs().sum() > 0


def test_mxfp8_converter_on_moe_model():
    from titan_b200.models.qwen3 import Qwen3Model, qwen3_configs

    torch.manual_seed(0)
    cfg = qwen3_configs["debugmodel_moe"]()
    cfg.max_seq_len = 64
    model = Qwen3Model(cfg)
    model.init_states()
    tok = torch.randint(0, cfg.vocab_size, (2, 64))
    ref = model(tok)
    conv = MXFP8Converter(MXFP8ConverterConfig(fqns=["attention.wq", "attention.wo", "moe.experts"]))
    conv.convert(model)
    assert any("moe.experts" in n for n in conv.converted) and any(n.endswith("attention.wq") for n in conv.converted)
    out = model(tok)
    assert 15 < sqnr(ref, out) < 80  # quantisation is visible but small
    out.float().logsumexp(-1).mean().backward()
    assert model.layers["0"].moe.experts.w1.grad is not None
    with pytest.raises(ValueError, match="matched no module"):
        MXFP8Converter(MXFP8ConverterConfig(fqns=["nothing.here"])).convert(model)
    with pytest.raises(ValueError, match="unknown MXFP8 recipe"):
        MXFP8Converter(MXFP8ConverterConfig(recipe_name="mxfp3"))


def test_quantisers_sqnr():
    torch.manual_seed(2)
    w = torch.randn(96, 160)
    assert sqnr(w, fp8_rowwise_fake_quantize(w)) > 25
    assert sqnr(w, block_fp8_fake_quantize(w)) > 20
    assert 8 < sqnr(w, mxfp4_fake_quantize(w)) < 25
    assert sqnr(w, block_fp8_fake_quantize(w, mxfp4_prepass=True)) > 8
    assert fp8_rowwise_fake_quantize(w[:0]).shape == (0, 160)


class _MLP(nn.Module):
    def __init__(self):
        super().__init__()
        self.tok_embeddings = nn.Embedding(16, 64)
        self.w_in = nn.Linear(64, 128, bias=False)
        self.norm = nn.LayerNorm(128)
        self.w_out = nn.Linear(128, 64, bias=False)

    def forward(self, x):
        return self.w_out(torch.tanh(self.w_in(x) * 0.1))


# two quantised layers: e4m3's 3 mantissa bits give ~28 dB per weight matrix
@pytest.mark.parametrize("kind,floors", [("fp8_rowwise", (22, 22, 18)), ("mx", (20, 20, 16)), ("block_fp8", (12, 12, 8))])
def test_param_swap_prepare_trains_and_convert_bakes(kind, floors):
    torch.manual_seed(3)
    model, ref = _MLP(), _MLP()
    ref.load_state_dict(model.state_dict())
    names = quantize_params(model, ParamSwapConfig(weight_config=QuantizeConfig(kind=kind)))
    assert sorted(names) == ["w_in.weight", "w_out.weight"]  # embeddings and norms stay in high precision
    x = torch.randn(32, 64, requires_grad=True)
    xr = x.detach().clone().requires_grad_()
    g = torch.randn(32, 64)
    model(x).backward(g)
    ref(xr).backward(g)
    orig = model.w_in.parametrizations.weight.original
    assert sqnr(ref(xr), model(x)) > floors[0] and sqnr(xr.grad, x.grad) > floors[1]
    assert sqnr(ref.w_in.weight.grad, orig.grad) > floors[2]
    before = model.w_in.weight.detach().clone()
    quantize_params(model, ParamSwapConfig(step="convert"))
    assert not hasattr(model.w_in, "parametrizations") and torch.equal(model.w_in.weight, before)


def test_activation_fake_quant_hook_and_filter():
    model = _MLP()
    cfg = ParamSwapConfig(weight_config=QuantizeConfig(kind="fp8_rowwise"),
                          activation_config=QuantizeConfig(kind="fp8_rowwise"),
                          params_filter_fn=lambda n, p: n == "w_out.weight")
    assert quantize_params(model, cfg) == ["w_out.weight"]
    assert hasattr(model.w_out, "_act_fq_hook") and not hasattr(model.w_in, "_act_fq_hook")
    assert model(torch.randn(4, 64)).shape == (4, 64)
    assert model(torch.randn(0, 64)).shape == (0, 64)


@pytest.mark.gpu
@pytest.mark.parametrize("axis", [-1, -2])
@pytest.mark.parametrize("round_mode", ["rceil", "floor"])
def test_mx_kernels_match_reference_on_gpu(axis, round_mode, cuda_device):
    torch.manual_seed(4)
    x = (torch.randn(256, 512, device="cuda") * torch.logspace(-3, 2, 512, device="cuda")).to(torch.bfloat16)
    x[3, :64] = 0
    q, s = mx_quantize(x, axis, round_mode)
    qr, sr = mx_quantize_ref(x, axis, round_mode)
    assert torch.equal(s, sr)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    back = mx_fake_quantize(x, axis, round_mode)
    assert torch.equal(back, mx_dequantize_ref(qr, sr, axis))
    assert sqnr(x, back) > 25


@pytest.mark.gpu
def test_mx_linear_on_gpu_uses_kernels(cuda_device):
    from titan_b200.ops import _lib

    torch.manual_seed(5)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 512, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    before = _lib.launch_count()
    y = mx_linear(x, w)
    y.backward(torch.randn_like(y))
    g = torch.randn_like(y)
    before = _lib.launch_count()
    x.grad = w.grad = None
    y = mx_linear(x, w)
    y.backward(g)
    assert _lib.launch_count() - before == 7  # quantise once: x, w | g, w-transposed; three block-scaled GEMMs
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xr @ wr.t()
    yr.backward(g.float())
    assert sqnr(yr, y) > 25 and sqnr(xr.grad, x.grad) > 25 and sqnr(wr.grad, w.grad) > 25


@pytest.mark.gpu
@pytest.mark.parametrize("shape", [(256, 512), (96, 160), (64, 4096), (384, 128)])
@pytest.mark.parametrize("round_mode", ["rceil", "floor"])
def test_mx_dual_axis_kernel_matches_both_single_axis_references(shape, round_mode, cuda_device):
    torch.manual_seed(6)
    R, C = shape
    x = (torch.randn(R, C, device="cuda") * torch.logspace(-3, 2, C, device="cuda")).to(torch.bfloat16)
    x[3, :64] = 0
    q1, s1, q2t, s2t = mx_quantize_dual(x, round_mode)
    qr, sr = mx_quantize_ref(x, -1, round_mode)
    qt, st = mx_quantize_ref(x.t().contiguous(), -1, round_mode)
    assert torch.equal(s1, sr) and torch.equal(q1.view(torch.uint8), qr.view(torch.uint8))
    assert torch.equal(s2t, st) and torch.equal(q2t.view(torch.uint8), qt.view(torch.uint8))
    only_t = mx_quantize_dual(x, round_mode, rows=False)
    assert only_t[0] is None and torch.equal(only_t[2].view(torch.uint8), qt.view(torch.uint8))
    if R % 128 == 0 and C % 128 == 0:  # scales straight in the GEMM's atom order
        from titan_b200.ops.mxfp8_gemm import pack_scale_atoms

        a1, p1, a2, p2 = mx_quantize_dual(x, round_mode, atoms=True)
        assert torch.equal(a1.view(torch.uint8), qr.view(torch.uint8)) and torch.equal(p1, pack_scale_atoms(sr))
        assert torch.equal(a2.view(torch.uint8), qt.view(torch.uint8)) and torch.equal(p2, pack_scale_atoms(st))


def test_block_fp8_linear_reuses_one_weight_quantisation_for_forward_and_dgrad():
    from titan_b200.lowp.block_fp8 import block_dequantize_weight, block_fp8_grouped_mm, block_fp8_linear, block_quantize_weight

    torch.manual_seed(7)
    x = torch.randn(64, 96, requires_grad=True)
    w = (torch.randn(128, 96) * 0.05).requires_grad_()
    g = torch.randn(64, 128)
    q, s = block_quantize_weight(w.detach())
    assert s.shape == (4, 3) and q.dtype == torch.float8_e4m3fn
    wd = block_dequantize_weight(q, s, dtype=torch.float32)
    assert torch.equal(wd, block_fp8_fake_quantize(w.detach()))  # same arithmetic as the fake quantiser
    y = block_fp8_linear(x, w)
    y.backward(g)
    fq = lambda t, ax: mx_fake_quantize(t.detach(), ax)  # noqa: E731
    assert torch.allclose(y, fq(x, -1) @ wd.t(), atol=1e-5)
    assert torch.allclose(x.grad, fq(g, -1) @ wd, atol=1e-5)  # dgrad reads the SAME quantised weight
    assert torch.allclose(w.grad, fq(g, -2).t() @ fq(x, -2), atol=1e-4)
    ref = x.detach() @ w.detach().t()
    assert sqnr(ref, y) > 20
    # MXFP4 pre-pass, ragged shapes (fallback statement), bias, grouped form
    yp = block_fp8_linear(x, w, mxfp4_prepass=True)
    assert 8 < sqnr(ref, yp) < sqnr(ref, y)
    x2, w2 = torch.randn(5, 40, requires_grad=True), torch.randn(7, 40, requires_grad=True)
    block_fp8_linear(x2, w2, torch.zeros(7)).sum().backward()
    assert x2.grad.shape == x2.shape and w2.grad.shape == w2.shape
    we = torch.randn(2, 64, 96) * 0.05
    offs = torch.tensor([32, 64])
    out = block_fp8_grouped_mm(x.detach(), we, offs)
    assert torch.allclose(out[:32], block_fp8_linear(x.detach()[:32], we[0]))
    assert torch.allclose(out[32:], block_fp8_linear(x.detach()[32:], we[1]))


def test_mxfp4_packed_format_roundtrip_and_pair_table():
    from titan_b200.lowp.mxfp4 import E2M1_GRID, mxfp4_dequantize, mxfp4_quantize

    torch.manual_seed(8)
    x = torch.randn(6, 128) * torch.logspace(-2, 2, 128)
    packed, scales = mxfp4_quantize(x)
    assert packed.shape == (6, 64) and packed.dtype == torch.uint8 and scales.shape == (6, 4)
    back = mxfp4_dequantize(packed, scales, torch.float32)
    assert torch.equal(back, mxfp4_fake_quantize(x))
    # every representable value survives exactly, in both nibbles, with both signs
    grid = torch.tensor(E2M1_GRID)
    vals = torch.cat([grid, -grid]).repeat(2)  # 32 values = one block, amax 6 -> scale 1
    p, s = mxfp4_quantize(vals[None])
    assert int(s[0, 0]) == 127 and torch.equal(mxfp4_dequantize(p, s, torch.float32)[0], vals)
    assert int(p[0, 0]) == (1 << 4) | 0 and int(p[0, 4]) == ((8 | 1) << 4) | 0  # (0, .5) and (-0 -> +0, -.5)
    # ties go to the even grid index: 2.5 -> 2 (index 4), 3.5 -> 4 (index 6), 0.25 -> 0, 0.75 -> 1
    t = torch.zeros(1, 32)
    t[0, :5] = torch.tensor([6.0, 2.5, 3.5, 0.25, 0.75])
    p, s = mxfp4_quantize(t)
    assert mxfp4_dequantize(p, s, torch.float32)[0, :5].tolist() == [6.0, 2.0, 4.0, 0.0, 1.0]


def test_param_filters_and_real_compute_mode():
    from titan_b200.lowp import filters as F_
    from titan_b200.lowp.qat import fake_quantize

    class Experts(nn.Module):
        def __init__(self):
            super().__init__()
            self.num_experts = 2
            self.w13 = nn.Parameter(torch.randn(2, 64, 32) * 0.05)
            self.w2 = nn.Parameter(torch.randn(2, 32, 32) * 0.05)

    model = nn.ModuleDict({"attn": nn.ModuleDict({"wq": nn.Linear(64, 64, bias=False), "wo": nn.Linear(64, 64)}),
                           "router": nn.Linear(64, 8, bias=False), "experts": Experts(), "norm": nn.LayerNorm(64)})
    names = lambda f: sorted(n for m_n, m in model.named_modules() for p_n, p in m.named_parameters(recurse=False)  # noqa: E731
                             for n in [f"{m_n}.{p_n}"] if F_.call_filter(f, n, p, m))
    assert names(F_.is_expert()) == ["experts.w13", "experts.w2"]
    assert names(F_.all_filters(F_.match_module_type(nn.Linear), F_.min_dims(2), F_.not_filter(F_.match_fqn_regex(r"^router")))) \
        == ["attn.wo.weight", "attn.wq.weight"]
    assert names(F_.any_filter(F_.match_fqn_exact("router.weight"), F_.match_fqn_suffix(".wq.weight"))) \
        == ["attn.wq.weight", "router.weight"]
    assert names(lambda fqn, p: fqn.startswith("norm")) == ["norm.bias", "norm.weight"]  # two-argument filters still work

    pick = F_.any_filter(F_.is_expert(), F_.all_filters(F_.match_fqn_regex(r"^attn\."), F_.min_dims(2)))
    for kind in ("mx", "block_fp8"):
        for p in model.parameters():
            if p.dim() >= 2:
                nn.init.normal_(p, std=0.05)
        cfg = ParamSwapConfig(weight_config=QuantizeConfig(kind=kind), params_filter_fn=pick, compute="real")
        touched = quantize_params(model, cfg)
        assert sorted(touched) == ["attn.wo.weight", "attn.wq.weight", "experts.w13", "experts.w2"]
        assert callable(model["experts"].mx_grouped_mm) and "forward" not in model["router"].__dict__
        x = torch.randn(32, 64, requires_grad=True)
        y = model["attn"]["wo"](model["attn"]["wq"](x))
        y.sum().backward()
        ref = nn.functional.linear(nn.functional.linear(x, model["attn"]["wq"].weight), model["attn"]["wo"].weight,
                                   model["attn"]["wo"].bias)
        assert 15 < sqnr(ref, y) < 60 and model["attn"]["wq"].weight.grad is not None
        out = model["experts"].mx_grouped_mm(torch.randn(64, 32), model["experts"].w13, torch.tensor([32, 64]), "rceil")
        assert out.shape == (64, 64)
        before = model["attn"]["wq"].weight.detach().clone()
        baked = quantize_params(model, ParamSwapConfig(step="convert", weight_config=QuantizeConfig(kind=kind)))
        assert sorted(baked) == sorted(touched) and "forward" not in model["attn"]["wq"].__dict__
        assert not hasattr(model["experts"], "mx_grouped_mm")
        w = model["attn"]["wq"].weight.detach()
        assert not torch.equal(w, before) and torch.equal(w, fake_quantize(w, QuantizeConfig(kind=kind)))  # idempotent
    with pytest.raises(ValueError):
        quantize_params(model, ParamSwapConfig(weight_config=QuantizeConfig(kind="fp8_rowwise"), compute="real"))


@pytest.mark.gpu
def test_block_fp8_linear_on_gpu_matches_the_cpu_statement(cuda_device):
    from titan_b200.lowp.block_fp8 import block_fp8_linear
    from titan_b200.ops import _lib

    torch.manual_seed(9)
    x = torch.randn(256, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 512, device="cuda", dtype=torch.bfloat16) * 0.05).requires_grad_()
    g = torch.randn(256, 384, device="cuda", dtype=torch.bfloat16)
    before = _lib.launch_count()
    y = block_fp8_linear(x, w)
    y.backward(g)
    assert _lib.launch_count() - before == 5  # x and g through the dual-axis quantiser, three block-scaled GEMMs
    xc, wc = x.detach().cpu().float().requires_grad_(), w.detach().cpu().float().requires_grad_()
    yc = block_fp8_linear(xc, wc)
    yc.backward(g.cpu().float())
    assert sqnr(yc, y.cpu()) > 40 and sqnr(xc.grad, x.grad.cpu()) > 40 and sqnr(wc.grad, w.grad.cpu()) > 40
