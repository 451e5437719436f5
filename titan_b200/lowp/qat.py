"""Parameter-level quantisation-aware training: matching parameters are swapped for quantising wrappers.

`quantize_params(model, ParamSwapConfig(...))` registers a parametrisation on every matching weight, so ANY use of the
weight (linear, matmul, grouped matmul, bmm, addmm) sees its quantise-dequantise image while the optimizer keeps
training the high-precision original; gradients pass straight through (STE).  ``step="prepare"`` installs the wrappers;
``step="convert"`` bakes the quantised values into the parameters and removes them (export).  An optional activation
config fake-quantises the inputs of converted `nn.Linear` modules along their last dim (skipped for empty inputs).

Quantisers (`weight_config.kind`):
* ``fp8_rowwise``  – one fp32 scale per row (last-dim reduction), e4m3 elements;
* ``mx``           – 1×32 blocks, e8m0 scale, e4m3 elements (`lowp.mx`);
* ``block_fp8``    – 32×32 weight blocks with one power-of-two scale each, e4m3 elements, optionally after an MXFP4
                     (e2m1, 1×32) fake-quant pre-pass (``mxfp4_prepass=True``);
* ``mxfp4``        – 1×32 blocks, e8m0 scale, e2m1 elements.

``compute="real"`` (kinds ``mx`` and ``block_fp8``) goes one step further for the modules that own a matching weight:
an `nn.Linear` runs `mx_linear` / `block_fp8_linear` and a grouped-experts module runs the grouped forms, i.e. real
block-scaled FP8 GEMMs on the tensor cores with fp8 saved activations, instead of a bf16 GEMM on fake-quantised values.
Filters may be two-argument ``(fqn, parameter)`` callables or the three-argument predicates of `lowp.filters`.

Parity: the experimental `torchao_npu` package of the reference (experiments/ao_npu/torchao_npu/configs.py,
quantization/quant_configs.py:24-104, quant_primitives/{mx,block_fp8}.py, wrapper_tensors/*.py): its tensor-subclass
wrappers become parametrisations here, which FSDP2 and DCP handle without extra hooks because the stored parameter
stays an ordinary tensor.
"""

from __future__ import annotations

from collections.abc import Callable
from dataclasses import dataclass, field

import torch
import torch.nn as nn
import torch.nn.utils.parametrize as parametrize

from titan_b200.lowp.mx import BLOCK, mx_fake_quantize
from titan_b200.protocols.converter import ModelConverter

__all__ = ["QuantizeConfig", "ParamSwapConfig", "quantize_params", "QuantizeConverter", "QuantizeConverterConfig",
           "fp8_rowwise_fake_quantize", "block_fp8_fake_quantize", "mxfp4_fake_quantize", "fake_quantize"]

E4M3_MAX = 448.0
_E2M1_GRID = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])


def fp8_rowwise_fake_quantize(x: torch.Tensor) -> torch.Tensor:
    amax = x.detach().abs().amax(dim=-1, keepdim=True).float().clamp_min(1e-12)
    scale = E4M3_MAX / amax
    q = (x.float() * scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float()
    return (q / scale).to(x.dtype)


def _pow2_scale(amax: torch.Tensor, elem_max: float) -> torch.Tensor:
    e = torch.ceil(torch.log2(amax.clamp_min(1e-30) / elem_max))
    return torch.exp2(e)


def mxfp4_fake_quantize(x: torch.Tensor) -> torch.Tensor:
    """1×32 blocks along the last dim, power-of-two scale, e2m1 elements (±{0, .5, 1, 1.5, 2, 3, 4, 6})."""
    shape = x.shape
    pad = (-shape[-1]) % BLOCK
    xf = torch.nn.functional.pad(x.float(), (0, pad)) if pad else x.float()
    blocks = xf.reshape(*xf.shape[:-1], -1, BLOCK)
    s = _pow2_scale(blocks.abs().amax(-1, keepdim=True), 6.0)
    v = blocks / s
    grid = _E2M1_GRID.to(v.device)
    idx = (v.abs().unsqueeze(-1) - grid).abs().argmin(-1)
    out = (grid[idx] * v.sign() * s).reshape(xf.shape)
    return out[..., : shape[-1]].to(x.dtype)


def block_fp8_fake_quantize(w: torch.Tensor, block: int = 32, mxfp4_prepass: bool = False) -> torch.Tensor:
    """32×32 blocks over the last two dims, one power-of-two scale per block, e4m3 elements."""
    if mxfp4_prepass:
        w = mxfp4_fake_quantize(w)
    *lead, r, c = w.shape
    pr, pc = (-r) % block, (-c) % block
    wf = torch.nn.functional.pad(w.float(), (0, pc, 0, pr))
    R, C = wf.shape[-2:]
    tiles = wf.reshape(*lead, R // block, block, C // block, block)
    s = _pow2_scale(tiles.abs().amax(dim=(-3, -1), keepdim=True), E4M3_MAX)
    q = (tiles / s).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn).float() * s
    return q.reshape(*lead, R, C)[..., :r, :c].to(w.dtype)


@dataclass(kw_only=True)
class QuantizeConfig:
    kind: str = "fp8_rowwise"  # fp8_rowwise | mx | block_fp8 | mxfp4
    round_mode: str = "rceil"
    block_size: int = 32
    mxfp4_prepass: bool = False


def fake_quantize(x: torch.Tensor, cfg: QuantizeConfig) -> torch.Tensor:
    if x.numel() == 0:
        return x
    if cfg.kind == "fp8_rowwise":
        return fp8_rowwise_fake_quantize(x)
    if cfg.kind == "mx":
        pad = (-x.shape[-1]) % BLOCK
        xp = torch.nn.functional.pad(x, (0, pad)) if pad else x
        out = mx_fake_quantize(xp.reshape(-1, xp.shape[-1]).contiguous(), -1, cfg.round_mode).reshape(xp.shape)
        return out[..., : x.shape[-1]]
    if cfg.kind == "block_fp8":
        return block_fp8_fake_quantize(x, cfg.block_size, cfg.mxfp4_prepass)
    if cfg.kind == "mxfp4":
        return mxfp4_fake_quantize(x)
    raise ValueError(f"unknown quantiser {cfg.kind!r}")


class _STE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cfg):
        return fake_quantize(x, cfg)

    @staticmethod
    def backward(ctx, g):
        return g, None


class FakeQuantParam(nn.Module):
    def __init__(self, cfg: QuantizeConfig):
        super().__init__()
        self.cfg = cfg

    def forward(self, w):
        local = w.to_local() if hasattr(w, "to_local") else w
        out = _STE.apply(local, self.cfg)
        if hasattr(w, "to_local"):
            from torch.distributed.tensor import DTensor

            return DTensor.from_local(out, w.device_mesh, w.placements, run_check=False)
        return out


@dataclass(kw_only=True)
class ParamSwapConfig:
    step: str = "prepare"  # prepare | convert
    weight_config: QuantizeConfig = field(default_factory=QuantizeConfig)
    activation_config: QuantizeConfig | None = None
    params_filter_fn: Callable[..., bool] | None = None
    """(fully qualified parameter name, parameter[, owning module]) → quantise it?  Default: every ≥2-D ``weight`` /
    expert matrix outside embeddings, norms and the output projection."""
    compute: str = "fake"  # fake: quantise-dequantise + bf16 GEMM | real: block-scaled FP8 GEMMs (mx, block_fp8)


def _default_filter(name: str, p: nn.Parameter) -> bool:
    leaf = name.rsplit(".", 1)[-1]
    if p.dim() < 2 or any(t in name for t in ("tok_embeddings", "norm", "output.")):
        return False
    return leaf in ("weight", "w1", "w2", "w3", "w13")


def _local(t):
    return t.to_local() if t is not None and hasattr(t, "to_local") else t


def _install_real(mod: nn.Module, wcfg: QuantizeConfig) -> bool:
    """Route ``mod``'s own GEMMs through real low-precision kernels; False when the module type has no such form."""
    import types

    from titan_b200.lowp.block_fp8 import block_fp8_grouped_mm, block_fp8_linear
    from titan_b200.lowp.mx_linear import mx_grouped_mm, mx_linear

    rm, pre = wcfg.round_mode, wcfg.mxfp4_prepass
    if isinstance(mod, nn.Linear):
        if wcfg.kind == "mx":
            fwd = lambda self_, x: mx_linear(x, _local(self_.weight), _local(self_.bias), rm)  # noqa: E731
        else:
            fwd = lambda self_, x: block_fp8_linear(x, _local(self_.weight), _local(self_.bias), round_mode=rm,  # noqa: E731
                                                    mxfp4_prepass=pre)
        mod._lowp_plain_forward = mod.__dict__.get("forward")
        mod.forward = types.MethodType(fwd, mod)
    elif hasattr(mod, "w2") and (hasattr(mod, "w13") or hasattr(mod, "w1")) and hasattr(mod, "num_experts"):
        mod.mx_round_mode = rm  # grouped experts consult this flag and call the function stored beside it
        if wcfg.kind == "mx":
            mod.mx_grouped_mm = mx_grouped_mm
        else:
            mod.mx_grouped_mm = lambda x, w, offs, r, aligned=False: block_fp8_grouped_mm(  # noqa: E731
                x, w, offs, round_mode=r, mxfp4_prepass=pre)
    else:
        return False
    mod._lowp_real = wcfg
    return True


def _remove_real(mod: nn.Module) -> list[str]:
    """Bake the quantised values into the weights of a module converted by `_install_real` and restore its forward."""
    wcfg = mod._lowp_real
    names = []
    with torch.no_grad():
        for pname, p in mod.named_parameters(recurse=False):
            if p.dim() >= 2:
                local = _local(p)
                local.copy_(fake_quantize(local, wcfg))
                names.append(pname)
    if isinstance(mod, nn.Linear):
        if mod.__dict__.get("_lowp_plain_forward") is None:
            mod.__dict__.pop("forward", None)
        else:
            mod.forward = mod._lowp_plain_forward
        mod.__dict__.pop("_lowp_plain_forward", None)
    else:
        for attr in ("mx_round_mode", "mx_grouped_mm"):
            mod.__dict__.pop(attr, None)
    del mod._lowp_real
    return names


def quantize_params(model: nn.Module, cfg: ParamSwapConfig) -> list[str]:
    """Install (``prepare``) or bake-and-remove (``convert``) the quantising wrappers; returns the affected names."""
    from titan_b200.lowp.filters import call_filter

    user = cfg.params_filter_fn
    if cfg.compute not in ("fake", "real"):
        raise ValueError(f"ParamSwapConfig.compute must be 'fake' or 'real', got {cfg.compute!r}")
    if cfg.compute == "real" and cfg.weight_config.kind not in ("mx", "block_fp8"):
        raise ValueError("compute='real' exists for the 'mx' and 'block_fp8' quantisers")
    touched = []
    for mod_name, mod in list(model.named_modules()):
        keep = (lambda fq, p, _m=mod: call_filter(user, fq, p, _m)) if user is not None else _default_filter
        if cfg.step == "convert" and hasattr(mod, "_lowp_real"):
            touched += [f"{mod_name}.{n}" if mod_name else n for n in _remove_real(mod)]
            continue
        if cfg.step == "prepare" and cfg.compute == "real":
            own = [(n, p) for n, p in mod.named_parameters(recurse=False)
                   if keep(f"{mod_name}.{n}" if mod_name else n, p)]
            if own and not hasattr(mod, "_lowp_real") and _install_real(mod, cfg.weight_config):
                # the module's forward is what changes, so every matrix it owns now runs (and is later baked) in low
                # precision, not only the ones the filter named
                touched += [f"{mod_name}.{n}" if mod_name else n
                            for n, p in mod.named_parameters(recurse=False) if p.dim() >= 2]
            continue
        for pname, p in list(mod.named_parameters(recurse=False)):
            fq = f"{mod_name}.{pname}" if mod_name else pname
            if cfg.step == "prepare":
                if parametrize.is_parametrized(mod, pname) or not keep(fq, p):
                    continue
                parametrize.register_parametrization(mod, pname, FakeQuantParam(cfg.weight_config), unsafe=True)
                touched.append(fq)
        if cfg.step == "convert" and parametrize.is_parametrized(mod):
            for pname in list(mod.parametrizations.keys()):
                if any(isinstance(f, FakeQuantParam) for f in mod.parametrizations[pname]):
                    parametrize.remove_parametrizations(mod, pname, leave_parametrized=True)
                    touched.append(f"{mod_name}.{pname}" if mod_name else pname)
        if cfg.step == "prepare" and cfg.activation_config is not None and isinstance(mod, nn.Linear) \
                and parametrize.is_parametrized(mod, "weight") and not hasattr(mod, "_act_fq_hook"):
            acfg = cfg.activation_config
            mod._act_fq_hook = mod.register_forward_pre_hook(lambda m, args, _c=acfg: (_STE.apply(args[0], _c), *args[1:]))
    if cfg.step not in ("prepare", "convert"):
        raise ValueError(f"ParamSwapConfig.step must be 'prepare' or 'convert', got {cfg.step!r}")
    return touched


@dataclass(kw_only=True)
class QuantizeConverterConfig:
    base_config: ParamSwapConfig = field(default_factory=ParamSwapConfig)
    filter_fn: Callable[[str, nn.Parameter], bool] | None = None
    name: str = "quantize"

    def build(self, **kwargs):
        return QuantizeConverter(self, **kwargs)


class QuantizeConverter(ModelConverter):
    """Model-converter face of `quantize_params` (recipes list it after the kernel converters)."""

    def __init__(self, config: QuantizeConverterConfig | None = None, *, model_spec=None, trainer_config=None, **kw):
        super().__init__(model_spec=model_spec, trainer_config=trainer_config)
        self.config = config or QuantizeConverterConfig()

    def convert(self, model: nn.Module) -> None:
        base = self.config.base_config
        if self.config.filter_fn is not None:
            base = ParamSwapConfig(step=base.step, weight_config=base.weight_config, compute=base.compute,
                                   activation_config=base.activation_config, params_filter_fn=self.config.filter_fn)
        self.converted = quantize_params(model, base)
        if not self.converted:
            raise ValueError("the quantize converter matched no parameter")
