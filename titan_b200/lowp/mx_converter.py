"""`MXFP8Converter`: run the selected linears and grouped experts in MXFP8 (1×32 e8m0 block scales, e4m3 elements).

``fqns`` are substrings of module names; an `nn.Linear` whose name matches gets an MX forward / backward
(`mx_linear`), a grouped-experts module whose name matches routes its expert GEMMs through `mx_grouped_mm`.  Module
classes, parameters and their names stay as they are, so checkpoints, FSDP wrapping and tensor-parallel plans are
unaffected.  Dims that the block size does not divide are padded inside the op.  The converter must come after the
grouped-GEMM converter in a recipe (it patches the module that converter leaves behind) and refuses devices without
FP8 tensor cores.

Parity: the upstream `MXFP8Converter.Config(recipe_name, fqns)` as the reference uses it
(torchtitan_npu/models/deepseek_v4/config_registry.py:22-34,103-111; patches/torchao_npu/mx_capability_check.py:24-47;
docs/feature_guides/low_precision_training.md).
"""

from __future__ import annotations

import types
from dataclasses import dataclass, field

import torch
import torch.nn as nn

from titan_b200.lowp.mx_linear import mx_grouped_mm, mx_linear
from titan_b200.protocols.converter import ModelConverter
from titan_b200.utils.logging import logger

__all__ = ["MXFP8Converter", "MXFP8ConverterConfig", "RECIPES"]

RECIPES = {"mxfp8_rceil": "rceil", "mxfp8_floor": "floor"}


@dataclass(kw_only=True)
class MXFP8ConverterConfig:
    recipe_name: str = "mxfp8_rceil"
    fqns: list[str] = field(default_factory=list)
    """Module-name substrings to convert; empty = every linear except the output projection."""
    name: str = "mxfp8"

    def build(self, **kwargs):
        return MXFP8Converter(self, **kwargs)


def _capable() -> bool:
    if not torch.cuda.is_available():
        return True  # CPU runs use the PyTorch statement of the same numerics (tests, dry runs)
    major, _ = torch.cuda.get_device_capability()
    return major >= 10


class MXFP8Converter(ModelConverter):
    Config = MXFP8ConverterConfig  # recipes write ``MXFP8Converter.Config(recipe_name=..., fqns=[...])``

    def __init__(self, config: MXFP8ConverterConfig | None = None, *, model_spec=None, trainer_config=None, **kw):
        super().__init__(model_spec=model_spec, trainer_config=trainer_config)
        self.config = config or MXFP8ConverterConfig()
        if self.config.recipe_name not in RECIPES:
            raise ValueError(f"unknown MXFP8 recipe {self.config.recipe_name!r}; available: {sorted(RECIPES)}")
        if not _capable():
            raise RuntimeError("MXFP8 training needs a GPU with block-scaled FP8 tensor cores (compute capability 10.0)")
        self.round_mode = RECIPES[self.config.recipe_name]
        self.converted: list[str] = []

    def _match(self, name: str) -> bool:
        if self.config.fqns:
            return any(f in name for f in self.config.fqns)
        return not name.endswith("output")

    def convert(self, model: nn.Module) -> None:
        rm = self.round_mode
        for name, mod in model.named_modules():
            if not self._match(name):
                continue
            if isinstance(mod, nn.Linear):
                def fwd(self_, x, _rm=rm):
                    w = self_.weight
                    w = w.to_local() if hasattr(w, "to_local") else w
                    b = self_.bias
                    b = b.to_local() if b is not None and hasattr(b, "to_local") else b
                    return mx_linear(x, w, b, _rm)

                mod.forward = types.MethodType(fwd, mod)
                mod.mx_round_mode = rm
                self.converted.append(name)
            elif hasattr(mod, "w2") and (hasattr(mod, "w13") or hasattr(mod, "w1")) and hasattr(mod, "num_experts"):
                mod.mx_round_mode = rm  # grouped experts consult this flag and call `mx_grouped_mm`
                mod.mx_grouped_mm = mx_grouped_mm
                self.converted.append(name)
        if not self.converted:
            raise ValueError(f"MXFP8Converter matched no module (fqns={self.config.fqns})")
        logger.info("MXFP8 (%s): %d modules converted", self.config.recipe_name, len(self.converted))
