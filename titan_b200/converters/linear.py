"""`b200_linear`: every bias-free `Linear` runs on the hand-written tcgen05 GEMM
(`csrc/gemm/gemm_bf16.cu`) for forward, input-gradient and weight-gradient.

Modules whose FQN matches an entry of the ``skip`` option keep the library GEMM
(e.g. ``skip=["output"]`` for a vocabulary head with ragged shapes).
"""

import torch

from titan_b200.models.common.layers import Linear
from titan_b200.ops.gemm import linear as tc_linear
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class TcLinear(Linear):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight
        if hasattr(w, "to_local") or hasattr(x, "to_local"):
            return torch.nn.functional.linear(x, w, self.bias)  # DTensor (TP) path stays on the library
        return tc_linear(x, w, self.bias)


class LinearConverter(ModelConverter):
    options: dict = {}

    def convert(self, model) -> None:
        skip = tuple(self.options.get("skip", ()))
        self.replaced = 0
        for name, mod in list(model.named_modules()):
            if type(mod) is Linear and not any(s in name for s in skip):
                mod.__class__ = TcLinear
                self.replaced += 1


LINEAR = register_model_converter("b200_linear")(ConverterSpec(model_converter=LinearConverter))
