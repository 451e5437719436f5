"""`b200_swiglu`: dense `FeedForward` blocks compute ``silu(w1 x) * w3 x`` with the fused kernel
(one pass instead of three elementwise launches; backward recomputes sigmoid instead of saving it).

The grouped-expert activation (clamp + routed score) is switched by `b200_gmm`; both use
`csrc/elementwise/swiglu.cu` (reference op: `npu_swiglu`, converters/kernels/gmm.py:87-104).
"""

import torch

from titan_b200.converters.convert_utils import replace_modules
from titan_b200.models.common.layers import FeedForward
from titan_b200.ops.swiglu import swiglu
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class FusedFeedForward(FeedForward):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w2(swiglu(self.w1(x), self.w3(x)))


def _swap(old: FeedForward) -> FusedFeedForward:
    new = FusedFeedForward.__new__(FusedFeedForward)
    new.__dict__ = old.__dict__
    return new


class SwiGLUConverter(ModelConverter):
    def convert(self, model) -> None:
        self.replaced = replace_modules(model, r"FeedForward", _swap)


SWIGLU = register_model_converter("b200_swiglu", "npu_swiglu")(ConverterSpec(model_converter=SwiGLUConverter))
