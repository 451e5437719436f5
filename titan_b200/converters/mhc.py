"""`b200_mhc_pre` / `b200_mhc_post` (aliases `npu_mhc_pre` / `npu_mhc_post`): hyper-connection kernels.

The hyper-connection math is a set of free functions (`ops.mhc`), so the converters only flip the dispatch switch:
on CUDA with bf16 streams `hc_pre` then runs as one kernel (RMS statistics + 24 mixing dot products + Sinkhorn +
stream collapse in a single pass over ``[T, 4, D]``) and `hc_post` as one kernel (``post·y + combᵀ·residual``).

Parity: torchtitan_npu/converters/kernels/mhc_prepost.py.
"""

from titan_b200.ops import mhc
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


def _check(model_name) -> None:
    if model_name not in (None, "deepseek_v4"):
        raise ValueError("the mHC converters apply to deepseek_v4 models only")


class MHCPreConverter(ModelConverter):
    def convert(self, model) -> None:
        _check(self.model_name)
        mhc.set_fused(pre=True)


class MHCPostConverter(ModelConverter):
    def convert(self, model) -> None:
        _check(self.model_name)
        mhc.set_fused(post=True)


MHC_PRE = register_model_converter("b200_mhc_pre", "npu_mhc_pre")(ConverterSpec(model_converter=MHCPreConverter))
MHC_POST = register_model_converter("b200_mhc_post", "npu_mhc_post")(ConverterSpec(model_converter=MHCPostConverter))
