"""`b200_rms_norm` (alias `npu_rms_norm`): every `RMSNorm` → the fused sm_100a version.

The replacement shares the original's ``__dict__`` (parameters, hooks, FQNs stay identical, so
checkpoints and parallel plans are unaffected); a missing eps falls back to the dtype epsilon.

Parity: torchtitan_npu/converters/kernels/rms_norm.py:31-63.
"""

import torch

from titan_b200.converters.convert_utils import replace_modules
from titan_b200.models.common.layers import RMSNorm
from titan_b200.ops.norm import rms_norm
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class FusedRMSNorm(RMSNorm):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        eps = self.eps if self.eps is not None else torch.finfo(x.dtype).eps
        w = self.weight
        if hasattr(w, "to_local"):  # sequence-parallel norm: weight is a replicated DTensor
            from titan_b200.parallel.tensor_parallel import norm_weight_local

            w = norm_weight_local(w, x)
        if hasattr(x, "to_local"):
            from torch.distributed.tensor import DTensor

            y = rms_norm(x.to_local(), w, eps)
            return DTensor.from_local(y, x.device_mesh, x.placements, run_check=False)
        return rms_norm(x, w, eps)


def _swap(old: RMSNorm) -> FusedRMSNorm:
    new = FusedRMSNorm.__new__(FusedRMSNorm)
    new.__dict__ = old.__dict__
    return new


class RMSNormConverter(ModelConverter):
    def convert(self, model) -> None:
        self.replaced = replace_modules(model, r"RMSNorm", _swap)


RMS_NORM = register_model_converter("b200_rms_norm", "npu_rms_norm")(ConverterSpec(model_converter=RMSNormConverter))
