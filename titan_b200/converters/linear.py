"""`b200_linear`: every bias-free `Linear` runs on the hand-written tcgen05 GEMMs (`csrc/gemm/gemm_pair.cuh` for
problems that fill the GPU, `csrc/gemm/gemm_bf16.cu` for small ones) for forward, input-gradient and weight-gradient.

Under tensor parallelism the weight is a DTensor shard and the module is wrapped by a column- or row-parallel style;
the forward then multiplies the LOCAL shards on the same kernels and hands back a DTensor in the layout the style
expects (`Shard(-1)` for a column shard, `Partial()` for a row shard), so nothing falls back to the library GEMM.
Layouts it does not know keep the DTensor dispatch path.

Modules whose FQN matches an entry of the ``skip`` option keep the library GEMM.
"""

import torch
from torch.distributed.tensor import DTensor, Partial, Replicate, Shard

from titan_b200.models.common.layers import Linear
from titan_b200.ops.gemm import linear as tc_linear
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


def _is_last_dim_shard(pl, ndim: int) -> bool:
    return isinstance(pl, Shard) and pl.dim in (-1, ndim - 1)


def dtensor_local_linear(x, w: DTensor, bias):
    """``x @ w.T`` for a tensor-parallel weight shard on the local shards; None when the layout is not covered."""
    if bias is not None or not isinstance(w, DTensor) or w.device_mesh.ndim != 1:
        return None
    mesh, (wp,) = w.device_mesh, w.placements
    if not isinstance(x, DTensor):
        return None
    if x.device_mesh != mesh or len(x.placements) != 1:
        return None
    (xp,) = x.placements
    if isinstance(wp, Shard) and wp.dim == 0 and isinstance(xp, Replicate):
        # column shard: every rank multiplies the full activations by its output features; the gradient of the
        # replicated input is a partial sum over the ranks
        y = tc_linear(x.to_local(grad_placements=(Partial(),)), w.to_local())
        return DTensor.from_local(y, mesh, (Shard(y.dim() - 1),), run_check=False)
    if isinstance(wp, Shard) and wp.dim == 1 and _is_last_dim_shard(xp, x.dim()):
        # row shard: local input features times the matching weight columns, a partial sum of the output
        y = tc_linear(x.to_local(), w.to_local())
        return DTensor.from_local(y, mesh, (Partial(),), run_check=False)
    return None


class TcLinear(Linear):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w = self.weight
        if isinstance(w, DTensor) or isinstance(x, DTensor):
            y = dtensor_local_linear(x, w, self.bias)
            if y is not None:
                return y
            return torch.nn.functional.linear(x, w, self.bias)  # other layouts: DTensor dispatch
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
