"""`b200_rope` (alias `npu_rope`): route every rotary-embedding call to the sm_100a kernel.

Rebinds `apply_rotary_emb_complex / _single_complex / _cos_sin` in every module that imported
them (including stale ``from … import`` bindings).  The replacements fall back to the PyTorch
oracle for CPU tensors, so the rebinding is safe in CPU dry runs.

Parity: torchtitan_npu/converters/kernels/rope.py:240-281.
"""

from titan_b200.converters.convert_utils import replace_functions
from titan_b200.models.common import rope as base
from titan_b200.ops import rope as fused
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter

_ORIGINALS = {
    "apply_rotary_emb_complex": base.apply_rotary_emb_complex,
    "apply_rotary_emb_single_complex": base.apply_rotary_emb_single_complex,
    "apply_rotary_emb_cos_sin": base.apply_rotary_emb_cos_sin,
}


class RopeConverter(ModelConverter):
    def convert(self, model) -> None:
        self.replaced = 0
        for name, old in _ORIGINALS.items():
            # the oracle module keeps its own definitions: the fused path calls them on CPU
            self.replaced += replace_functions(old, getattr(fused, name),
                                               skip_modules=("titan_b200.models.common.rope", "titan_b200.ops.rope",
                                                             "titan_b200.converters.rope"))


def restore() -> None:
    """Undo the rebinding (tests use this to compare fused and baseline paths in one process)."""
    for name, old in _ORIGINALS.items():
        replace_functions(getattr(fused, name), old, skip_modules=("titan_b200.ops.rope",))


ROPE = register_model_converter("b200_rope", "npu_rope")(ConverterSpec(model_converter=RopeConverter))
