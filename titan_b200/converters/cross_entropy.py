"""`b200_cross_entropy`: the loss is computed by the fused softmax cross-entropy kernel.

Nothing in the model changes; `build_cross_entropy_loss` looks for this converter in the recipe and
returns the fused loss.  The fused loss reads bf16 logits directly (no fp32 copy of the [T, V]
matrix) and may write the logits gradient in place.
"""

from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class CrossEntropyConverter(ModelConverter):
    def convert(self, model) -> None:
        return None


CROSS_ENTROPY = register_model_converter("b200_cross_entropy")(ConverterSpec(model_converter=CrossEntropyConverter))
