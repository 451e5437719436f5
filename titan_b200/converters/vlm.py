"""`b200_vlm` (alias `npu_vlm`): the explicit opt-in the VLM recipe must carry.

The dense-mask attention cores of both towers are chosen when the model is built; the converter checks that they are
in place (and is the hook where a fused masked-attention kernel replaces them).

Parity: torchtitan_npu/converters/features/vlm.py.
"""

from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class VLMConverter(ModelConverter):
    def convert(self, model) -> None:
        if self.model_name not in (None, "vlm"):
            raise ValueError("b200_vlm applies to vlm models only")
        from titan_b200.models.multimodal import DenseMaskSDPA

        cores = [m for m in model.modules() if isinstance(m, DenseMaskSDPA)]
        if not cores:
            raise ValueError("b200_vlm found no dense-mask attention core in the model")
        self.replaced = len(cores)


VLM = register_model_converter("b200_vlm", "npu_vlm")(ConverterSpec(model_converter=VLMConverter))
