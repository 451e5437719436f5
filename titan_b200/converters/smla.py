"""`b200_smla` (alias `npu_smla`): DeepSeek-V4 attention core → chunked sparse path with fused selection.

`InnerAttention` keeps its parameters (`attn_sink`); only its two hooks are set:
* ``core``   – `ops.smla.smla_attention`: sliding window ∪ selected compressed keys ∪ sink without any ``S × T``
  tensor, returning the indexer's teacher distribution from the same pass;
* ``select`` – `ops.smla.li_select`: tcgen05 index scoring + radix top-k over compressed keys.

Parity: torchtitan_npu/converters/kernels/npu_smla.py (v4 only).
"""

from functools import partial

from titan_b200.ops.smla import li_select, smla_attention
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class SMLAConverter(ModelConverter):
    def convert(self, model) -> None:
        if self.model_name not in (None, "deepseek_v4"):
            raise ValueError("b200_smla applies to deepseek_v4 models only")
        from titan_b200.models.deepseek_v4.model import InnerAttention

        self.replaced = 0
        for mod in model.modules():
            if isinstance(mod, InnerAttention):
                mod.core = partial(smla_attention, n_heads_total=mod.n_heads)
                mod.select = li_select
                mod.cp_layout = "compressor"
                self.replaced += 1
        if self.replaced == 0:
            raise ValueError("b200_smla found no DeepSeek-V4 attention core in the model")


SMLA = register_model_converter("b200_smla", "npu_smla")(ConverterSpec(model_converter=SMLAConverter))
