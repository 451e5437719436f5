"""`b200_flash_attention` (alias `npu_flash_attention`): dense causal attention cores → the tcgen05 forward kernel.

Every `ScaledDotProductAttention` core of the model is swapped for `FlashAttentionCore`; calls the kernel does not
cover (explicit masks, other head sizes, ragged lengths) stay on the library path inside the op.

Parity: the reference routes attention to its fused op through the attention wrapper (K7); this is the opt-in
counterpart here.  Not part of the default recipes while the library's Blackwell kernel is faster (see profiles/).
"""

from titan_b200.converters.convert_utils import replace_modules
from titan_b200.models.common.layers import ScaledDotProductAttention
from titan_b200.ops.flash_attention import flash_attention
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class FlashAttentionCore(ScaledDotProductAttention):
    def forward(self, q, k, v, *, scale=None, attn_mask=None):
        if attn_mask is not None or not self.causal:
            return super().forward(q, k, v, scale=scale, attn_mask=attn_mask)
        return flash_attention(q, k, v, scale=scale)


def _swap(old):
    new = FlashAttentionCore.__new__(FlashAttentionCore)
    new.__dict__ = old.__dict__
    return new


class FlashAttentionConverter(ModelConverter):
    def convert(self, model) -> None:
        self.replaced = replace_modules(model, r"^ScaledDotProductAttention$", _swap)


FLASH = register_model_converter("b200_flash_attention", "npu_flash_attention")(
    ConverterSpec(model_converter=FlashAttentionConverter))
