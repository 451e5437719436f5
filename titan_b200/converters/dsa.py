"""`b200_dsa` (alias `npu_dsa`): the eager sparse-attention oracle → the fused DSA path.

`DSASparseAttention.forward` is replaced by: lightning-indexer top-k (tcgen05 scoring kernel with a fused
relu·weight·head-sum epilogue + radix-select kernel, no gradient) → sparse attention over the selected rows
of the shared KV latent (long key streams: the gathered-tile tcgen05 kernel `csrc/attention/sparse_mla_fwd.cu`; short
ones: one masked GEMM) → KL indexer loss from the head-summed attention mass and the index scores
re-evaluated at the selected keys only.  Cost drops from O(S²·H) to O(S·k·H) and no [S, S] tensor exists.

Parity: torchtitan_npu/converters/kernels/dsa.py:195-304 (v3.2 only).
"""

from titan_b200.converters.convert_utils import replace_modules
from titan_b200.models.deepseek_v32.model import DSASparseAttention
from titan_b200.ops.dsa import dsa_attention
from titan_b200.protocols.converter import ConverterSpec, ModelConverter, register_model_converter


class FusedDSAttention(DSASparseAttention):
    cp_layout = "dsa"

    def forward(self, q, k, v, attn_mask=None, scale=None, q_indexer=None, k_indexer=None, weights=None,
                index_topk=None):
        if q_indexer is None or attn_mask is not None:
            return super().forward(q, k, v, attn_mask, scale, q_indexer, k_indexer, weights, index_topk)
        scale = scale if scale is not None else q.shape[-1] ** -0.5
        prefix = getattr(self, "_values_are_key_prefix", None)
        if prefix is None and k.shape[1] == 1 and (q.is_cuda or q.is_meta):
            from titan_b200.ops.dsa import _values_are_key_prefix

            # MLA absorb: the values are the latent part of the keys; decided once per module (a layout property)
            prefix = self._values_are_key_prefix = _values_are_key_prefix(k, v)
        return dsa_attention(q, k, v, scale=scale, q_indexer=q_indexer, k_indexer=k_indexer, weights=weights,
                             index_topk=index_topk or k.shape[2], values_are_key_prefix=prefix)


def _swap(old):
    new = FusedDSAttention.__new__(FusedDSAttention)
    new.__dict__ = old.__dict__
    return new


class DSAConverter(ModelConverter):
    def convert(self, model) -> None:
        if self.model_name not in (None, "deepseek_v32"):
            raise ValueError("b200_dsa applies to deepseek_v32 models only")
        self.replaced = replace_modules(model, r"DSASparseAttention", _swap)


DSA = register_model_converter("b200_dsa", "npu_dsa")(ConverterSpec(model_converter=DSAConverter))
