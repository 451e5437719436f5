"""Llama-3 native ↔ Hugging Face parameter mapping.

HF stores q/k projections for the half-rotate RoPE layout; this model rotates
interleaved pairs, so wq/wk rows are permuted per head on the way in and out.
"""

from __future__ import annotations

from typing import Any

import torch

from titan_b200.protocols.state_dict_adapter import StateDictAdapter

__all__ = ["Llama3StateDictAdapter"]


class Llama3StateDictAdapter(StateDictAdapter):
    from_hf_map = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.wq.weight",
        "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.wk.weight",
        "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.wv.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.self_attn.rotary_emb.inv_freq": None,
        "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
        "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
        "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "output.weight",
    }

    def _heads(self, key: str) -> int:
        c = self.model_config
        return c.n_heads if key.endswith("wq.weight") else (c.n_kv_heads or c.n_heads)

    @staticmethod
    def _permute(w: torch.Tensor, n_heads: int) -> torch.Tensor:
        # native (interleaved) → HF (half-rotate)
        d1, d2 = w.shape
        return w.view(n_heads, d1 // n_heads // 2, 2, d2).transpose(1, 2).reshape(d1, d2)

    @staticmethod
    def _reverse_permute(w: torch.Tensor, n_heads: int) -> torch.Tensor:
        d1, d2 = w.shape
        return w.view(n_heads, 2, d1 // n_heads // 2, d2).transpose(1, 2).reshape(d1, d2)

    def _to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        sd = {}
        for k, v in state_dict.items():
            if k.endswith(("attention.wq.weight", "attention.wk.weight")):
                v = self._permute(v, self._heads(k))
            sd[k] = v
        return super()._to_hf(sd)

    def _from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        sd = super()._from_hf(hf_state_dict)
        for k in list(sd):
            if k.endswith(("attention.wq.weight", "attention.wk.weight")):
                sd[k] = self._reverse_permute(sd[k], self._heads(k))
        return sd
