"""Qwen3 native ↔ Hugging Face mapping (dense and MoE; tied embeddings have no ``lm_head`` entry).

The rotary layout is half-rotate on both sides, so projections map without permutation.

Parity: the upstream `Qwen3StateDictAdapter` that the reference registers (torchtitan_npu/models/qwen3/__init__.py:26).
"""

from __future__ import annotations

from typing import Any

from titan_b200.models.deepseek_v3.state_dict_adapter import MoEStateDictAdapter

__all__ = ["Qwen3StateDictAdapter"]


class Qwen3StateDictAdapter(MoEStateDictAdapter):
    from_hf_map = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.wq.weight",
        "model.layers.{}.self_attn.k_proj.weight": "layers.{}.attention.wk.weight",
        "model.layers.{}.self_attn.v_proj.weight": "layers.{}.attention.wv.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.self_attn.q_norm.weight": "layers.{}.attention.q_norm.weight",
        "model.layers.{}.self_attn.k_norm.weight": "layers.{}.attention.k_norm.weight",
        "model.layers.{}.self_attn.rotary_emb.inv_freq": None,
        "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
        "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
        "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
        "model.layers.{}.mlp.gate.weight": "layers.{}.moe.router.gate.weight",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "output.weight",
    }

    def _to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        sd = {k: v for k, v in state_dict.items() if not k.endswith("moe.expert_bias")}  # HF has no balancing bias
        out = super()._to_hf(sd)
        if getattr(self.model_config, "enable_weight_tying", False):
            out.pop("lm_head.weight", None)
        return out

    def _from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        out = super()._from_hf(hf_state_dict)
        if getattr(self.model_config, "enable_weight_tying", False) and "output.weight" not in out:
            out["output.weight"] = out["tok_embeddings.weight"]
        return out
