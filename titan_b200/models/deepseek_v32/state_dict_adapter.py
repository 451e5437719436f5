"""DeepSeek-V3.2 native ↔ Hugging Face mapping (three-stage attention, indexer, MTP layers).

Parity: torchtitan_npu/models/deepseek_v32/state_dict_adapter.py:32-120.
"""

from __future__ import annotations

import re
from typing import Any

from titan_b200.models.deepseek_v3.state_dict_adapter import DeepSeekV3StateDictAdapter

__all__ = ["DeepSeekV32StateDictAdapter"]

_A = "layers.{}.attention.pre_attention."


class DeepSeekV32StateDictAdapter(DeepSeekV3StateDictAdapter):
    from_hf_map = {k: v for k, v in DeepSeekV3StateDictAdapter.from_hf_map.items() if ".self_attn." not in k}
    from_hf_map.update({
        "model.layers.{}.self_attn.q_a_proj.weight": _A + "wq_a.weight",
        "model.layers.{}.self_attn.q_a_layernorm.weight": _A + "q_norm.weight",
        "model.layers.{}.self_attn.q_b_proj.weight": _A + "wq_b.weight",
        "model.layers.{}.self_attn.kv_a_proj_with_mqa.weight": _A + "wkv_a.weight",
        "model.layers.{}.self_attn.kv_a_layernorm.weight": _A + "kv_norm.weight",
        "model.layers.{}.self_attn.kv_b_proj.weight": _A + "wkv_b.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.post_attention.wo.weight",
        "model.layers.{}.self_attn.indexer.wq_b.weight": _A + "indexer.wq_b.weight",
        "model.layers.{}.self_attn.indexer.wk.weight": _A + "indexer.wk.weight",
        "model.layers.{}.self_attn.indexer.k_norm.weight": _A + "indexer.k_norm.weight",
        "model.layers.{}.self_attn.indexer.k_norm.bias": _A + "indexer.k_norm.bias",
        "model.layers.{}.self_attn.indexer.weights_proj.weight": _A + "indexer.weights_proj.weight",
        "model.layers.{}.enorm.weight": "layers.{}.enorm.weight",
        "model.layers.{}.hnorm.weight": "layers.{}.hnorm.weight",
        "model.layers.{}.eh_proj.weight": "layers.{}.eh_proj.weight",
        "model.layers.{}.shared_head.norm.weight": "layers.{}.norm.weight",
    })

    def _mtp_to_layer(self, key: str) -> str:
        """``mtp_layers.i.block.X`` / ``mtp_layers.i.X`` → ``layers.(n_layers+i).X`` (HF numbers MTP depths as layers)."""
        m = re.match(r"^mtp_layers\.(\d+)\.(block\.)?(.*)$", key)
        if not m:
            return key
        return f"layers.{self.model_config.n_layers + int(m.group(1))}.{m.group(3)}"

    def _layer_to_mtp(self, key: str) -> str:
        m = re.match(r"^layers\.(\d+)\.(.*)$", key)
        if not m or int(m.group(1)) < self.model_config.n_layers:
            return key
        i, rest = int(m.group(1)) - self.model_config.n_layers, m.group(2)
        own = rest.split(".")[0] in ("enorm", "hnorm", "eh_proj", "norm")
        return f"mtp_layers.{i}.{rest}" if own else f"mtp_layers.{i}.block.{rest}"

    def _to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        return super()._to_hf({self._mtp_to_layer(k): v for k, v in state_dict.items()})

    def _from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        return {self._layer_to_mtp(k): v for k, v in super()._from_hf(hf_state_dict).items()}
