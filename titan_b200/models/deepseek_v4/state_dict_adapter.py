"""DeepSeek-V4 native ↔ released-checkpoint mapping.

Checkpoint conventions handled here:
* attention parameters live under ``layers.N.attn.*``; both compressors are called ``attn.compressor`` there while the
  model names them ``compressor`` (ratio 4) or ``compressor_128`` (any other ratio > 1);
* experts are stored one tensor per expert (``layers.N.ffn.experts.E.w1.weight``) and stacked ``[E, ...]`` natively;
* the load-balancing bias is ``ffn.gate.bias``; hash-routed layers store their table ``ffn.gate.tid2eid`` as fp32;
* the final stream-collapsing head is stored at the root (``hc_head_*``) and lives in the last main block natively;
* MTP depth ``i`` is stored as ``mtp.i.*`` and is native layer ``n_layers + i`` (its norm / head are ``norm`` /
  ``hc_head_*`` inside that prefix).

Parity: torchtitan_npu/models/deepseek_v4/state_dict_adapter.py:29-364.
"""

from __future__ import annotations

import re
from typing import Any

import torch

from titan_b200.models.deepseek_v3.state_dict_adapter import MoEStateDictAdapter
from titan_b200.protocols.state_dict_adapter import StateDictAdapter

__all__ = ["DeepSeekV4StateDictAdapter"]

_PRE, _POST, _INNER = "attention.pre_attention.", "attention.post_attention.", "attention.inner_attention."

# suffix inside ``layers.N.`` : checkpoint → native
_LAYER_MAP = {
    "attn.attn_sink": _INNER + "attn_sink",
    "attn.kv_norm.weight": _PRE + "kv_norm.weight",
    "attn.q_norm.weight": _PRE + "q_norm.weight",
    "attn.wkv.weight": _PRE + "wkv.weight",
    "attn.wq_a.weight": _PRE + "wq_a.weight",
    "attn.wq_b.weight": _PRE + "wq_b.weight",
    "attn.wo_a.weight": _POST + "wo_a.weight",
    "attn.wo_b.weight": _POST + "wo_b.weight",
    "attn.indexer.wq_b.weight": _PRE + "indexer.wq_b.weight",
    "attn.indexer.weights_proj.weight": _PRE + "indexer.weights_proj.weight",
    "attn_norm.weight": "attention_norm.weight",
    "ffn_norm.weight": "ffn_norm.weight",
    "ffn.gate.weight": "moe.router.gate.weight",
    "ffn.gate.bias": "moe.expert_bias",
    "ffn.gate.tid2eid": "moe.router.tid2eid",
    "ffn.shared_experts.w1.weight": "moe.shared_experts.w1.weight",
    "ffn.shared_experts.w2.weight": "moe.shared_experts.w2.weight",
    "ffn.shared_experts.w3.weight": "moe.shared_experts.w3.weight",
    "enorm.weight": "enorm.weight",
    "hnorm.weight": "hnorm.weight",
    "e_proj.weight": "e_proj.weight",
    "h_proj.weight": "h_proj.weight",
}
for _p in ("hc_attn_base", "hc_attn_fn", "hc_attn_scale", "hc_ffn_base", "hc_ffn_fn", "hc_ffn_scale"):
    _LAYER_MAP[_p] = _p
_COMPRESSOR_PARTS = ("ape", "norm.weight", "wgate.weight", "wkv.weight")
_ROOT_MAP = {"embed.weight": "tok_embeddings.weight", "norm.weight": "norm.weight", "head.weight": "output.weight"}
_HEAD = ("hc_head_fn", "hc_head_base", "hc_head_scale")
_EXPERT_CKPT = re.compile(r"^ffn\.experts\.(\d+)\.(w1|w2|w3)\.weight$")
_EXPERT_NATIVE = re.compile(r"^moe\.experts\.(w1|w2|w3)$")


class DeepSeekV4StateDictAdapter(StateDictAdapter):
    def _ratio(self, layer: int) -> int:
        c = self.model_config
        return c.compress_ratios[layer] if layer < c.n_layers else c.mtp_layer_compress_ratio

    def _compressor_name(self, layer: int) -> str:
        return "compressor" if self._ratio(layer) == 4 else "compressor_128"

    # ---------------------------------------------------------------------------------------------- native → ckpt
    def _suffix_to_ckpt(self, layer: int, suffix: str, is_mtp: bool) -> str:
        inv = {v: k for k, v in _LAYER_MAP.items()}
        if suffix in inv:
            return inv[suffix]
        m = re.match(r"^attention\.pre_attention\.(indexer\.)?(compressor(?:_128)?)\.(.+)$", suffix)
        if m and m.group(3) in _COMPRESSOR_PARTS:
            return f"attn.{m.group(1) or ''}compressor.{m.group(3)}"
        if is_mtp and suffix == "mtp_norm.weight":
            return "norm.weight"
        if is_mtp and suffix.startswith("mtp_hc_head."):
            return suffix[len("mtp_hc_head."):]
        raise KeyError(f"no checkpoint name for layer parameter {suffix!r}")

    def _to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        n_layers = self.model_config.n_layers
        inv_root = {v: k for k, v in _ROOT_MAP.items()}
        out: dict[str, Any] = {}
        for key, value in state_dict.items():
            m = re.match(r"^layers\.(\d+)\.(.+)$", key)
            if not m:
                out[inv_root[key]] = value
                continue
            layer, suffix = int(m.group(1)), m.group(2)
            is_mtp = layer >= n_layers
            prefix = f"mtp.{layer - n_layers}." if is_mtp else f"layers.{layer}."
            if suffix.startswith("hc_head.") and not is_mtp:
                out[suffix[len("hc_head."):]] = value  # stored at the root
                continue
            em = _EXPERT_NATIVE.match(suffix)
            if em:
                first, n, local = MoEStateDictAdapter._local_expert_range(value)
                for e in range(n):
                    out[f"{prefix}ffn.experts.{first + e}.{em.group(1)}.weight"] = local[e]
                continue
            if suffix.endswith("tid2eid"):
                value = value.to(torch.float32)
            out[prefix + self._suffix_to_ckpt(layer, suffix, is_mtp)] = value
        return out

    # ---------------------------------------------------------------------------------------------- ckpt → native
    def _suffix_to_native(self, layer: int, suffix: str, is_mtp: bool) -> str:
        if suffix in _LAYER_MAP:
            return _LAYER_MAP[suffix]
        m = re.match(r"^attn\.(indexer\.)?compressor\.(.+)$", suffix)
        if m and m.group(2) in _COMPRESSOR_PARTS:
            name = "compressor" if m.group(1) else self._compressor_name(layer)
            return f"{_PRE}{m.group(1) or ''}{name}.{m.group(2)}"
        if is_mtp and suffix == "norm.weight":
            return "mtp_norm.weight"
        if is_mtp and suffix in _HEAD:
            return "mtp_hc_head." + suffix
        raise KeyError(f"no native name for checkpoint parameter {suffix!r}")

    def _from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        n_layers = self.model_config.n_layers
        out: dict[str, Any] = {}
        experts: dict[tuple[int, str], dict[int, Any]] = {}
        for key, value in hf_state_dict.items():
            if key.endswith(".scale") or key.endswith(".weight_scale_inv"):
                continue  # block scales of a quantised export; the loader dequantises before this point
            m = re.match(r"^(layers|mtp)\.(\d+)\.(.+)$", key)
            if not m:
                if key in _HEAD:
                    out[f"layers.{n_layers - 1}.hc_head.{key}"] = value
                else:
                    out[_ROOT_MAP[key]] = value
                continue
            is_mtp = m.group(1) == "mtp"
            layer = int(m.group(2)) + (n_layers if is_mtp else 0)
            suffix = m.group(3)
            em = _EXPERT_CKPT.match(suffix)
            if em:
                experts.setdefault((layer, em.group(2)), {})[int(em.group(1))] = value
                continue
            if suffix.endswith("tid2eid"):
                value = value.to(torch.int64)
            out[f"layers.{layer}.{self._suffix_to_native(layer, suffix, is_mtp)}"] = value
        for (layer, w), by_e in experts.items():
            idx = sorted(by_e)
            if idx != list(range(idx[0], idx[0] + len(idx))):
                raise ValueError(f"layer {layer} {w}: expert indices are not contiguous: {idx[:8]}…")
            out[f"layers.{layer}.moe.experts.{w}"] = torch.stack([by_e[i] for i in idx], dim=0)
        return out
