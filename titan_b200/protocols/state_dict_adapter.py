"""Base class for native ↔ Hugging Face state-dict adapters.

An adapter maps parameter names (and, where layouts differ, tensors) between
this framework's FQNs and the Hugging Face checkpoint of the same model.
Converter state-dict updaters that are active (e.g. fused ``w13`` experts) run
before ``to_hf`` and after ``from_hf`` so checkpoints always keep the canonical
layout.

Parity: torchtitan_npu/converters/framework/state_dict_update_wrapper.py:17-56,
models/*/state_dict_adapter.py.
"""

from __future__ import annotations

import json
import os
import re
from typing import Any

from titan_b200.protocols.converter import active_state_dict_updaters

__all__ = ["StateDictAdapter"]


class StateDictAdapter:
    #: native-name template → HF-name template; ``{}`` stands for a layer (or expert) index
    from_hf_map: dict[str, str | None] = {}

    def __init__(self, model_config, hf_assets_path: str | None = None):
        self.model_config = model_config
        self.hf_assets_path = hf_assets_path
        self.fqn_to_index_mapping: dict[str, int] | None = None
        if hf_assets_path:
            idx = os.path.join(hf_assets_path, "model.safetensors.index.json")
            if os.path.exists(idx):
                with open(idx) as f:
                    weight_map = json.load(f).get("weight_map", {})
                self.fqn_to_index_mapping = {
                    k: int(re.search(r"\d+", v).group(0)) if re.search(r"\d+", v) else 1 for k, v in weight_map.items()
                }

    # ---- template helpers
    @staticmethod
    def _abstract(key: str) -> tuple[str, list[str]]:
        nums = re.findall(r"(?<=\.)\d+(?=\.)", key)
        return re.sub(r"(?<=\.)\d+(?=\.)", "{}", key), nums

    def _rename(self, key: str, table: dict[str, str | None]) -> str | None:
        abstract, nums = self._abstract(key)
        if abstract in table:
            tgt = table[abstract]
            return None if tgt is None else tgt.format(*nums)
        if key in table:
            return table[key]
        raise KeyError(f"no mapping for parameter {key!r}")

    # ---- subclass surface
    def _to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        inv = {v: k for k, v in self.from_hf_map.items() if v is not None}
        out = {}
        for k, v in state_dict.items():
            nk = self._rename(k, inv)
            if nk is not None:
                out[nk] = v
        return out

    def _from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        out = {}
        for k, v in hf_state_dict.items():
            nk = self._rename(k, self.from_hf_map)
            if nk is not None:
                out[nk] = v
        return out

    # ---- public API (runs converter updaters around the subclass mapping)
    def to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        for up in active_state_dict_updaters():
            state_dict = up.to_hf(state_dict)
        return self._to_hf(state_dict)

    def from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        sd = self._from_hf(hf_state_dict)
        for up in reversed(active_state_dict_updaters()):
            sd = up.from_hf(sd)
        return sd

    def get_hf_storage_reader(self, path: str, from_quantized: bool = False):
        """HF safetensors reader, or a plain DCP reader when `path` holds a DCP checkpoint."""
        from titan_b200.checkpoint.weight_utils import is_dcp_checkpoint

        if is_dcp_checkpoint(path):
            from torch.distributed.checkpoint import FileSystemReader

            return FileSystemReader(path)
        from torch.distributed.checkpoint import HuggingFaceStorageReader

        return HuggingFaceStorageReader(path)
