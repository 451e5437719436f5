"""Convert a DCP checkpoint (a ``step-N`` folder written by the trainer) to Hugging Face safetensors.

    python scripts/checkpoint_conversion/convert_to_hf.py outputs/checkpoint/step-100 out_hf \
        --model_name qwen3 --model_flavor 1.7B --hf_assets_path assets/hf/Qwen3-1.7B --export_dtype bfloat16

The model is built on CPU to obtain names and shapes, the checkpoint is loaded into its state dict (checkpoints saved
with fused grouped-expert weights ``w13`` are split back to ``w1`` / ``w3`` first), the model's state-dict adapter maps
native names to Hugging Face names, and the tensors are written as ``model-0000i-of-0000n.safetensors`` plus
``model.safetensors.index.json`` (shard assignment follows the asset folder's index when it has one).

(reference: scripts/checkpoint_conversion/convert_to_hf.py:28-150)
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint import FileSystemReader

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DTYPES = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


def _checkpoint_keys(input_dir) -> set[str]:
    return set(FileSystemReader(str(input_dir)).read_metadata().state_dict_metadata)


@torch.inference_mode()
def convert_to_hf(input_dir, output_dir, model_name, model_flavor, hf_assets_path, export_dtype="float32",
                  max_shard_bytes: int = 5 * 2 ** 30) -> list[str]:
    from safetensors.torch import save_file

    from titan_b200.checkpoint.weight_utils import split_fused_experts
    from titan_b200.protocols.model_spec import get_model_spec

    spec = get_model_spec(model_name, model_flavor)
    if spec.state_dict_adapter is None:
        raise ValueError(f"model {model_name} has no state-dict adapter: cannot name its tensors for Hugging Face")
    with torch.device("cpu"):
        model = spec.model.build()
    state = {k: v for k, v in model.state_dict().items()}
    keys = _checkpoint_keys(input_dir)
    fused = any(".moe.experts.w13" in k for k in keys)
    if fused:  # load the fused tensors as stored, split afterwards
        for k in [k for k in state if k.endswith(".moe.experts.w1")]:
            w1, w3 = state.pop(k), state.pop(k[:-1] + "3")
            state[k[:-2] + "w13"] = torch.empty(w1.shape[0], w1.shape[1] + w3.shape[1], w1.shape[2], dtype=w1.dtype)
    prefix = "model." if any(k.startswith("model.") for k in keys) else ""
    to_load = {prefix + k: v for k, v in state.items() if prefix + k in keys}
    missing = [k for k in state if prefix + k not in keys]
    if missing:
        print(f"warning: {len(missing)} model tensors are not in the checkpoint (kept at init): {missing[:5]} ...")
    dcp.load(to_load, checkpoint_id=str(input_dir))
    state.update({k[len(prefix):]: v for k, v in to_load.items()})
    if fused:
        state = split_fused_experts(state)
    adapter = spec.state_dict_adapter(spec.model, str(hf_assets_path) if hf_assets_path else None)
    hf = adapter.to_hf(state)
    dt = DTYPES[export_dtype]
    hf = {k: (v.to(dt) if v.is_floating_point() else v).contiguous() for k, v in hf.items()}

    os.makedirs(output_dir, exist_ok=True)
    index = getattr(adapter, "fqn_to_index_mapping", None) or {}
    index = {k: v for k, v in index.items() if k in hf}
    shards: dict[int, dict[str, torch.Tensor]] = {}
    if index:
        first = min(index.values())
        for k, v in hf.items():
            shards.setdefault(index.get(k, first), {})[k] = v
    else:  # greedy size-based sharding
        cur, size = 1, 0
        for k, v in hf.items():
            n = v.numel() * v.element_size()
            if size and size + n > max_shard_bytes:
                cur, size = cur + 1, 0
            shards.setdefault(cur, {})[k] = v
            size += n
    ids = sorted(shards)
    weight_map, files, total = {}, [], 0
    for i, sid in enumerate(ids, 1):
        name = f"model-{i:05d}-of-{len(ids):05d}.safetensors"
        save_file(shards[sid], os.path.join(output_dir, name), metadata={"format": "pt"})
        files.append(name)
        for k, v in shards[sid].items():
            weight_map[k] = name
            total += v.numel() * v.element_size()
    with open(os.path.join(output_dir, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    return files


if __name__ == "__main__":
    ap = argparse.ArgumentParser(description="Convert DCP weights to HF format.")
    ap.add_argument("input_dir", type=Path, help="Input directory with DCP weights.")
    ap.add_argument("output_dir", type=Path, help="Output directory for HF checkpoint.")
    ap.add_argument("--hf_assets_path", type=Path, default=None,
                    help="HF asset folder; its model.safetensors.index.json decides the shard of every tensor")
    ap.add_argument("--model_name", type=str, default="llama3")
    ap.add_argument("--model_flavor", type=str, default="8B")
    ap.add_argument("--export_dtype", type=str, choices=list(DTYPES), default="float32")
    a = ap.parse_args()
    out = convert_to_hf(a.input_dir, a.output_dir, a.model_name, a.model_flavor, a.hf_assets_path, a.export_dtype)
    print(f"wrote {len(out)} shard(s) to {a.output_dir}")
