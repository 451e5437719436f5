"""DeepSeek-V3 native ↔ Hugging Face parameter mapping.

`MoEStateDictAdapter` handles stacked experts: HF stores one matrix per expert
(``…mlp.experts.<e>.gate_proj.weight``), this framework one stacked tensor per layer
(``layers.N.moe.experts.w1`` of shape ``[E, H, D]``).  Stacking / splitting is DTensor-aware: for an
expert tensor sharded on dim 0 only the local experts' HF keys are produced / consumed.

`DeepSeek16BStateDictAdapter` additionally converts the multi-head K/V projections of the HF
``deepseek-moe-16b`` checkpoint into the MLA parameterisation (``kv_lora_rank = n_heads·(64+128)``):
per head the latent interleaves ``[k_nope | v]`` rows, the rotary key shared by all heads is the mean
of the heads' rotary rows, ``wkv_b`` is the identity and ``kv_norm`` is all ones.

Parity: torchtitan_npu/models/deepseek_v3/state_dict_adapter.py:24-385.
"""

from __future__ import annotations

import re
from typing import Any

import torch
from torch.distributed.tensor import DTensor, Replicate, Shard

from titan_b200.protocols.state_dict_adapter import StateDictAdapter

__all__ = ["MoEStateDictAdapter", "DeepSeekV3StateDictAdapter", "DeepSeek16BStateDictAdapter"]

_EXPERT_HF = re.compile(r"^(.*\.mlp\.experts)\.(\d+)\.(gate_proj|up_proj|down_proj)\.weight$")
_EXPERT_NATIVE = re.compile(r"^layers\.(\d+)\.moe\.experts\.(w1|w2|w3)$")
_PROJ = {"gate_proj": "w1", "up_proj": "w3", "down_proj": "w2"}
_PROJ_INV = {v: k for k, v in _PROJ.items()}


class MoEStateDictAdapter(StateDictAdapter):
    def _num_experts(self) -> int:
        return self.model_config.moe_args.num_experts

    @staticmethod
    def _local_expert_range(t) -> tuple[int, int, Any]:
        """(first expert, count, local tensor) for a possibly sharded DTensor.  Shards of the expert dim (0) stay
        local: every rank exports its own experts.  A weight that is also split inside the expert (expert tensor
        parallelism, or FSDP on dim 1 when a rank has fewer experts than shard ranks) is gathered over those mesh
        dims first (a collective: every rank of the mesh exports together, as it does under DCP)."""
        if isinstance(t, DTensor):
            inner = [isinstance(pl, Shard) and pl.dim != 0 for pl in t.placements]
            if any(inner):
                t = t.redistribute(placements=[Replicate() if g else pl for g, pl in zip(inner, t.placements)])
            local = t.to_local()
            first = 0
            stride = 1   # several mesh dims may split the expert dim: the last one varies fastest
            for mesh_dim in reversed(range(len(t.placements))):
                pl = t.placements[mesh_dim]
                if isinstance(pl, Shard) and pl.dim == 0:
                    first += t.device_mesh.get_local_rank(mesh_dim) * stride * local.shape[0]
                    stride *= t.device_mesh.size(mesh_dim)
            return first, local.shape[0], local
        return 0, t.shape[0], t

    def _split_experts(self, key: str, value) -> dict[str, Any]:
        m = _EXPERT_NATIVE.match(key)
        layer, w = m.group(1), m.group(2)
        first, n, local = self._local_expert_range(value)
        return {f"model.layers.{layer}.mlp.experts.{first + e}.{_PROJ_INV[w]}.weight": local[e] for e in range(n)}

    def _stack_experts(self, hf: dict[str, Any]) -> tuple[dict[str, Any], dict[str, Any]]:
        """→ (stacked native expert tensors, the remaining HF entries)."""
        groups: dict[tuple[str, str], dict[int, Any]] = {}
        rest = {}
        for k, v in hf.items():
            m = _EXPERT_HF.match(k)
            if not m:
                rest[k] = v
                continue
            layer = re.search(r"layers\.(\d+)\.", k).group(1)
            groups.setdefault((layer, _PROJ[m.group(3)]), {})[int(m.group(2))] = v
        out = {}
        for (layer, w), by_e in groups.items():
            idx = sorted(by_e)
            if idx != list(range(idx[0], idx[0] + len(idx))):
                raise ValueError(f"layer {layer} {w}: expert indices are not contiguous: {idx[:8]}…")
            out[f"layers.{layer}.moe.experts.{w}"] = torch.stack([by_e[i] for i in idx], dim=0)
        return out, rest

    def _to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        plain, out = {}, {}
        for k, v in state_dict.items():
            if _EXPERT_NATIVE.match(k):
                out.update(self._split_experts(k, v))
            else:
                plain[k] = v
        out.update(super()._to_hf(plain))
        return out

    def _from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        hf = {k: v for k, v in hf_state_dict.items() if not k.endswith(".weight_scale_inv")}
        stacked, rest = self._stack_experts(hf)
        out = super()._from_hf(rest)
        out.update(stacked)
        return out


class DeepSeekV3StateDictAdapter(MoEStateDictAdapter):
    from_hf_map = {
        "model.embed_tokens.weight": "tok_embeddings.weight",
        "model.layers.{}.self_attn.q_proj.weight": "layers.{}.attention.wq.weight",
        "model.layers.{}.self_attn.q_a_proj.weight": "layers.{}.attention.wq_a.weight",
        "model.layers.{}.self_attn.q_a_layernorm.weight": "layers.{}.attention.q_norm.weight",
        "model.layers.{}.self_attn.q_b_proj.weight": "layers.{}.attention.wq_b.weight",
        "model.layers.{}.self_attn.kv_a_proj_with_mqa.weight": "layers.{}.attention.wkv_a.weight",
        "model.layers.{}.self_attn.kv_a_layernorm.weight": "layers.{}.attention.kv_norm.weight",
        "model.layers.{}.self_attn.kv_b_proj.weight": "layers.{}.attention.wkv_b.weight",
        "model.layers.{}.self_attn.o_proj.weight": "layers.{}.attention.wo.weight",
        "model.layers.{}.mlp.gate_proj.weight": "layers.{}.feed_forward.w1.weight",
        "model.layers.{}.mlp.up_proj.weight": "layers.{}.feed_forward.w3.weight",
        "model.layers.{}.mlp.down_proj.weight": "layers.{}.feed_forward.w2.weight",
        "model.layers.{}.input_layernorm.weight": "layers.{}.attention_norm.weight",
        "model.layers.{}.post_attention_layernorm.weight": "layers.{}.ffn_norm.weight",
        "model.layers.{}.mlp.gate.weight": "layers.{}.moe.router.gate.weight",
        "model.layers.{}.mlp.gate.e_score_correction_bias": "layers.{}.moe.expert_bias",
        "model.layers.{}.mlp.shared_experts.gate_proj.weight": "layers.{}.moe.shared_experts.w1.weight",
        "model.layers.{}.mlp.shared_experts.up_proj.weight": "layers.{}.moe.shared_experts.w3.weight",
        "model.layers.{}.mlp.shared_experts.down_proj.weight": "layers.{}.moe.shared_experts.w2.weight",
        "model.norm.weight": "norm.weight",
        "lm_head.weight": "output.weight",
    }


class DeepSeek16BStateDictAdapter(MoEStateDictAdapter):
    from_hf_map = {k: v for k, v in DeepSeekV3StateDictAdapter.from_hf_map.items()
                   if "kv_a" not in k and "kv_b" not in k and "q_a_" not in k and "q_b_" not in k}

    def _dims(self):
        c = self.model_config
        return c.n_heads, c.qk_nope_head_dim, c.qk_rope_head_dim, c.v_head_dim

    def _from_hf(self, hf_state_dict: dict[str, Any]) -> dict[str, Any]:
        n_h, qn, qr, vh = self._dims()
        kv = {k: v for k, v in hf_state_dict.items() if ".self_attn.k_proj." in k or ".self_attn.v_proj." in k}
        rest = {k: v for k, v in hf_state_dict.items() if k not in kv}
        out = super()._from_hf(rest)
        layers = sorted({int(re.search(r"layers\.(\d+)\.", k).group(1)) for k in kv})
        for li in layers:
            k_w = kv[f"model.layers.{li}.self_attn.k_proj.weight"].view(n_h, qn + qr, -1)
            v_w = kv[f"model.layers.{li}.self_attn.v_proj.weight"].view(n_h, vh, -1)
            latent = torch.cat([k_w[:, :qn], v_w], dim=1).reshape(n_h * (qn + vh), -1)  # per head [k_nope | v]
            k_pe = k_w[:, qn:].float().mean(0).to(k_w.dtype)  # one rotary key shared by all heads
            out[f"layers.{li}.attention.wkv_a.weight"] = torch.cat([latent, k_pe], dim=0)
            rank = n_h * (qn + vh)
            out[f"layers.{li}.attention.wkv_b.weight"] = torch.eye(rank, dtype=k_w.dtype)
            out[f"layers.{li}.attention.kv_norm.weight"] = torch.ones(rank, dtype=k_w.dtype)
        return out

    def _to_hf(self, state_dict: dict[str, Any]) -> dict[str, Any]:
        n_h, qn, qr, vh = self._dims()
        full = lambda t: t.full_tensor() if isinstance(t, DTensor) else t  # noqa: E731
        mla = {k: v for k, v in state_dict.items() if re.search(r"attention\.(wkv_a|wkv_b|kv_norm)\.weight$", k)}
        rest = {k: v for k, v in state_dict.items() if k not in mla}
        out = super()._to_hf(rest)
        layers = sorted({int(re.search(r"layers\.(\d+)\.", k).group(1)) for k in mla if "wkv_a" in k})
        for li in layers:
            wkv_a = full(mla[f"layers.{li}.attention.wkv_a.weight"])
            rank = n_h * (qn + vh)
            latent, k_pe = wkv_a[:rank], wkv_a[rank:]
            kb, kn = f"layers.{li}.attention.wkv_b.weight", f"layers.{li}.attention.kv_norm.weight"
            if kb in mla and kn in mla:
                # training may have moved wkv_b / kv_norm away from identity: fold them back into the latent rows
                latent = (full(mla[kb]).float() @ torch.diag(full(mla[kn]).float()) @ latent.float()).to(wkv_a.dtype)
            per_head = latent.view(n_h, qn + vh, -1)
            k_nope, v_w = per_head[:, :qn], per_head[:, qn:]
            k_w = torch.cat([k_nope, k_pe.unsqueeze(0).expand(n_h, -1, -1)], dim=1).reshape(n_h * (qn + qr), -1)
            out[f"model.layers.{li}.self_attn.k_proj.weight"] = k_w
            out[f"model.layers.{li}.self_attn.v_proj.weight"] = v_w.reshape(n_h * vh, -1)
        return out
