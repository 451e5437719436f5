"""Qwen3 model family (dense 0.6B–32B, MoE 30B-A3B / 235B-A22B).

Flavors follow the upstream registry the reference re-exports (torchtitan_npu/models/qwen3/__init__.py:15-28).
"""

from titan_b200.models.common.moe import MoEArgs
from titan_b200.models.qwen3.model import Qwen3Model
from titan_b200.models.qwen3.parallelize import parallelize_qwen3
from titan_b200.models.qwen3.state_dict_adapter import Qwen3StateDictAdapter
from titan_b200.protocols.model_spec import ModelSpec

__all__ = ["Qwen3Model", "qwen3_configs", "model_registry"]

C = Qwen3Model.Config


def _moe(**kw):
    base = dict(num_experts=128, num_shared_experts=0, top_k=8, score_func="softmax", route_norm=True,
                route_scale=1.0, score_before_experts=False)
    base.update(kw)
    return MoEArgs(**base)


qwen3_configs = {
    "debugmodel": lambda: C(vocab_size=2048, dim=256, n_layers=4, n_heads=8, n_kv_heads=4, head_dim=32,
                            hidden_dim=512, max_seq_len=2048),
    "debugmodel_moe": lambda: C(vocab_size=2048, dim=256, n_layers=4, n_heads=8, n_kv_heads=4, head_dim=32,
                                hidden_dim=512, max_seq_len=2048, moe_enabled=True, moe_inter_dim=128,
                                moe_args=_moe(num_experts=8, top_k=2)),
    "0.6B": lambda: C(dim=1024, n_layers=28, n_heads=16, n_kv_heads=8, hidden_dim=3072, enable_weight_tying=True),
    "1.7B": lambda: C(dim=2048, n_layers=28, n_heads=16, n_kv_heads=8, hidden_dim=6144, enable_weight_tying=True),
    "4B": lambda: C(dim=2560, n_layers=36, n_heads=32, n_kv_heads=8, hidden_dim=9728, enable_weight_tying=True),
    "8B": lambda: C(dim=4096, n_layers=36, n_heads=32, n_kv_heads=8, hidden_dim=12288),
    "14B": lambda: C(dim=5120, n_layers=40, n_heads=40, n_kv_heads=8, hidden_dim=17408),
    "32B": lambda: C(dim=5120, n_layers=64, n_heads=64, n_kv_heads=8, hidden_dim=25600),
    "30B-A3B": lambda: C(dim=2048, n_layers=48, n_heads=32, n_kv_heads=4, hidden_dim=6144, moe_enabled=True,
                         moe_inter_dim=768, moe_args=_moe(), max_seq_len=262144),
    "235B-A22B": lambda: C(dim=4096, n_layers=94, n_heads=64, n_kv_heads=4, hidden_dim=12288, moe_enabled=True,
                           moe_inter_dim=1536, moe_args=_moe(), rope_theta=5_000_000.0),
}


def model_registry(flavor: str) -> ModelSpec:
    from titan_b200.parallel.pipeline import pipeline_llm
    from titan_b200.trainer.loss import build_cross_entropy_loss
    from titan_b200.trainer.moe_balance import register_moe_load_balancing_hook

    if flavor not in qwen3_configs:
        raise KeyError(f"unknown qwen3 flavor {flavor!r}; available: {sorted(qwen3_configs)}")
    cfg = qwen3_configs[flavor]()
    return ModelSpec(name="qwen3", flavor=flavor, model=cfg, parallelize_fn=parallelize_qwen3,
                     pipelining_fn=pipeline_llm, build_loss_fn=build_cross_entropy_loss,
                     post_optimizer_build_fn=register_moe_load_balancing_hook if cfg.moe_enabled else None,
                     state_dict_adapter=Qwen3StateDictAdapter)
