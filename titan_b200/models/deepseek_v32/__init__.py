"""DeepSeek-V3.2 model family (MLA-absorb + lightning-indexer sparse attention + MTP)."""

from titan_b200.models.common.moe import MoEArgs
from titan_b200.models.deepseek_v32.model import DeepSeekV32Model
from titan_b200.models.deepseek_v32.parallelize import parallelize_deepseekv32
from titan_b200.models.deepseek_v32.state_dict_adapter import DeepSeekV32StateDictAdapter
from titan_b200.protocols.model_spec import ModelSpec

__all__ = ["DeepSeekV32Model", "deepseekv32_configs", "model_registry"]

C = DeepSeekV32Model.Config


def _moe(**kw):
    base = dict(num_experts=8, num_shared_experts=1, top_k=2, score_func="sigmoid", route_norm=True,
                route_scale=2.5, score_before_experts=False)
    base.update(kw)
    return MoEArgs(**base)


deepseekv32_configs = {
    # dim 128, 2 layers, seq 128 (reference tests/smoke_tests/config_registry.py:25-73)
    "smoketest": lambda: C(vocab_size=2048, dim=128, inter_dim=256, moe_inter_dim=64, n_layers=2, n_dense_layers=1,
                           n_heads=4, moe_args=_moe(num_experts=8), q_lora_rank=64, kv_lora_rank=64,
                           qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32, index_n_heads=4,
                           index_head_dim=32, index_topk=16),
    # long-context sparse-attention benchmark model: 12 layers, dim 2048, 16 heads, 64 experts top-6
    "sparse_12l": lambda: C(vocab_size=102400, dim=2048, inter_dim=10944, moe_inter_dim=1408, n_layers=12,
                            n_dense_layers=1, n_heads=16,
                            moe_args=_moe(num_experts=64, num_shared_experts=2, top_k=6, score_func="softmax",
                                          route_norm=False, route_scale=1.0),
                            q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                            v_head_dim=128, index_n_heads=64, index_head_dim=128, index_topk=2048),
    "671B": lambda: C(vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=61, n_dense_layers=3,
                      n_heads=128, moe_args=_moe(num_experts=256, top_k=8, num_expert_groups=8, num_limited_groups=4),
                      q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128),
    "671B_debug_4_layers": lambda: C(vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=4,
                                     n_dense_layers=1, n_heads=128, moe_args=_moe(num_experts=16, top_k=8),
                                     q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                                     v_head_dim=128),
}


def model_registry(flavor: str) -> ModelSpec:
    from titan_b200.parallel.pipeline import pipeline_llm
    from titan_b200.trainer.loss import build_mtp_loss
    from titan_b200.trainer.moe_balance import register_moe_load_balancing_hook

    if flavor not in deepseekv32_configs:
        raise KeyError(f"unknown deepseek_v32 flavor {flavor!r}; available: {sorted(deepseekv32_configs)}")
    return ModelSpec(name="deepseek_v32", flavor=flavor, model=deepseekv32_configs[flavor](),
                     parallelize_fn=parallelize_deepseekv32, pipelining_fn=pipeline_llm, build_loss_fn=build_mtp_loss,
                     post_optimizer_build_fn=register_moe_load_balancing_hook,
                     state_dict_adapter=DeepSeekV32StateDictAdapter)
