"""DeepSeek-V3 model family: flavors and registry entry.

Flavors: ``debugmodel`` / ``smoketest`` (tiny), ``16B`` (the HF ``deepseek-moe-16b`` weights expressed
as MLA: kv_lora 3072 = 16 heads x (64 + 128), reference models/deepseek_v3/__init__.py:27-80),
``16B_mla`` (true MLA dims: 27 layers, kv_lora 512, qk_nope 128, rope 64, v 128, first layer dense
FFN 10944, 64 routed experts of hidden 1408 with top-6 softmax routing, 2 shared experts),
``671B`` and pruned ``671B_debug*`` variants.
"""

from titan_b200.models.common.moe import MoEArgs
from titan_b200.models.deepseek_v3.model import DeepSeekV3Model
from titan_b200.models.deepseek_v3.parallelize import parallelize_deepseekv3
from titan_b200.models.deepseek_v3.state_dict_adapter import (
    DeepSeek16BStateDictAdapter,
    DeepSeekV3StateDictAdapter,
)
from titan_b200.protocols.model_spec import ModelSpec

__all__ = ["DeepSeekV3Model", "deepseekv3_configs", "model_registry", "parallelize_deepseekv3"]

C = DeepSeekV3Model.Config


def _moe(**kw):
    base = dict(num_experts=8, num_shared_experts=2, top_k=3, score_func="softmax", route_norm=False,
                score_before_experts=False)
    base.update(kw)
    return MoEArgs(**base)


deepseekv3_configs = {
    "debugmodel": lambda: C(vocab_size=2048, dim=256, inter_dim=1024, moe_inter_dim=256, n_layers=6, n_dense_layers=1,
                            n_heads=16, moe_args=_moe(), q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128,
                            qk_rope_head_dim=64, v_head_dim=128, mscale=0.70),
    "smoketest": lambda: C(vocab_size=2048, dim=128, inter_dim=256, moe_inter_dim=64, n_layers=4, n_dense_layers=1,
                           n_heads=4, moe_args=_moe(num_experts=8, top_k=2, num_shared_experts=1), q_lora_rank=0,
                           kv_lora_rank=64, qk_nope_head_dim=32, qk_rope_head_dim=16, v_head_dim=32),
    "16B": lambda: C(vocab_size=102400, dim=2048, inter_dim=10944, moe_inter_dim=1408, n_layers=28, n_dense_layers=1,
                     n_heads=16, moe_args=_moe(num_experts=64, num_shared_experts=2, top_k=6), q_lora_rank=0,
                     kv_lora_rank=3072, qk_nope_head_dim=64, qk_rope_head_dim=64, v_head_dim=128, mscale=0.70),
    "16B_mla": lambda: C(vocab_size=102400, dim=2048, inter_dim=10944, moe_inter_dim=1408, n_layers=27,
                         n_dense_layers=1, n_heads=16,
                         moe_args=_moe(num_experts=64, num_shared_experts=2, top_k=6, score_func="softmax"),
                         q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                         mscale=0.70),
    # the 16B_mla layer shapes with 5 of the 27 layers: fits two GPUs with fp32 AdamW state (expert-parallel benchmarks)
    "16B_mla_5l": lambda: C(vocab_size=102400, dim=2048, inter_dim=10944, moe_inter_dim=1408, n_layers=5,
                            n_dense_layers=1, n_heads=16,
                            moe_args=_moe(num_experts=64, num_shared_experts=2, top_k=6, score_func="softmax"),
                            q_lora_rank=0, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128,
                            mscale=0.70),
    "236B": lambda: C(vocab_size=102400, dim=5120, inter_dim=12288, moe_inter_dim=1536, n_layers=60, n_dense_layers=1,
                      n_heads=128, moe_args=_moe(num_experts=160, num_shared_experts=2, top_k=6, route_norm=False,
                                                 route_scale=16.0, num_expert_groups=8, num_limited_groups=3),
                      q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128),
    "671B": lambda: C(vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=61, n_dense_layers=3,
                      n_heads=128, moe_args=_moe(num_experts=256, num_shared_experts=1, top_k=8, score_func="sigmoid",
                                                 route_norm=True, route_scale=2.5, num_expert_groups=8,
                                                 num_limited_groups=4),
                      q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64, v_head_dim=128),
    # pruned 671B shapes for single-node debugging (full width, few layers / experts)
    "671B_debug": lambda: C(vocab_size=129280, dim=7168, inter_dim=18432, moe_inter_dim=2048, n_layers=4,
                            n_dense_layers=1, n_heads=128,
                            moe_args=_moe(num_experts=8, num_shared_experts=1, top_k=2, score_func="sigmoid",
                                          route_norm=True, route_scale=2.5),
                            q_lora_rank=1536, kv_lora_rank=512, qk_nope_head_dim=128, qk_rope_head_dim=64,
                            v_head_dim=128),
}


def model_registry(flavor: str) -> ModelSpec:
    from titan_b200.parallel.pipeline import pipeline_llm
    from titan_b200.trainer.loss import build_cross_entropy_loss
    from titan_b200.trainer.moe_balance import register_moe_load_balancing_hook

    if flavor not in deepseekv3_configs:
        raise KeyError(f"unknown deepseek_v3 flavor {flavor!r}; available: {sorted(deepseekv3_configs)}")
    return ModelSpec(
        name="deepseek_v3", flavor=flavor, model=deepseekv3_configs[flavor](),
        parallelize_fn=parallelize_deepseekv3, pipelining_fn=pipeline_llm, build_loss_fn=build_cross_entropy_loss,
        post_optimizer_build_fn=register_moe_load_balancing_hook,
        state_dict_adapter=DeepSeek16BStateDictAdapter if flavor == "16B" else DeepSeekV3StateDictAdapter,
    )
