"""DeepSeek-V4 model family (hyper-connections, compressed sparse attention, hash / sqrt-softplus MoE, MTP).

Flavors follow the reference registry (torchtitan_npu/models/deepseek_v4/__init__.py:40-200).
"""

from titan_b200.models.common.moe import MoEArgs
from titan_b200.models.deepseek_v4.transformer import DeepSeekV4Model
from titan_b200.protocols.model_spec import ModelSpec

__all__ = ["DeepSeekV4Model", "deepseekv4_configs", "model_registry"]

C = DeepSeekV4Model.Config


def _moe(**kw):
    base = dict(num_experts=8, num_shared_experts=1, top_k=2, score_func="sqrtsoftplus", route_norm=True,
                route_scale=1.5, score_before_experts=False, swiglu_limit=10.0, n_hash_layers=3)
    base.update(kw)
    return MoEArgs(**base)


def _flash(**kw):
    """V4-Flash: 43 layers, dim 4096, 64 heads of one shared 512-wide KV latent, 256 experts top-6."""
    base = dict(vocab_size=129280, n_layers=43, n_heads=64, max_seq_len=4096, dim=4096, moe_inter_dim=2048,
                head_dim=512, rope_head_dim=64, q_lora_rank=1024, o_lora_rank=1024, o_groups=8, window_size=128,
                compress_ratios=(1, 1, 4) + (128, 4) * 20, moe_args=_moe(num_experts=256, top_k=6),
                hc_sinkhorn_iters=20, hc_mult=4, hc_eps=1e-6, compress_rope_theta=160000.0, original_seq_len=65536,
                rope_theta=10000.0, rope_factor=16, beta_fast=32, beta_slow=1, enable_indexer_loss=True,
                index_n_heads=64, index_head_dim=128, index_topk=512)
    base.update(kw)
    return C(**base)


def _pro(**kw):
    """V4-Pro: 61 layers, dim 7168, 128 heads, 384 experts top-6."""
    return _flash(**{**dict(n_layers=61, n_heads=128, dim=7168, moe_inter_dim=3072, q_lora_rank=1536, o_groups=16,
                            compress_ratios=(128,) + (128, 4) * 30, moe_args=_moe(num_experts=384, top_k=6),
                            index_topk=1024), **kw})


_SINGLE_NODE_MOE = dict(num_experts=16, top_k=2, use_grouped_mm=False, n_hash_layers=0)

deepseekv4_configs = {
    "v4_flash_43layers_16experts": lambda: _flash(moe_args=_moe(**_SINGLE_NODE_MOE)),
    "v4_flash_43layers_256experts": _flash,
    "v4_pro_16layers_16experts": lambda: _pro(n_layers=16, compress_ratios=((128,) + (128, 4) * 30)[:16],
                                              moe_args=_moe(**_SINGLE_NODE_MOE)),
    "v4_pro_61layers_384experts": _pro,
    "mini_1b": lambda: _flash(n_layers=24, n_heads=16, dim=1024, moe_inter_dim=512, head_dim=64, rope_head_dim=32,
                              q_lora_rank=384, o_lora_rank=384, o_groups=4, window_size=64,
                              compress_ratios=(1, 1) + (4, 96) * 10 + (4, 1), original_seq_len=0, rope_factor=1,
                              moe_args=_moe(num_experts=16, top_k=2, n_hash_layers=2), index_n_heads=8,
                              index_head_dim=64, index_topk=128),
    "smoketest": lambda: C(vocab_size=2048, dim=128, moe_inter_dim=64, n_layers=4, n_heads=4, head_dim=64,
                           rope_head_dim=16, q_lora_rank=64, o_lora_rank=32, o_groups=2, window_size=16,
                           compress_ratios=(1, 1, 4, 128), index_n_heads=4, index_head_dim=32, index_topk=8,
                           moe_args=_moe(num_experts=8, n_hash_layers=1), original_seq_len=0),
}


def model_registry(flavor: str) -> ModelSpec:
    from titan_b200.models.deepseek_v4.parallelize import parallelize_deepseekv4
    from titan_b200.models.deepseek_v4.state_dict_adapter import DeepSeekV4StateDictAdapter
    from titan_b200.parallel.pipeline import pipeline_llm
    from titan_b200.trainer.loss import build_mtp_loss
    from titan_b200.trainer.moe_balance import register_moe_load_balancing_hook

    if flavor not in deepseekv4_configs:
        raise KeyError(f"unknown deepseek_v4 flavor {flavor!r}; available: {sorted(deepseekv4_configs)}")
    return ModelSpec(name="deepseek_v4", flavor=flavor, model=deepseekv4_configs[flavor](),
                     parallelize_fn=parallelize_deepseekv4, pipelining_fn=pipeline_llm, build_loss_fn=build_mtp_loss,
                     post_optimizer_build_fn=register_moe_load_balancing_hook,
                     state_dict_adapter=DeepSeekV4StateDictAdapter)
