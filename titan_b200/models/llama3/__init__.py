"""Llama-3 model family: flavors, registry entry, HF adapter."""

from titan_b200.models.llama3.model import Llama3Model
from titan_b200.models.llama3.parallelize import parallelize_llama
from titan_b200.models.llama3.state_dict_adapter import Llama3StateDictAdapter
from titan_b200.protocols.model_spec import ModelSpec

__all__ = ["Llama3Model", "llama3_configs", "model_registry", "parallelize_llama"]

_ROPE_SCALING = {"scaling_factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_pos": 8192}


def _cfg(**kw):
    return lambda: Llama3Model.Config(**kw)


llama3_configs = {
    # dim 256, 6 layers, 16 heads (head_dim 16), SwiGLU hidden 768, vocab 2048, theta 500000
    "debugmodel": _cfg(dim=256, n_layers=6, n_heads=16, vocab_size=2048, ffn_hidden=768, rope_theta=500000,
                       norm_eps=1e-5, max_seq_len=2048),
    "8B": _cfg(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024,
               rope_theta=500000, vocab_size=128256, max_seq_len=8192),
    "70B": _cfg(dim=8192, n_layers=80, n_heads=64, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=4096,
                rope_theta=500000, vocab_size=128256, max_seq_len=8192),
    "405B": _cfg(dim=16384, n_layers=126, n_heads=128, n_kv_heads=8, ffn_dim_multiplier=1.2, multiple_of=4096,
                 rope_theta=500000, vocab_size=128256, max_seq_len=8192),
}


def model_registry(flavor: str) -> ModelSpec:
    from titan_b200.parallel.pipeline import pipeline_llm
    from titan_b200.trainer.loss import build_cross_entropy_loss

    if flavor not in llama3_configs:
        raise KeyError(f"unknown llama3 flavor {flavor!r}; available: {sorted(llama3_configs)}")
    return ModelSpec(
        name="llama3",
        flavor=flavor,
        model=llama3_configs[flavor](),
        parallelize_fn=parallelize_llama,
        pipelining_fn=pipeline_llm,
        build_loss_fn=build_cross_entropy_loss,
        post_optimizer_build_fn=None,
        state_dict_adapter=Llama3StateDictAdapter,
    )
