"""Vision-language model family: Llama-3 decoder + Siglip2 vision tower (reference: torchtitan_npu/models/vlm)."""

from titan_b200.models.vlm.model import Llama3Siglip2Transformer
from titan_b200.models.vlm.parallelize import parallelize_vlm
from titan_b200.models.vlm.siglip2 import VisionTransformer
from titan_b200.protocols.model_spec import ModelSpec

__all__ = ["Llama3Siglip2Transformer", "vlm_configs", "model_registry", "parallelize_vlm"]

C, E = Llama3Siglip2Transformer.Config, VisionTransformer.Config

vlm_configs = {
    "debugmodel": lambda: C(dim=256, n_layers=6, n_heads=16, vocab_size=2048, rope_theta=500000.0,
                            encoder=E(dim=128, ffn_dim=256, n_layers=4, n_heads=2)),
    "debugmodel_large_projector": lambda: C(dim=512, n_layers=6, n_heads=16, vocab_size=2048, rope_theta=500000.0,
                                            encoder=E(dim=256, ffn_dim=512, n_layers=4, n_heads=4)),
    "8B": lambda: C(dim=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_dim_multiplier=1.3, multiple_of=1024,
                    rope_theta=500000.0, img_token_id=128256 - 4, boi_token_id=128256 - 3,
                    eoi_token_id=128256 - 2, pad_token_id=128256 - 1, eos_token_id=128001,
                    encoder=E(dim=768, ffn_dim=3072, n_layers=12, n_heads=12)),
}


def model_registry(flavor: str) -> ModelSpec:
    from titan_b200.trainer.loss import build_cross_entropy_loss

    if flavor not in vlm_configs:
        raise KeyError(f"unknown vlm flavor {flavor!r}; available: {sorted(vlm_configs)}")
    return ModelSpec(name="vlm", flavor=flavor, model=vlm_configs[flavor](), parallelize_fn=parallelize_vlm,
                     pipelining_fn=None, build_loss_fn=build_cross_entropy_loss, post_optimizer_build_fn=None,
                     state_dict_adapter=None)
