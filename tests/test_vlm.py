"""VLM on CPU: masks, scatter, position-embedding resize, loader/token bookkeeping, model step, FSDP2 run."""

import pytest
import torch

from _launch import launch, losses
from titan_b200.config.configs import MultiModalDataLoaderConfig, TrainingConfig
from titan_b200.data.mm_synthetic import build_mm_dataloader, patchify
from titan_b200.models.multimodal import (
    build_document_ids,
    build_encoder_causal_mask,
    build_encoder_full_mask,
    build_text_document_causal_mask,
    build_valid_patch_mask,
    scatter_visual_embeddings,
)
from titan_b200.models.vlm import Llama3Siglip2Transformer, vlm_configs
from titan_b200.models.vlm.siglip2 import resize_positional_embeddings_zero_padded


def test_document_ids_and_text_mask():
    tok = torch.tensor([[5, 6, 2, 7, 8, 2, 9]])
    assert build_document_ids(tok, 2).tolist() == [[0, 0, 0, 1, 1, 1, 2]]
    m = build_text_document_causal_mask(tok, 2)[0]
    assert m[2, 0] and m[4, 3] and not m[3, 2] and not m[0, 1] and not m[6, 5]


def test_encoder_masks_keep_padding_rows_finite():
    grid = torch.tensor([[[0, 0], [0, 1], [-1, -1]]])
    valid = build_valid_patch_mask(grid)
    assert valid.tolist() == [[True, True, False]]
    causal = build_encoder_causal_mask(valid)[0]
    assert causal[1, 0] and not causal[0, 1] and causal[2, 2] and not causal[2, 0]
    full = build_encoder_full_mask(valid)[0]
    assert full[0, 1] and full[2, 2] and not full[0, 2]
    assert not build_encoder_full_mask(valid, allow_padding_self_attention=False)[0, 2, 2]


def test_scatter_places_valid_patches_in_order_and_validates_count():
    h = torch.zeros(1, 6, 2)
    tok = torch.tensor([[1, 9, 9, 3, 9, 4]])
    vis = torch.arange(1, 9, dtype=torch.float32).view(2, 2, 2)
    mask = torch.tensor([[True, True], [True, False]])
    out = scatter_visual_embeddings(h, tok, vis, mask, 9)
    assert out[0, 1].tolist() == [1, 2] and out[0, 2].tolist() == [3, 4] and out[0, 4].tolist() == [5, 6]
    assert out[0, 0].abs().sum() == 0
    with pytest.raises(ValueError, match="image placeholder tokens"):
        scatter_visual_embeddings(h, tok, vis, torch.ones(2, 2, dtype=torch.bool), 9)


def test_position_embedding_resize_is_zero_on_padding_and_identity_at_native_size():
    table = torch.randn(4, 4, 8)
    out = resize_positional_embeddings_zero_padded(table, torch.tensor([[4, 4], [2, 3]]), 20)
    assert torch.allclose(out[0, :16], table.reshape(16, 8), atol=1e-6)
    assert out[0, 16:].abs().sum() == 0 and out[1, 6:].abs().sum() == 0 and out[1, :6].abs().sum() > 0


def test_patchify_grid_and_crop():
    img = torch.arange(3 * 32 * 48, dtype=torch.float32).view(3, 32, 48)
    p, g = patchify(img, 16, 64)
    assert p.shape == (6, 768) and g[:, 1].tolist() == [0, 0, 0, 1, 1, 1] and g[:, 2].tolist() == [0, 1, 2, 0, 1, 2]
    assert torch.equal(p[4].view(3, 16, 16), img[:, 16:32, 16:32])
    p, g = patchify(img, 16, 4)
    assert p.shape[0] <= 4


def test_loader_placeholders_match_valid_patches_and_model_step():
    cfg = vlm_configs["debugmodel"]()
    cfg.max_seq_len = 512
    torch.manual_seed(0)
    model = Llama3Siglip2Transformer(cfg)
    model.init_states()
    dl = build_mm_dataloader(MultiModalDataLoaderConfig(max_patches_per_image=64, max_images_per_batch=8),
                             model_config=cfg, training=TrainingConfig(local_batch_size=2, seq_len=512), dp_rank=0,
                             dp_world_size=1)
    batch, labels = next(iter(dl))
    valid = build_valid_patch_mask(batch["grid_thw"][:, :, 1:])
    assert int((batch["input"] == cfg.img_token_id).sum()) == int(valid.sum())
    assert not (labels == cfg.img_token_id).any() and (labels != -100).sum() > 0
    out = model(batch["input"], pixel_values=batch["pixel_values"], grid_thw=batch["grid_thw"])
    loss = torch.nn.functional.cross_entropy(out.flatten(0, 1).float(), labels.flatten(), ignore_index=-100)
    loss.backward()
    assert torch.isfinite(loss)
    assert model.encoder.layers["0"].self_attn.q_proj.weight.grad.abs().sum() > 0
    assert model.projector.w2.weight.grad.abs().sum() > 0
    # the same step is reproducible from the loader state
    dl2 = build_mm_dataloader(MultiModalDataLoaderConfig(max_patches_per_image=64, max_images_per_batch=8),
                              model_config=cfg, training=TrainingConfig(local_batch_size=2, seq_len=512), dp_rank=0,
                              dp_world_size=1)
    b2, l2 = next(iter(dl2))
    assert torch.equal(b2["input"], batch["input"]) and torch.equal(l2, labels)


def test_vlm_requires_its_converter_and_data_parallel_only(tmp_path):
    base = ["--module", "vlm", "--config", "vlm_debugmodel", "--comm.backend", "gloo", "--training.local_batch_size",
            "2", "--training.seq_len", "256", "--training.steps", "3", "--dataloader.max_patches_per_image", "64",
            "--dataloader.max_images_per_batch", "8", "--training.mixed_precision_param", "float32",
            "--job.dump_folder", str(tmp_path)]
    log = launch(base, 2, 29611)
    ls = losses(log)
    assert len(ls) == 3 and all(x == x and x < 12 for x in ls), log[-2000:]
    with pytest.raises(AssertionError, match="only supports FSDP/HSDP"):
        launch([*base, "--parallelism.tensor_parallel_degree", "2"], 2, 29612)
