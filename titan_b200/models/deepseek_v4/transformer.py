"""DeepSeek-V4 hyper-connected transformer block, MTP module and the full model.

Parity: torchtitan_npu/models/deepseek_v4/model.py:1077-1660 (block, HcHead, MTPModule, DeepSeekV4Model).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.nn as nn

from titan_b200.models.common.layers import Embedding, Linear, RMSNorm
from titan_b200.models.common.moe import MoEArgs
from titan_b200.models.common.rope import apply_rotary_emb_single_complex  # noqa: F401  (re-exported for adapters)
from titan_b200.models.deepseek_v4.layers import precompute_v4_freqs
from titan_b200.models.deepseek_v4.model import HcHead, V4Attention, V4MoE, _ratio_of
from titan_b200.ops import mhc
from titan_b200.protocols.module import BaseModelConfig, Module, ModuleDict
from titan_b200.utils.logging import logger

__all__ = ["DeepSeekV4Model", "V4Block", "V4MTPModule"]


class V4Block(Module):
    def __init__(self, layer_id: int, cfg: "DeepSeekV4Model.Config"):
        super().__init__()
        self.layer_id, self.moe_enabled = layer_id, True
        self.hc_mult, self.hc_iters, self.hc_eps, self.norm_eps = (cfg.hc_mult, cfg.hc_sinkhorn_iters, cfg.hc_eps,
                                                                     cfg.norm_eps)
        self.compress_ratio = _ratio_of(cfg, layer_id)
        self.attention = V4Attention(layer_id, cfg)
        self.moe = V4MoE(cfg.dim, cfg.moe_inter_dim, cfg.moe_args, layer_id=layer_id, vocab_size=cfg.vocab_size)
        self.attention_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.ffn_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        mix, hc_dim = (2 + cfg.hc_mult) * cfg.hc_mult, cfg.hc_mult * cfg.dim
        f32 = dict(dtype=torch.float32)  # the mixing parameters stay in fp32
        self.hc_attn_fn = nn.Parameter(torch.empty(mix, hc_dim, **f32))
        self.hc_ffn_fn = nn.Parameter(torch.empty(mix, hc_dim, **f32))
        self.hc_attn_base = nn.Parameter(torch.empty(mix, **f32))
        self.hc_ffn_base = nn.Parameter(torch.empty(mix, **f32))
        self.hc_attn_scale = nn.Parameter(torch.empty(3, **f32))
        self.hc_ffn_scale = nn.Parameter(torch.empty(3, **f32))
        self.weight_init_std = 0.02 / (2 * (layer_id + 1)) ** 0.5
        # the final collapse of the streams lives in the last main block, so it shares that block's FSDP unit and
        # stays on the last pipeline stage without special splitting
        self.is_last_layer = layer_id == cfg.n_layers - 1
        if self.is_last_layer:
            self.hc_head = HcHead(cfg)

    def _pre(self, x, fn, scale, base):
        return mhc.hc_pre(x, fn, scale, base, self.hc_mult, self.hc_iters, self.hc_eps, self.norm_eps)

    def _sublayers(self, x, input_ids, freqs_cis, attention_masks, positions):
        y, post, comb = self._pre(x, self.hc_attn_fn, self.hc_attn_scale, self.hc_attn_base)
        y = self.attention(self.attention_norm(y), freqs_cis, attention_masks, positions)
        x = mhc.hc_post(y, x, post, comb)
        y, post, comb = self._pre(x, self.hc_ffn_fn, self.hc_ffn_scale, self.hc_ffn_base)
        y = self.moe(self.ffn_norm(y), input_ids)
        return mhc.hc_post(y, x, post, comb)

    def forward(self, x, input_ids, freqs_cis, attention_masks=None, positions=None):
        """x [B, S, hc, D] → same; the last main block returns the collapsed [B, S, D]."""
        x = self._sublayers(x, input_ids, freqs_cis, attention_masks, positions)
        return self.hc_head(x) if self.is_last_layer else x

    def init_states(self, *, buffer_device=None, **kw):
        for n in (self.attention_norm, self.ffn_norm):
            nn.init.trunc_normal_(n.weight, mean=1.0, std=0.02)
        self.attention.init_states(init_std=self.weight_init_std)
        self.moe.init_states(init_std=self.weight_init_std, buffer_device=buffer_device)
        for p in (self.hc_attn_fn, self.hc_ffn_fn, self.hc_attn_base, self.hc_ffn_base, self.hc_attn_scale,
                  self.hc_ffn_scale):
            nn.init.trunc_normal_(p, mean=0.0, std=0.02)
        if self.is_last_layer:
            self.hc_head.init_states()


class V4MTPModule(V4Block):
    """Multi-token-prediction depth: ``e_proj(enorm(emb(next token))) + h_proj(hnorm(h_prev))`` spread over the hc
    streams → one block → its own stream collapse and norm."""

    def __init__(self, layer_id: int, cfg: "DeepSeekV4Model.Config"):
        super().__init__(layer_id, cfg)
        self.enorm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.hnorm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.e_proj = Linear(cfg.dim, cfg.dim, bias=False)
        self.h_proj = Linear(cfg.dim, cfg.dim, bias=False)
        self.mtp_hc_head = HcHead(cfg)
        self.mtp_norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)

    def forward(self, emb_next, h_prev, input_ids, freqs_cis, attention_masks=None, positions=None):
        x = self.e_proj(self.enorm(emb_next)) + self.h_proj(self.hnorm(h_prev))
        x = x.unsqueeze(2).repeat(1, 1, self.hc_mult, 1)
        x = self.mtp_hc_head(self._sublayers(x, input_ids, freqs_cis, attention_masks, positions))
        return x, self.mtp_norm(x)

    def init_states(self, *, buffer_device=None, **kw):
        super().init_states(buffer_device=buffer_device)
        for n in (self.enorm, self.hnorm, self.mtp_norm):
            nn.init.trunc_normal_(n.weight, mean=1.0, std=0.02)
        nn.init.trunc_normal_(self.e_proj.weight, mean=0.0, std=0.02)
        nn.init.trunc_normal_(self.h_proj.weight, mean=0.0, std=0.02)
        self.mtp_hc_head.init_states()


class DeepSeekV4Model(Module):
    @dataclass(kw_only=True)
    class Config(BaseModelConfig):
        norm_eps: float = 1e-6
        index_n_heads: int = 64
        index_head_dim: int = 128
        index_topk: int = 512
        enable_indexer_loss: bool = True
        dim: int = 4096
        moe_args: MoEArgs = field(default_factory=lambda: MoEArgs(
            score_func="sqrtsoftplus", route_scale=1.5, score_before_experts=False, swiglu_limit=10.0,
            n_hash_layers=3, num_limited_groups=8))
        rope_head_dim: int = 64
        q_lora_rank: int = 1024
        max_seq_len: int = 4096
        n_heads: int = 64
        o_lora_rank: int = 1024
        head_dim: int = 512
        o_groups: int = 8
        window_size: int = 128
        compress_ratios: tuple = (1, 1, 4, 128)
        hc_sinkhorn_iters: int = 20
        hc_mult: int = 4
        hc_eps: float = 1e-6
        vocab_size: int = 129280
        moe_inter_dim: int = 2048
        load_balance_coeff: float | None = 1e-3
        compress_rope_theta: float = 40000.0
        original_seq_len: int = 65536
        rope_theta: float = 10000.0
        rope_factor: float = 4
        beta_fast: int = 32
        beta_slow: int = 1
        n_layers: int = 4
        use_smla: bool = False
        num_mtp_modules: int = 0
        mtp_layer_compress_ratio: int = 1
        use_global_tnd: bool = False
        """Pack every valid token of a batch of documents into one [1, T] stream (needs dataloader positions)."""

        def update_from_config(self, *, trainer_config, **kw) -> None:
            from titan_b200.protocols.converter import has_converter

            seq_len = trainer_config.training.seq_len
            if seq_len > self.max_seq_len:
                logger.warning("sequence length %d exceeds the model's configured maximum %d", seq_len,
                               self.max_seq_len)
            self.max_seq_len = seq_len
            self.moe_args._debug_force_load_balance = trainer_config.debug.moe_force_load_balance
            self.moe_args.load_balance_coeff = self.load_balance_coeff
            self.use_smla = has_converter(trainer_config.model_converters.converters, "b200_smla")
            self.num_mtp_modules = trainer_config.training.num_mtp_modules
            if trainer_config.parallelism.pipeline_parallel_degree > 1 and self.num_mtp_modules > 0:
                raise NotImplementedError("DeepSeek-V4 MTP with pipeline parallelism is not supported: set "
                                          "training.num_mtp_modules=0 when PP is enabled")

        def get_nparams_and_flops(self, model, seq_len):
            nparams = emb = routed = 0
            for name, p in model.named_parameters():
                nparams += p.numel()
                if "tok_embeddings" in name:
                    emb += p.numel()
                elif ".moe.experts." in name:
                    routed += p.numel()
            active = nparams - emb - routed + routed * self.moe_args.top_k // max(self.moe_args.num_experts, 1)
            layers = self.n_layers + self.num_mtp_modules
            attn = 0
            for i in range(layers):
                r = _ratio_of(self, i)
                keys = min(self.window_size, seq_len)
                if r == 4:
                    keys += min(self.index_topk, seq_len // 4)
                elif r > 1:
                    keys += seq_len // r // 2
                attn += 12 * self.n_heads * self.head_dim * keys
            return nparams, 6 * active + attn

    def __init__(self, cfg: "DeepSeekV4Model.Config"):
        super().__init__()
        self.config = cfg
        self.n_layers, self.hc_mult = cfg.n_layers, cfg.hc_mult
        self.tok_embeddings = Embedding(cfg.vocab_size, cfg.dim)
        self.layers = ModuleDict()
        for i in range(cfg.n_layers + cfg.num_mtp_modules):
            self.layers[str(i)] = V4Block(i, cfg) if i < cfg.n_layers else V4MTPModule(i, cfg)
        self.norm = RMSNorm(cfg.dim, eps=cfg.norm_eps)
        self.output = Linear(cfg.dim, cfg.vocab_size, bias=False)
        self.register_buffer("freqs_cis", precompute_v4_freqs(cfg, True), persistent=False)
        self.register_buffer("freqs_cis_wo_compressor", precompute_v4_freqs(cfg, False), persistent=False)

    def init_states(self, *, buffer_device=None, **kw):
        buffer_device = buffer_device or self.freqs_cis.device
        with torch.device(buffer_device):
            self.freqs_cis = precompute_v4_freqs(self.config, True, buffer_device)
            self.freqs_cis_wo_compressor = precompute_v4_freqs(self.config, False, buffer_device)
        if self.tok_embeddings is not None:
            nn.init.normal_(self.tok_embeddings.weight)
        for layer in self.layers.values():
            if layer is not None:
                layer.init_states(buffer_device=buffer_device)
        if self.norm is not None:
            nn.init.trunc_normal_(self.norm.weight, mean=1.0, std=0.02)
        if self.output is not None:
            std = self.config.dim ** -0.5
            nn.init.trunc_normal_(self.output.weight, mean=0.0, std=std, a=-3 * std, b=3 * std)

    def _freqs_for(self, layer_id: int):
        return self.freqs_cis if _ratio_of(self.config, layer_id) > 1 else self.freqs_cis_wo_compressor

    def forward(self, tokens, input_ids=None, attention_masks=None, positions=None, mtp_inputs=None):
        """tokens [B, S + num_mtp] ids (first stage) or hidden streams [B, S, hc, D] (later pipeline stages, which
        get the token ids as ``input_ids`` for hash routing).  A packed stream (``attention_masks`` = the packed
        layout) is [1, T] without an MTP tail; its MTP depths read ``mtp_inputs`` [num_mtp, 1, T] instead."""
        cfg = self.config
        raw = None
        if self.tok_embeddings is not None:
            raw = tokens
            s = tokens.shape[1] - (cfg.num_mtp_modules if mtp_inputs is None else 0)
            input_ids = tokens[:, :s].detach().long()
            h = self.tok_embeddings(tokens[:, :s]).unsqueeze(2).repeat(1, 1, self.hc_mult, 1)
        else:
            if not isinstance(input_ids, torch.Tensor) or input_ids.ndim != 2:
                raise RuntimeError("a DeepSeek-V4 pipeline stage needs the token ids as input_ids [B, S]")
            h, input_ids = tokens, input_ids.detach().long()
            s = h.shape[1]
        for key, layer in self.layers.items():
            if int(key) < cfg.n_layers:
                h = layer(h, input_ids, self._freqs_for(int(key)), attention_masks, positions)
        if self.output is None:
            return h
        prev = h
        out = self.output(self.norm(h) if self.norm is not None else h)
        if cfg.num_mtp_modules <= 0:
            return out
        if raw is None:
            raise RuntimeError("DeepSeek-V4 MTP needs the token ids on the stage that owns the output head")
        outs = [out]
        for k in range(cfg.num_mtp_modules):
            emb = self.tok_embeddings(raw[:, k + 1: k + 1 + s] if mtp_inputs is None else mtp_inputs[k])
            layer_id = cfg.n_layers + k
            prev, hn = self.layers[str(layer_id)](emb, prev, input_ids, self.freqs_cis_wo_compressor, attention_masks,
                                                  positions)
            outs.append(self.output(hn))
        return outs
