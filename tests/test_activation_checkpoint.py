"""Selective activation checkpointing policies: the upstream rule recomputes every second matmul, the
`op_save_all_mm` rule recomputes none; both give the gradients of the unwrapped model."""

import torch
from torch.utils._python_dispatch import TorchDispatchMode

from titan_b200.config.configs import ActivationCheckpointConfig
from titan_b200.models.llama3 import Llama3Model, llama3_configs
from titan_b200.parallel.activation_checkpoint import apply_ac


class _CountMM(TorchDispatchMode):
    def __init__(self):
        super().__init__()
        self.n = 0

    def __torch_dispatch__(self, func, types, args=(), kwargs=None):
        if func == torch.ops.aten.mm.default:
            self.n += 1
        return func(*args, **(kwargs or {}))


def _run(option):
    torch.manual_seed(0)
    cfg = llama3_configs["debugmodel"]()
    cfg.max_seq_len = 64
    cfg.n_layers = 2
    model = Llama3Model(cfg)
    model.init_states()
    if option is not None:
        apply_ac(model, ActivationCheckpointConfig(mode="selective", selective_ac_option=option))
    tok = torch.randint(0, cfg.vocab_size, (2, 64))
    with _CountMM() as c:
        model(tok).float().logsumexp(-1).mean().backward()
    grads = torch.cat([p.grad.flatten() for p in model.parameters()])
    return c.n, grads


def test_save_all_mm_recomputes_no_matmul():
    n_plain, g_plain = _run(None)
    n_all, g_all = _run("op_save_all_mm")
    n_half, g_half = _run("op")
    assert n_all == n_plain            # nothing recomputed
    assert n_half > n_plain            # the upstream rule runs some forward matmuls twice
    assert torch.allclose(g_all, g_plain, atol=1e-6) and torch.allclose(g_half, g_plain, atol=1e-6)
