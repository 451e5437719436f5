"""Optimizer subsystem on CPU: swap / virtual / Muon / dispatcher / LR schedule."""

import copy

import pytest
import torch
import torch.nn as nn

from titan_b200.config.configs import LRSchedulerConfig, OptimizerConfig
from titan_b200.optim import containers, muon, swap_optimizer, virtual_optimizer


def _model():
    torch.manual_seed(0)
    return nn.Sequential(nn.Linear(16, 32, bias=False), nn.LayerNorm(32), nn.Linear(32, 8))


def _train(model, opt, steps=3, seed=1):
    g = torch.Generator().manual_seed(seed)
    for _ in range(steps):
        opt.zero_grad()
        x = torch.randn(4, 16, generator=g)
        model(x).pow(2).mean().backward()
        opt.step()


def test_dispatcher_rejects_swap_plus_virtual():
    cfg = OptimizerConfig(swap_optimizer=True, virtual_optimizer=True)
    with pytest.raises(ValueError):
        containers.build_optimizers([_model()], cfg)
    with pytest.raises(NotImplementedError):
        containers.build_optimizers([_model()], OptimizerConfig(name="SGD"))


def test_swap_optimizer_matches_adamw_and_keeps_state_on_host():
    ref_model, model = _model(), _model()
    cfg = OptimizerConfig(lr=1e-2, weight_decay=0.1, swap_optimizer=True, swap_optimizer_times=3)
    opt = containers.build_optimizers([model], cfg)
    assert isinstance(opt, swap_optimizer.SwapOptimizersContainer)
    ref = torch.optim.AdamW(ref_model.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    _train(model, opt)
    _train(ref_model, ref)
    for p, r in zip(model.parameters(), ref_model.parameters()):
        torch.testing.assert_close(p, r, rtol=1e-5, atol=1e-6)
    inner = opt.optimizers[0]
    assert inner.m_host.device.type == "cpu" and len(inner.slices) >= 2
    sd = opt.state_dict()
    assert "state.0.weight.exp_avg" in sd and "param_groups.0.weight.lr" in sd and "state.2.bias.step" in sd
    assert float(sd["state.0.weight.step"]) == 3


def test_swap_optimizer_state_dict_roundtrip_and_transactional_load():
    model = _model()
    cfg = OptimizerConfig(lr=1e-2, swap_optimizer=True, swap_optimizer_times=2)
    opt = containers.build_optimizers([model], cfg)
    _train(model, opt)
    sd = {k: (v.clone() if torch.is_tensor(v) else copy.deepcopy(v)) for k, v in opt.state_dict().items()}
    model2 = _model()
    opt2 = containers.build_optimizers([model2], cfg)
    opt2.load_state_dict(sd)
    torch.testing.assert_close(opt2.optimizers[0].m_host, opt.optimizers[0].m_host)
    assert opt2.optimizers[0].steps == {id(p): 3 for p in opt2.optimizers[0].params_list}
    # a broken entry must leave the previous state untouched
    before = opt2.optimizers[0].v_host.clone()
    bad = dict(sd)
    bad["state.2.weight.exp_avg_sq"] = torch.zeros(3, 3)
    with pytest.raises(ValueError):
        opt2.load_state_dict(bad)
    torch.testing.assert_close(opt2.optimizers[0].v_host, before)


def test_virtual_allocator_budget_and_size_parsing():
    alloc = virtual_optimizer.VirtualAllocator(budget_gb=1e-6, pin=False)  # 1000 bytes
    assert alloc.try_alloc((100,)) is not None  # 400 B
    assert alloc.try_alloc((100,)) is not None  # 800 B
    assert alloc.try_alloc((100,)) is None
    assert virtual_optimizer.parse_virtual_size("all", 2) == [65.0, 65.0]
    assert virtual_optimizer.parse_virtual_size(3, 2) == [3.0, 3.0]
    assert virtual_optimizer.parse_virtual_size([1, 2], 2) == [1.0, 2.0]
    with pytest.raises(ValueError):
        virtual_optimizer.parse_virtual_size([1, 2, 3], 2)


def test_virtual_optimizer_matches_adamw_on_cpu():
    ref_model, model = _model(), _model()
    cfg = OptimizerConfig(lr=1e-2, weight_decay=0.1, virtual_optimizer=True, virtual_optimizer_size=5e-6)
    opt = containers.build_optimizers([model], cfg)
    ref = torch.optim.AdamW(ref_model.parameters(), lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    _train(model, opt)
    _train(ref_model, ref)
    for p, r in zip(model.parameters(), ref_model.parameters()):
        torch.testing.assert_close(p, r, rtol=1e-5, atol=1e-6)
    inner = opt.optimizers[0]
    assert 0 < len(inner.virtual_params) < len(list(model.parameters()))  # the budget covered only the first tensors


@pytest.mark.parametrize("shape", [(64, 32), (32, 64), (3, 16, 48)])
@pytest.mark.parametrize("hybrid", [False, True])
def test_newton_schulz_orthogonalises(shape, hybrid):
    torch.manual_seed(0)
    g = torch.randn(*shape)
    u = muon.zeropower_via_newtonschulz5(g, steps=5, hybrid_ns=hybrid).float()
    s = torch.linalg.svdvals(u)
    assert s.max() < 1.3 and s.min() > (0.85 if hybrid else 0.4), (s.min(), s.max())
    assert u.shape == g.shape
    with pytest.raises(ValueError):
        muon.zeropower_via_newtonschulz5(torch.randn(4))


def test_normalise_update_rules():
    u = torch.ones(8, 2)
    assert torch.allclose(muon.normalise_update(u, "original"), u * 2.0)
    assert torch.allclose(muon.normalise_update(u, "match_rms_adamw"), u * 0.18 * 8 ** 0.5)
    assert torch.allclose(muon.normalise_update(u.t(), None), u.t())


def test_muon_split_and_step():
    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.tok_embeddings = nn.Embedding(10, 8)
            self.wq = nn.Linear(8, 8, bias=False)
            self.norm = nn.LayerNorm(8)
            self.experts_w = nn.Parameter(torch.randn(2, 8, 8))
            self.output = nn.Linear(8, 10, bias=False)

        def forward(self, t):
            h = self.norm(self.wq(self.tok_embeddings(t)))
            return self.output(h @ self.experts_w[0])

    torch.manual_seed(0)
    m = M()
    mp, mn, ap, an = muon.split_parameters_for_muon([m])
    assert set(mn) == {"wq.weight", "experts_w"} and "tok_embeddings.weight" in an and "output.weight" in an
    cfg = OptimizerConfig(name="Muon", lr=1e-2, weight_decay=0.0,
                          extra_param_group_split_rules=[{"str_match": "experts", "backend_steps": 3}])
    opt = containers.build_optimizers([m], cfg)
    assert isinstance(opt, muon.MuonHybridOptimizersContainer)
    assert opt.muon[0].param_groups[0]["backend_steps"] == 3 and len(opt.muon[0].param_groups) == 2
    before = m.wq.weight.detach().clone()
    t = torch.randint(0, 10, (4, 5))
    m(t).pow(2).mean().backward()
    opt.step()
    delta = (m.wq.weight.detach() - before)
    # update = -lr * 0.18 * sqrt(8) * (near-orthogonal matrix): every singular value close to that constant
    s = torch.linalg.svdvals(delta) / (1e-2 * 0.18 * 8 ** 0.5)
    assert s.max() < 1.4 and s.median() > 0.3  # the tiny batch makes the gradient nearly rank-deficient
    sd = opt.state_dict()
    assert any(k.endswith("momentum_buffer") for k in sd)
    sched = containers.build_lr_schedulers(opt, LRSchedulerConfig(warmup_steps=2), 10)
    assert len(sched.schedulers) == 2
    sched.step()


class _MuonNet(nn.Module):
    def __init__(self):
        super().__init__()
        self.tok_embeddings = nn.Embedding(10, 8)
        self.wq = nn.Linear(8, 16, bias=False)
        self.wk = nn.Linear(16, 8, bias=False)
        self.norm = nn.LayerNorm(8)
        self.experts_w = nn.Parameter(torch.randn(2, 8, 8))
        self.output = nn.Linear(8, 10, bias=False)

    def forward(self, t):
        h = self.norm(self.wk(self.wq(self.tok_embeddings(t))))
        return self.output(h @ self.experts_w[0])


def _muon_steps(opt, m, n=3):
    g = torch.Generator().manual_seed(5)
    for _ in range(n):
        opt.zero_grad()
        m(torch.randint(0, 10, (4, 5), generator=g)).pow(2).mean().backward()
        opt.step()


def test_swap_muon_matches_resident_muon_and_checkpoints_every_state():
    """Swap-Muon keeps the Muon momenta AND the AdamW moments in host arenas: same parameters as the resident
    optimizer after 3 steps, nothing left in `optimizer.state` between steps, and a state dict with every momentum and
    moment that a resident optimizer loads (and the other way round)."""
    torch.manual_seed(0)
    ref_m = _MuonNet()
    m = copy.deepcopy(ref_m)
    base = dict(name="Muon", lr=1e-2, weight_decay=0.01)
    ref = containers.build_optimizers([ref_m], OptimizerConfig(**base))
    opt = containers.build_optimizers([m], OptimizerConfig(**base, swap_optimizer=True, swap_merge_buckets=1))
    assert isinstance(opt.muon[0], muon.SwapDistributedMuon)
    assert len(opt.muon[0]._merge_groups(list(opt.muon[0].params_list))) == 3   # one matrix per merge group here
    _muon_steps(ref, ref_m)
    _muon_steps(opt, m)
    for (n, a), b in zip(ref_m.named_parameters(), m.parameters()):
        torch.testing.assert_close(b, a, rtol=1e-5, atol=1e-6, msg=lambda s, n=n: f"{n}: {s}")
    assert all("momentum_buffer" not in st for st in opt.muon[0].state.values())
    sd = opt.state_dict()
    assert {"state.wq.weight.momentum_buffer", "state.experts_w.momentum_buffer", "state.norm.weight.exp_avg",
            "state.output.weight.exp_avg_sq", "state.tok_embeddings.weight.step"} <= set(sd)
    ref_sd = ref.state_dict()
    torch.testing.assert_close(sd["state.wq.weight.momentum_buffer"], ref_sd["state.wq.weight.momentum_buffer"])
    torch.testing.assert_close(sd["state.norm.weight.exp_avg"], ref_sd["state.norm.weight.exp_avg"])
    # resident checkpoint -> swapped optimizer, one more step on both: still equal
    torch.manual_seed(0)
    m2 = copy.deepcopy(ref_m)
    opt2 = containers.build_optimizers([m2], OptimizerConfig(**base, swap_optimizer=True, swap_merge_buckets=2))
    opt2.load_state_dict(ref_sd)
    _muon_steps(ref, ref_m, 1)
    _muon_steps(opt2, m2, 1)
    for a, b in zip(ref_m.parameters(), m2.parameters()):
        torch.testing.assert_close(b, a, rtol=1e-5, atol=1e-6)
    # swapped checkpoint -> resident optimizer
    m3 = copy.deepcopy(m)
    opt3 = containers.build_optimizers([m3], OptimizerConfig(**base))
    opt3.load_state_dict(sd)
    torch.testing.assert_close(opt3.state_dict()["state.wk.weight.momentum_buffer"],
                               sd["state.wk.weight.momentum_buffer"])


def test_lr_schedule_shape():
    f = lambda s, **k: containers.linear_warmup_stable_decay(s, warmup_steps=2, stable_steps=3, decay_steps=4, **k)
    vals = [f(s, decay_type="linear", min_lr_factor=0.1) for s in range(9)]
    assert vals[0] < vals[1] < 1.0 and vals[2] == vals[4] == 1.0 and vals[5] > vals[8] >= 0.1
    assert abs(f(8, decay_type="cosine", min_lr_factor=0.0)) < 1e-6
    with pytest.raises(ValueError):
        f(8, decay_type="exp", min_lr_factor=0.0)
