import torch

from titan_b200.converters import convert_utils
from titan_b200.converters.rms_norm import FusedRMSNorm
from titan_b200.models.common.layers import RMSNorm
from titan_b200.models.llama3 import llama3_configs
from titan_b200.protocols import converter as conv


def _tiny():
    cfg = llama3_configs["debugmodel"]()
    cfg.n_layers = 2
    return cfg.build()


def test_registry_names_and_aliases():
    names = conv.converter_names()
    for n in ("b200_rms_norm", "b200_rope", "b200_swiglu", "b200_cross_entropy", "b200_linear"):
        assert n in names
    assert conv.get_model_converter_config("npu_rms_norm").name == "b200_rms_norm"
    lst = [conv.get_model_converter_config("npu_rope")]
    assert conv.has_converter(lst, "b200_rope") and conv.has_converter(lst, "npu_rope")
    assert not conv.has_converter(lst, "b200_swiglu")


def test_rms_norm_converter_keeps_params_and_numerics():
    model = _tiny()
    before = dict(model.named_parameters())
    c = conv.ModelConvertersContainer([conv.get_model_converter_config("b200_rms_norm")])
    c.convert(model)
    norms = [m for m in model.modules() if isinstance(m, RMSNorm)]
    assert norms and all(isinstance(m, FusedRMSNorm) for m in norms)
    after = dict(model.named_parameters())
    assert before.keys() == after.keys() and all(before[k] is after[k] for k in before)
    x = torch.randn(3, 5, 256)
    ref = torch.nn.functional.rms_norm(x, (256,), norms[0].weight, norms[0].eps)
    torch.testing.assert_close(norms[0](x), ref)


def test_rope_converter_rebinds_from_imports():
    import titan_b200.models.llama3.model as lm
    from titan_b200.converters import rope as rope_conv
    from titan_b200.ops import rope as fused

    model = _tiny()
    conv.ModelConvertersContainer([conv.get_model_converter_config("b200_rope")]).convert(model)
    try:
        assert lm.apply_rotary_emb_complex is fused.apply_rotary_emb_complex
        tokens = torch.randint(0, 2048, (2, 16))
        with torch.device("cpu"):
            model.init_states()
        out = model(tokens)
        assert out.shape == (2, 16, 2048) and torch.isfinite(out).all()
    finally:
        rope_conv.restore()
    assert lm.apply_rotary_emb_complex is not fused.apply_rotary_emb_complex


def test_replace_utils():
    model = _tiny()
    hits = convert_utils.find_modules(model, r"RMSNorm")
    assert len(hits) == 2 * 2 + 1
    n = convert_utils.replace_modules(model, r"FeedForward", lambda old: torch.nn.Identity())
    assert n == 2 and isinstance(model.layers["0"].feed_forward, torch.nn.Identity)
    classes = convert_utils.find_methods(model, r"Attention", "forward")
    assert len(classes) == 1


def test_unknown_converter_raises():
    import pytest

    with pytest.raises(KeyError):
        conv.ModelConvertersContainer(["no_such_converter"])
