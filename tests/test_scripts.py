"""User-facing scripts: DCP → Hugging Face export round trip, the chat server's load + decode path, trace summary."""

import importlib.util
import json
import os
import subprocess
import sys

import torch
import torch.distributed.checkpoint as dcp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, path))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_convert_to_hf_and_server_generate(tmp_path):
    from titan_b200.models.qwen3 import Qwen3Model, qwen3_configs

    torch.manual_seed(0)
    cfg = qwen3_configs["debugmodel"]()
    model = Qwen3Model(cfg)
    model.init_states()
    dcp.save(dict(model.state_dict()), checkpoint_id=str(tmp_path / "step-1"))
    conv = _load("scripts/checkpoint_conversion/convert_to_hf.py", "convert_to_hf")
    files = conv.convert_to_hf(tmp_path / "step-1", tmp_path / "hf", "qwen3", "debugmodel", None, "float32")
    assert files == ["model-00001-of-00001.safetensors"]
    index = json.load(open(tmp_path / "hf" / "model.safetensors.index.json"))
    assert "model.layers.0.self_attn.q_norm.weight" in index["weight_map"]
    srv = _load("scripts/infer_server.py", "infer_server")
    tok, loaded = srv.load(str(tmp_path / "hf"), "qwen3", "debugmodel", "byte", "cpu")
    for k, v in model.state_dict().items():
        assert torch.equal(loaded.state_dict()[k], v), k
    ids = tok.encode(tok.apply_chat_template([{"role": "user", "content": "hi"}], add_generation_prompt=True), add_bos=True)
    out = srv.generate(loaded, tok, ids, max_new_tokens=4, temperature=0.0, device="cpu")
    ref = model(torch.tensor([ids]))[0, -1].argmax().item()
    assert len(out) <= 4 and (not out or out[0] == ref)


def test_parse_profiling_data(tmp_path):
    trace = {"traceEvents": [
        {"ph": "X", "cat": "kernel", "name": "tbg::gemm_tcgen05_kernel(...)", "dur": 3000},
        {"ph": "X", "cat": "kernel", "name": "tbg::gemm_tcgen05_kernel(...)", "dur": 1000},
        {"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllGather", "dur": 2000},
        {"ph": "X", "cat": "cpu_op", "name": "aten::mm", "dur": 99999},
    ]}
    f = tmp_path / "rank0.json"
    f.write_text(json.dumps(trace))
    out = subprocess.run([sys.executable, os.path.join(ROOT, "scripts/parse_profiling_data.py"), str(f)],
                         capture_output=True, text=True, check=True).stdout
    assert "6.00 ms on device" in out and "4.00 ms (66.7 %)" in out and "ncclDevKernel_AllGather" in out


def test_launch_scripts_are_shell_clean():
    for s in ("scripts/run_train.sh", "scripts/run_train_multinodes.sh"):
        subprocess.run(["bash", "-n", os.path.join(ROOT, s)], check=True)
        text = open(os.path.join(ROOT, s)).read()
        assert "kill" not in text.replace("pkill", "kill") or "kill -9" not in text
