"""User-facing scripts: DCP → Hugging Face export round trip, the chat server's load + decode path, trace summary."""

import importlib.util
import json
import os
import subprocess
import sys

import pytest
import torch
import torch.distributed.checkpoint as dcp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, path))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod  # dataclasses resolve string annotations through sys.modules
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


def _fake_snapshot(extra_activation=0):
    fr = lambda f, n, line=1: {"filename": f, "name": n, "line": line}  # noqa: E731
    act = [fr("torch/nn/modules/module.py", "_call_impl"), fr("titan_b200/models/llama3/model.py", "forward", 88)]
    opt = [fr("titan_b200/optim/fused_adamw.py", "_init_group", 40)]
    par = [fr("titan_b200/models/llama3/model.py", "init_weights", 12)]
    com = [fr("torch/distributed/distributed_c10d.py", "all_gather_into_tensor", 3)]
    blocks = [
        {"size": 512 << 20, "state": "active_allocated", "frames": par},
        {"size": 1024 << 20, "state": "active_allocated", "frames": opt},
        {"size": (256 << 20) + extra_activation, "state": "active_allocated", "frames": act},
        {"size": 64 << 20, "state": "active_allocated", "frames": com},
        {"size": 32 << 20, "state": "active_pending_free", "frames": act},
        {"size": 100 << 20, "state": "inactive"},
        {"size": 512 << 10, "state": "inactive"},
    ]
    total = sum(b["size"] for b in blocks)
    traces = [{"action": "alloc", "size": 512 << 20, "frames": par},
              {"action": "alloc", "size": 1024 << 20, "frames": opt},
              {"action": "alloc", "size": 700 << 20, "frames": act},
              {"action": "free_requested", "size": 700 << 20},
              {"action": "free_completed", "size": 700 << 20},
              {"action": "alloc", "size": 256 << 20, "frames": act}]
    return {"segments": [{"device": 0, "total_size": total, "blocks": blocks},
                         {"device": 0, "total_size": 20 << 20, "blocks": [{"size": 20 << 20, "state": "inactive"}]}],
            "device_traces": [traces]}


def test_memory_snapshot_analyser(tmp_path, capsys):
    import pickle

    mod = _load("scripts/analyze_memory_snapshot.py", "analyze_memory_snapshot")
    paths = []
    for i, extra in enumerate((0, 128 << 20, 256 << 20)):
        p = tmp_path / f"s{i}.pickle"
        p.write_bytes(pickle.dumps(_fake_snapshot(extra)))
        paths.append(str(p))
    r = mod.analyze(mod.load_snapshot(paths[0]), paths[0], top_n=3)
    assert r.allocated == (512 + 1024 + 256 + 64) << 20 and r.active == r.allocated + (32 << 20)
    assert r.by_category["optimizer"] == 1024 << 20 and r.by_category["parameter"] == 512 << 20
    assert r.by_category["activation"] == 256 << 20 and r.by_category["communication"] == 64 << 20
    assert [b.category for b in r.top_blocks] == ["optimizer", "parameter", "activation"]
    assert r.top_blocks[2].frames == ["titan_b200/models/llama3/model.py:forward:88"]  # torch plumbing frames dropped
    f = r.fragmentation
    assert (f.free_blocks, f.small_free_blocks, f.largest_free, f.segments_fully_free) == (3, 1, 100 << 20, 1)
    t = r.timeline
    assert t.peak_bytes == (512 + 1024 + 700) << 20 and t.peak_event == 2 and t.end_bytes == (512 + 1024 + 256) << 20
    assert t.before_peak[0]["category"] == "optimizer"
    assert mod.main([paths[0]]) == 0 and "live bytes by kind" in capsys.readouterr().out
    assert mod.main(paths[:2]) == 0
    assert "activation" in capsys.readouterr().out.split("minus")[1]
    assert mod.main(paths) == 0 and "a leak" in capsys.readouterr().out
    assert mod.main([paths[0], "--json"]) == 0
    import json as _json

    assert _json.loads(capsys.readouterr().out)[0]["reserved"] == r.reserved
    bad = tmp_path / "bad.pickle"
    bad.write_bytes(pickle.dumps([1, 2]))
    with pytest.raises(ValueError):
        mod.load_snapshot(str(bad))


def test_training_log_summary_compare_plot(tmp_path, capsys):
    mod = _load("scripts/training_log.py", "training_log")
    line = ("[titan] 2026-01-01 step: {s:2d}  loss: {l:7.4f}  grad_norm: {g:7.4f}  memory: 41.07GiB(22.94%)  "
            "tps: {t:,}  tflops: 917.21  mfu: 40.77%  elapsed_time_per_step: 0.4101s\n")
    a, b, c = tmp_path / "a.log", tmp_path / "b.log", tmp_path / "c.log"
    a.write_text("noise\n" + "".join(line.format(s=s, l=8.0 - 0.1 * s, g=1.0 + 0.01 * s, t=19000 + s) for s in range(1, 11)))
    b.write_text("".join(line.format(s=s, l=8.0 - 0.1 * s, g=1.0 + 0.01 * s, t=15000) for s in range(1, 13)))
    c.write_text("".join(line.format(s=s, l=8.0 - 0.1 * s + (0.01 if s >= 7 else 0), g=1.0 + 0.01 * s, t=15000)
                         for s in range(1, 11)))
    rec = mod.parse_log(str(a))
    assert sorted(rec) == list(range(1, 11)) and rec[3]["tps"] == 19003 and rec[3]["memory_pct"] == 22.94
    s = mod.summarize(rec, skip=5)
    assert s["steps_logged"] == 10 and s["tps_best"] == 19010 and abs(s["tps_mean"] - 19008) < 1e-9
    assert abs(s["last_loss"] - 7.0) < 1e-9 and s["memory_gib_peak"] == 41.07
    out = tmp_path / "rep"
    assert mod.main(["compare", "--baseline", str(a), "--candidate", str(b), "--output", str(out)]) == 0
    rep = json.loads((out / "compare_report.json").read_text())
    assert rep["passed"] and rep["steps_compared"] == 10 and rep["only_in_candidate"] == [11, 12]
    assert mod.main(["compare", "--baseline", str(a), "--candidate", str(c), "--output", str(out)]) == 1
    rep = json.loads((out / "compare_report.json").read_text())
    assert rep["metrics"]["loss"]["first_step_over_tolerance"] == 7 and rep["metrics"]["grad_norm"]["passed"]
    assert "**FAIL**" in (out / "compare_report.md").read_text()
    assert mod.main(["compare", "--baseline", str(a), "--candidate", str(c), "--output", str(out), "--tolerance", "0.1"]) == 0
    svg = tmp_path / "p.svg"
    assert mod.main(["plot", "--log-a", str(a), "--log-b", str(c), "--output", str(svg), "--smooth", "0.5"]) == 0
    text = svg.read_text()
    assert text.startswith("<svg") and text.count("<polyline") == 9 and "c.log - a.log" in text  # 3 x (2 curves + diff)
    assert mod.ema([1.0, 3.0], 0.5) == [1.0, 2.0] and mod.main(["summary", str(a)]) == 0
