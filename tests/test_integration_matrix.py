"""The feature-matrix runner itself: its log check, the case table, and one real case on gloo ranks."""

import importlib.util
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_spec = importlib.util.spec_from_file_location("run_matrix", os.path.join(ROOT, "tests", "integration", "run_matrix.py"))
run_matrix = importlib.util.module_from_spec(_spec)
sys.modules["run_matrix"] = run_matrix
_spec.loader.exec_module(run_matrix)


def _log(*losses):
    return "\n".join(f"[titan_b200 r0] 10:00:00 INFO step: {i + 1:2d}  loss: {v}  grad_norm: 1.0" for i, v in enumerate(losses))


def test_assessment_reads_the_log_not_only_the_exit_code():
    j = run_matrix.assess
    assert j(_log(8.1, 7.9, 7.5), 0, 3) == (True, "3 steps")
    assert j(_log(8.1, 7.9), 0, 3)[0] is False                       # too few steps
    assert j(_log(8.1, "nan", 7.5), 0, 3) == (False, "loss is NaN / Inf at step 2")
    assert j(_log(8.1, 7.9, 7.5), 1, 3) == (False, "exit code 1")
    assert j(_log(8.1, 7.9, 7.5), None, 3) == (False, "timeout")
    assert j(_log(8.1, 7.9, 7.5) + "\nTraceback (most recent call last):\n", 0, 3)[0] is False
    assert j(_log(8.1, 7.9, 7.5) + "\nRuntimeError: boom", 0, 3)[0] is False
    # warnings that mention errors are not failures
    ok = _log(8.1, 7.9, 7.5) + "\n[rank0]:W1125 20:40:17.753000 1 x.py:350] this is error-prone\nUserWarning: error x"
    assert j(ok, 0, 3)[0] is True


def test_case_table_names_real_recipes():
    from titan_b200.config.manager import resolve_recipe

    names = [c.name for c in run_matrix.CASES]
    assert len(names) == len(set(names)) and len(names) >= 20
    for c in run_matrix.CASES:
        resolve_recipe(c.module, c.config)
    families = {c.module for c in run_matrix.CASES}
    assert {"llama3", "deepseek_v3", "deepseek_v32", "deepseek_v4", "qwen3"} <= families


def test_one_case_end_to_end_on_gloo(tmp_path):
    case = next(c for c in run_matrix.CASES if c.name == "deepseek_v32_cp")
    rec = run_matrix.run_case(case, "cpu", str(tmp_path), 29791, 600)
    assert rec["status"] == "passed", open(tmp_path / "deepseek_v32_cp.log").read()[-3000:]
