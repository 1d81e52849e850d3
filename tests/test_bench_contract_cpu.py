"""bench.py's contract, as far as it can be checked without a GPU: the reference arm's JSON line (with the CPU
sample replaced by a stub so the test takes no time), the launch-count claim and the workload table."""
import json
import os
import sys
import types

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402


def test_reference_arm_prints_one_contract_line(monkeypatch, capsys):
    stub = {"tok_s": 1.5, "threads": 8, "sample": "stub sample", "step_s_measured": 5.12, "step_s": 5.12,
            "layers_run": 32, "layers": 32, "steps": 4}
    monkeypatch.setattr(bench, "cpu_decode_sample", lambda steps, warmup=1, budget_s=15.0, threads=None: dict(stub))
    monkeypatch.setenv("RANK", "0")
    bench.run_reference(types.SimpleNamespace(steps=4, warmup=3, gpus=1))
    lines = [ln for ln in capsys.readouterr().out.splitlines() if ln.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == bench.METRIC and d["unit"] == "tokens/s"
    assert d["value"] == 1.5 and d["higher_is_better"] is True and d["vs_baseline"] is None
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] == 8
    assert d["e2e"] == {"value": 1.5, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert d["config"]["workload"] == bench.WORKLOAD
    # both arms print the same config keys, so the driver can tell that they ran the same thing
    assert d["config"] == bench.bench_config(32, 1, True, 3, 4)
    assert d["ms_per_step"] == pytest.approx(5120.0) and d["extrapolated"] is None


def test_reference_arm_says_when_it_extrapolates(monkeypatch, capsys):
    stub = {"tok_s": 1.5, "threads": 8, "sample": "stub sample", "step_s_measured": 1.28, "step_s": 5.12,
            "layers_run": 8, "layers": 32, "steps": 128}
    monkeypatch.setattr(bench, "cpu_decode_sample", lambda *a, **k: dict(stub))
    monkeypatch.setenv("RANK", "0")
    bench.run_reference(types.SimpleNamespace(steps=128, warmup=3, gpus=1))
    d = json.loads(capsys.readouterr().out.strip())
    assert d["extrapolated"] == {"layers_run": 8, "factor": 4.0, "ms_per_step_measured": 1280.0}


def test_cpu_sample_runs_every_layer_when_the_budget_allows(monkeypatch):
    """The sample itself, on a toy architecture so that it takes a moment: all layers run, nothing is scaled."""
    monkeypatch.setattr(bench, "CFG", dict(bench.CFG, hidden_size=256, num_attention_heads=2, intermediate_size=512,
                                           num_hidden_layers=3))
    monkeypatch.setattr(bench, "PROMPT", 8)
    monkeypatch.setattr(bench, "BATCH", 2)
    r = bench.cpu_decode_sample(2, warmup=1, budget_s=60.0, threads=2)
    assert r["layers_run"] == 3 and r["layers"] == 3 and r["step_s"] == r["step_s_measured"] and r["tok_s"] > 0
    r = bench.cpu_decode_sample(2, warmup=1, budget_s=0.0, threads=2)
    assert r["layers_run"] == 1 and r["step_s"] == pytest.approx(3 * r["step_s_measured"])


def test_reference_arm_is_silent_on_other_ranks(monkeypatch, capsys):
    monkeypatch.setattr(bench, "cpu_decode_sample", lambda *a, **k: pytest.fail("rank 1 must not run the sample"))
    monkeypatch.setenv("RANK", "1")
    bench.run_reference(types.SimpleNamespace(steps=4, warmup=3, gpus=2))
    assert capsys.readouterr().out.strip() == ""


def test_launch_count_and_workloads():
    assert bench.kernel_launches_per_step(32, 8, 1) == 8 * 32 + 5         # int8 lm_head: GEMM + fused argmax
    assert bench.kernel_launches_per_step(32, 8, 4) == 8 * 32 + 5
    assert bench.kernel_launches_per_step(40, 32, 1) == 8 * 40 + 5        # deferred chain up to 64 rows
    assert bench.kernel_launches_per_step(80, 64, 4) == 8 * 80 + 5        # ... with tensor parallelism too
    assert bench.kernel_launches_per_step(80, 128, 4) == 16 * 80 + 5
    assert set(bench.WORKLOADS) == {"llama7b", "baichuan13b", "llama65b"}
    assert bench.WORKLOADS["llama7b"] is None and bench.BATCH == 8 and bench.PROMPT == 512
