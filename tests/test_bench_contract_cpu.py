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
    monkeypatch.setattr(bench, "cpu_decode_sample", lambda steps, layers=1, threads=None: (1.5, 8, "stub sample", 0.16))
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
    assert d["ms_per_step"] == pytest.approx(0.16 * 32 * 1e3)


def test_reference_arm_is_silent_on_other_ranks(monkeypatch, capsys):
    monkeypatch.setattr(bench, "cpu_decode_sample", lambda *a, **k: pytest.fail("rank 1 must not run the sample"))
    monkeypatch.setenv("RANK", "1")
    bench.run_reference(types.SimpleNamespace(steps=4, warmup=3, gpus=2))
    assert capsys.readouterr().out.strip() == ""


def test_launch_count_and_workloads():
    assert bench.kernel_launches_per_step(32, 8, 1) == 8 * 32 + 4
    assert bench.kernel_launches_per_step(32, 8, 4) == 8 * 32 + 4
    assert bench.kernel_launches_per_step(40, 32, 1) == 8 * 40 + 4        # deferred chain up to 64 rows on one GPU
    assert bench.kernel_launches_per_step(80, 64, 4) == 16 * 80 + 4       # tensor parallel above 16 rows
    assert set(bench.WORKLOADS) == {"llama7b", "baichuan13b", "llama65b"}
    assert bench.WORKLOADS["llama7b"] is None and bench.BATCH == 8 and bench.PROMPT == 512
