"""The benchmark's output contract on a real GPU: one short default run and one run of each
whole-sequence workload, each must print exactly one JSON line with the agreed keys."""
from __future__ import annotations

import json
import pathlib
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = pathlib.Path(__file__).resolve().parents[1]
BASE_KEYS = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
             "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline"}


def _run(*flags: str) -> dict:
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), *flags], capture_output=True, text=True, timeout=900,
                         cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [line for line in out.stdout.splitlines() if line.strip()]
    assert len(lines) == 1, lines
    return json.loads(lines[0])


def _check_common(line: dict, steps: int) -> None:
    assert BASE_KEYS <= set(line), BASE_KEYS - set(line)
    assert line["n_gpus"] == 1 and line["steps"] == steps and line["warmup"] >= 3
    assert line["value"] > 0 and line["ms_per_step"] > 0 and line["higher_is_better"] is True
    assert line["unit"] == "tokens/s" and line["data"] == "synthetic" and line["vs_baseline"] is None
    assert "workload" in line["config"] and "model" not in line["config"]
    e2e = line["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert line["gpu_launches"] > 0
    roof = line["roofline"]
    assert {"bound", "achieved", "peak", "unit", "frac", "traffic"} <= set(roof)
    assert roof["bound"] in ("hbm", "tensor") and abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9
    clocks = line["clocks"]
    assert clocks["sm_mhz"] > 0 and clocks["sm_max_mhz"] >= clocks["sm_mhz"] * 0.5 and isinstance(clocks["reasons"], list)


def test_default_decode_line():
    line = _run("--steps", "8", "--warmup", "3", "--no-cfg5", "--no-extras")
    _check_common(line, 8)
    assert line["dtype"] == "bf16" and line["scaling"] == "weak"
    assert line["metric"] == "relation decode tokens/s at ctx512 K=8"
    cpu = line["cpu_baseline"]
    assert {"value", "unit", "cores", "kind", "sample"} <= set(cpu) and cpu["kind"] in ("port", "reference")
    assert cpu["value"] > 0 and cpu["cores"] >= 1
    assert line["launches_per_step"] == 16 and line["gpu_launches"] == 16 * 8
    assert "l2" in line["config"]


@pytest.mark.parametrize("workload", ["cfg3", "cfg4"])
def test_whole_sequence_workload_lines(workload):
    line = _run("--workload", workload, "--steps", "3", "--warmup", "3")
    _check_common(line, 3)
    assert workload in line["config"]["workload"]
    assert line["cpu_baseline"]["value"] > 0


def test_reference_arm_line():
    line = _run("--impl", "reference", "--steps", "1", "--warmup", "1")
    assert line["impl"] == "reference" and line["value"] > 0 and line["unit"] == "tokens/s"
    assert line["cpu_baseline"]["value"] == line["value"] and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
