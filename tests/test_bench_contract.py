"""bench.py on a machine without a GPU: the reference arm (the oracle on the host cores) prints one
JSON line with the agreed keys, and the product arm refuses to run rather than fall back to a CPU path."""
import json
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args, timeout=600):
  return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                        timeout=timeout, cwd=ROOT)


def test_reference_arm_prints_the_contract_line():
  out = _run("--impl", "reference", "--steps", "1", "--warmup", "0")
  assert out.returncode == 0, out.stderr[-2000:]
  lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
  assert len(lines) == 1
  line = json.loads(lines[0])
  assert line["impl"] == "reference" and line["n_gpus"] == 1 and line["steps"] == 1
  for key in ("metric", "value", "unit", "ms_per_step", "higher_is_better", "scaling", "vs_baseline", "dtype", "data",
              "config", "cpu_baseline", "e2e"):
    assert key in line, key
  assert line["unit"] == "TFLOP/s" and line["value"] > 0 and line["higher_is_better"] is True
  assert line["config"]["workload"] == "c2" and "model" not in line["config"]
  base = line["cpu_baseline"]
  assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == pytest.approx(line["value"])
  assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.skipif(torch.cuda.is_available(), reason="this checks the behaviour without a GPU")
def test_product_arm_refuses_to_run_without_a_gpu():
  out = _run("--steps", "1", "--warmup", "3", timeout=300)
  assert out.returncode != 0
  assert "CUDA" in (out.stderr + out.stdout)
  assert not [l for l in out.stdout.splitlines() if l.startswith("{")]
