"""bench.py's output contract, checked on the CPU arm (the GPU arm needs a B200): one JSON line with the keys the
measurement contract names, and a loud failure - not a silent CPU run - when the GPU arm is asked for without a GPU."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_contract_line():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600, cwd=str(ROOT))
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [ln for ln in p.stdout.strip().splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "vs_baseline",
                "dtype", "data", "config", "impl", "cpu_baseline", "e2e"):
        assert key in d, key
    assert d["impl"] == "reference" and d["metric"] == "w8a16_decode_gemv_hbm_GBps" and d["unit"] == "GB/s"
    assert d["vs_baseline"] is None and d["data"] == "synthetic" and d["value"] > 0
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0 and d["e2e"]["value"] == d["value"]
    assert "workload" in d["config"] and "model" not in d["config"]
    c1 = d["cpu_baseline"]["config1"]          # BASELINE config 1 exactly, dequant and matmul timed separately
    assert "N=K=4096" in c1["what"] and c1["ms_dequant"] > 0 and c1["ms_matmul"] > 0 and c1["GBps"] > 0


@pytest.mark.skipif(torch.cuda.is_available(), reason="only meaningful on a box without a GPU")
def test_gpu_arm_refuses_to_run_without_a_gpu():
    p = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--steps", "1", "--warmup", "1"], capture_output=True, text=True,
                       timeout=300, cwd=str(ROOT))
    assert p.returncode != 0
    assert "no CPU path" in (p.stderr + p.stdout)
