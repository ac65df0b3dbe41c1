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


def test_traffic_figure_follows_the_kernel_source(monkeypatch, tmp_path):
    """roofline.traffic comes from the figures file beside the committed ncu summary and is only reported while the
    kernel source is the one it was captured on.  The committed pair must be in step (else the bench line would carry
    null), and a changed source must demote the figure to `traffic_stale`."""
    sys.path.insert(0, str(ROOT))
    import bench
    got = bench.capture_traffic()
    assert got["traffic"] is not None and got["traffic"] >= got["traffic_algorithmic_bytes"] > 0, got
    assert got["traffic"] < 1.2 * got["traffic_algorithmic_bytes"], "DRAM traffic far above the algorithmic bytes means re-reads"
    # same figures, different source: stale
    fake = tmp_path / "repo"
    (fake / "profiles").mkdir(parents=True)
    (fake / "vllm_fp8_w8a16_sm70_b200" / "csrc").mkdir(parents=True)
    (fake / "profiles" / "k_gemm_tc_decode_gate_up_m16.json").write_text((ROOT / "profiles" / "k_gemm_tc_decode_gate_up_m16.json").read_text())
    (fake / "vllm_fp8_w8a16_sm70_b200" / "csrc" / "gemm_tc.cu").write_text("// something else\n")
    monkeypatch.setattr(bench, "ROOT", fake)
    stale = bench.capture_traffic()
    assert stale["traffic"] is None and stale["traffic_stale"] == got["traffic"] and "changed" in stale["traffic_note"]
