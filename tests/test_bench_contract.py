"""What can be checked of the benchmark driver without a GPU: the reference arm's answer and the
argument parser's defaults."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_reference_arm_reports_unavailable():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                         capture_output=True, text=True, timeout=120, cwd=str(ROOT))
    assert out.returncode == 0, out.stderr
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" in line and len(line["unavailable"]) > 20


def test_bench_needs_a_gpu_and_says_so():
    import torch
    if torch.cuda.is_available():
        return
    out = subprocess.run([sys.executable, str(ROOT / "bench.py")], capture_output=True, text=True, timeout=120, cwd=str(ROOT))
    assert out.returncode != 0 and "CUDA device" in (out.stderr + out.stdout)
