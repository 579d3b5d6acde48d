"""What bench.py answers without a GPU: the refusal of more than one GPU, the reference arm's
line, and that it fails loudly (no CPU path) when asked to measure without a device."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def run_bench(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=300)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    done = run_bench("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert done.returncode == 2
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_its_unavailable_line_and_exits_0():
    done = run_bench("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert done.returncode == 0
    record = json.loads(done.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference" and isinstance(record["unavailable"], str) and "\n" not in record["unavailable"]
    assert set(record) == {"impl", "unavailable"}


@pytest.mark.skipif(torch.cuda.is_available(), reason="with a device the run measures")
def test_without_a_device_the_run_fails_loudly():
    done = run_bench("--steps", "4", "--warmup", "3")
    assert "no CUDA device" in done.stderr and "value" not in done.stdout
