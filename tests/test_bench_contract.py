"""What bench.py promises: more than one GPU is refused with one line and exit code 2; without a GPU the reference arm
says so in one JSON line; on a GPU it runs the reference's own language path and prints the contract's line."""

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=600)


def test_more_than_one_gpu_is_refused_with_one_line_and_exit_code_2():
    r = _run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    assert len(r.stdout.strip().splitlines()) == 1 and "one GPU" in r.stdout


def test_reference_arm_without_a_gpu_says_that_it_needs_one():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present: the arm runs (see the gpu test)")
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "no CUDA device" in line["unavailable"] and "\n" not in line["unavailable"]


@pytest.mark.gpu
def test_reference_arm_runs_the_reference_language_path_on_the_gpu():
    """Two layers of the bench's sizes through the reference's LanguageModel, KVCache and DecodeGraphs: the line has a
    value, an end-to-end value and a prefill figure, and names the reference's attention backend and page size."""
    r = _run("--impl", "reference", "--gpus", "1", "--steps", "3", "--warmup", "3", "--layers", "2", "--skip-points")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and "unavailable" not in line, line
    assert line["value"] > 0 and line["e2e"]["value"] > 0 and line["prefill"]["value"] > 0
    assert line["config"]["layers"] == 2 and line["config"]["page_size"] == 256 and line["config"]["attention"] in ("fa2", "fa4")
