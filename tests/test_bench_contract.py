"""What bench.py answers without a GPU: more than one GPU is refused with one line and exit
code 2, and the reference arm answers with one JSON line and exit code 0 (its numbers where
a GPU and the reference's copy are present, else the reason)."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run(*args):
    return subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_with_one_line():
    r = run("--gpus", "2", "--steps", "4", "--warmup", "3")
    assert r.returncode == 2
    lines = [l for l in r.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]


def test_reference_arm_prints_one_json_line():
    r = run("--impl", "reference", "--gpus", "1", "--steps", "4", "--warmup", "3")
    assert r.returncode == 0, r.stderr[-2000:]
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference"
    assert ("unavailable" in line and line["unavailable"]) or line["value"] > 0
