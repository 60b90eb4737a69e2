"""The forms of bench.py that need no GPU: more than one GPU is refused with one line and
status 2, the reference arm says why it cannot run, and the option list names what the
measurement contract asks for."""
import json
import subprocess
import sys
from pathlib import Path

BENCH = str(Path(__file__).resolve().parents[1] / "bench.py")


def run(*args):
    return subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, timeout=120)


def test_more_than_one_gpu_is_refused_in_one_line():
    done = run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert done.returncode == 2
    lines = [line for line in done.stdout.splitlines() if line.strip()]
    assert len(lines) == 1 and "--gpus 2" in lines[0]


def test_the_reference_arm_says_why_it_is_unavailable():
    done = run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert done.returncode == 0
    record = json.loads(done.stdout.strip().splitlines()[-1])
    assert record["impl"] == "reference" and len(record["unavailable"]) > 20
    assert "\n" not in record["unavailable"]


def test_help_names_the_contract_options():
    done = run("--help")
    assert done.returncode == 0
    for option in ("--gpus", "--steps", "--warmup", "--impl", "--workload", "--layers", "--batch", "--context"):
        assert option in done.stdout
