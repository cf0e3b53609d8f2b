"""What `bench.py` has to answer without a GPU: more than one GPU is refused with one line and exit
code 2, and the reference arm says in one JSON line why it cannot run."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench(*args, env=None):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          timeout=120, env=env)


def test_more_than_one_gpu_is_refused_in_one_line():
    p = _bench("--gpus", "2", "--steps", "3", "--warmup", "3")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "one GPU" in lines[0]
    # launched as a rank of several, it says the same
    env = dict(os.environ, WORLD_SIZE="2", RANK="0", LOCAL_RANK="0")
    p = _bench("--gpus", "1", env=env)
    assert p.returncode == 2


def test_the_reference_arm_says_why_it_is_unavailable():
    p = _bench("--impl", "reference", "--gpus", "1", "--steps", "3", "--warmup", "3")
    assert p.returncode == 0
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and "\n" not in d["unavailable"]
