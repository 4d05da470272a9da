"""bench.py contract pieces that need no GPU: the reference arm answers with one JSON line and exit
code 0 when the reference cannot run here, and the option parser has the documented defaults."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable_or_runs():
    # the model is shrunk on this CPU box (BERT-large would take minutes per step); the arm is otherwise the same
    res = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "3"], capture_output=True, text=True, timeout=600,
                         env=dict(os.environ, BENCH_REFERENCE_SMALL="1"))
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l.startswith("{")][-1]
    out = json.loads(line)
    assert out["impl"] == "reference"
    assert "unavailable" in out or "value" in out


def test_defaults():
    sys.path.insert(0, ROOT)
    import bench
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        o = bench.parse()
    finally:
        sys.argv = argv
    assert o.gpus == 1 and o.warmup >= 3 and o.steps >= 1 and o.impl == "ours"
