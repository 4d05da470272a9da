"""Rank-failure detection among gloo ranks on CPU: a worker that exits between steps makes the
survivors raise RankFailureError (naming it) within the heartbeat timeout instead of hanging in the
next collective; with no failure everybody finishes.  Resume-after-restart with identical losses is
covered by tests/test_checkpoint_cpu.py."""
import json
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SCRIPT = os.path.join(HERE, "dist_scripts", "failure_worker.py")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(tmp_path, world, extra):
    out = str(tmp_path / "res")
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   LOCAL_RANK=str(r), OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, SCRIPT, "--out", out] + extra, env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    codes = []
    for p in procs:
        try:
            p.communicate(timeout=120)
        except subprocess.TimeoutExpired:
            p.kill()
            raise AssertionError("a worker hung instead of reporting the failure")
        codes.append(p.returncode)
    res = {}
    for r in range(world):
        f = "%s.%d" % (out, r)
        if os.path.exists(f):
            res[r] = json.load(open(f))
    return codes, res


def test_all_ranks_alive(tmp_path):
    codes, res = _launch(tmp_path, 3, ["--steps", "4"])
    assert codes == [0, 0, 0]
    assert all(res[r]["completed"] == 4 and res[r]["error"] is None for r in range(3))


def test_worker_exit_is_detected_by_survivors(tmp_path):
    codes, res = _launch(tmp_path, 3, ["--steps", "6", "--die_rank", "2", "--die_after", "2"])
    assert codes[2] == 17 and codes[0] == 0 and codes[1] == 0
    for r in (0, 1):
        assert res[r]["completed"] == 2
        assert res[r]["error"]["type"] == "RankFailureError" and res[r]["error"]["ranks"] == [2]
        assert res[r]["error"]["after_s"] < 30
    assert 2 not in res
