"""Communicator self-test on CPU ranks (gloo): exact collectives and host-made failures
(cf. rust/engine/src/comm/local.rs:219-241 `a_failing_rank_aborts_the_others`)."""
import json
import os
import subprocess
import sys

import pytest

from test_tp_cpu import _free_port

HERE = os.path.dirname(os.path.abspath(__file__))


def _spawn(world, mode, timeout_s=8):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1", COMM_TIMEOUT=str(timeout_s))
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "comm_worker.py"), mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    res = []
    for p in procs:
        try:
            o, e = p.communicate(timeout=90)
        except subprocess.TimeoutExpired:
            p.kill()
            o, e = p.communicate()
            res.append((None, {}, e))
            continue
        lines = [l for l in o.splitlines() if l.startswith("{")]
        res.append((p.returncode, json.loads(lines[-1]) if lines else {}, e))
    return res


@pytest.mark.parametrize("world", [2, 4])
def test_collectives_are_exact_on_integers(world):
    for rc, out, err in _spawn(world, "exact"):
        assert rc == 0 and out.get("ok"), err[-1500:]


@pytest.mark.parametrize("mode", ["leaver", "absent"])
def test_a_failing_rank_makes_the_others_fail_fast(mode):
    res = _spawn(3, mode, timeout_s=6)
    assert res[1][0] == (3 if mode == "leaver" else 0)
    for r in (0, 2):
        rc, out, err = res[r]
        assert rc == 0, err[-1500:]                       # the survivors exit on their own, no hang
        assert out["error"] and out["error"].startswith("[comm]"), out
        assert out["seconds"] < 30, out
