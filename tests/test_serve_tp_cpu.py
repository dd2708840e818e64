"""One HTTP front end driving a two-rank tensor-parallel model instance (gloo ranks on CPU): the step-control
messages keep the ranks' schedulers in lock-step, and a rank that leaves between steps turns the server
not-ready with 503 answers instead of hanging it."""
import json
import os
import socket
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _run(world, mode, timeout=180, env_extra=None):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1",
                   MASTER_PORT=str(port), OMP_NUM_THREADS="1", CONTROL_TIMEOUT="6")
        env.update(env_extra or {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "serve_worker.py"), mode], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    try:
        for p in procs:
            o, e = p.communicate(timeout=timeout)
            outs.append((p.returncode, o, e))
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    res = []
    for rc, o, e in outs:
        lines = [l for l in o.splitlines() if l.startswith("{")]
        assert lines, (rc, e[-2000:])
        res.append(json.loads(lines[-1]))
    return res


def test_http_request_to_rank0_is_served_by_both_ranks():
    r0, r1 = _run(2, "tokens")
    assert r0["total"] == 18 and r0["agree"] == r0["total"], r0
    assert r0["ready"] == 200 and r0["sampled_status"] == 200
    import re
    assert r0["guided_status"] == 200 and re.fullmatch("[ab]{3}c", r0["guided_text"]), r0
    assert r0["bad_grammar_status"] == 400 and r0["after_refusal_status"] == 200
    assert r1["ended"] == "stop" and r1["steps"] > 0


def test_follower_leaving_between_steps_gives_503_not_a_hang():
    r0, r1 = _run(2, "leaver")
    assert r1.get("left") is True
    assert r0["first_status"] == 200
    assert r0["second_status"] == 503, r0
    assert r0["seconds"] < 20, r0
    assert r0["ready"] == 503 and r0["health"] == 200
