"""Child process of the communicator tests (gloo ranks on CPU): exact-integer collectives, and failure
cases made on the host (a rank that leaves before a collective, a rank that never joins it)."""
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fllm_b200.comm import CommError, Group, init_distributed  # noqa: E402


def exact(g: Group):
    r, n = g.rank, g.size
    x = torch.arange(6, dtype=torch.float32) + 10 * r
    assert torch.equal(g.all_reduce(x.clone()), torch.arange(6, dtype=torch.float32) * n + 10 * sum(range(n)))
    ag = g.all_gather(torch.tensor([r, r * r], dtype=torch.int64))
    assert ag.tolist() == [[i, i * i] for i in range(n)]
    rs = g.reduce_scatter(torch.ones(2 * n, 3) * (r + 1))
    assert rs.shape == (2, 3) and torch.equal(rs, torch.full((2, 3), float(sum(range(1, n + 1)))))
    b = torch.tensor([7.0, 8.0]) if r == 1 else torch.zeros(2)
    assert g.broadcast(b, src=1).tolist() == [7.0, 8.0]
    # variable-size all-to-all: rank r sends (d + 1) rows holding r * 100 + d to rank d
    recv = g.all_to_all([torch.full((d + 1, 2), float(r * 100 + d)) for d in range(n)])
    assert [t.shape[0] for t in recv] == [r + 1] * n and [float(t[0, 0]) for t in recv] == [s * 100.0 + r for s in range(n)]
    if r == 0:
        g.send(torch.tensor([41.0, 42.0]), dst=n - 1)
    if r == n - 1:
        assert g.recv(torch.zeros(2), src=0).tolist() == [41.0, 42.0]
    sub = g.split(color=r % 2, key=-r)                      # odd / even ranks, reversed order
    assert sub.ranks == sorted([i for i in range(n) if i % 2 == r % 2], reverse=True)
    assert float(sub.all_reduce(torch.tensor([float(r)]))[0]) == float(sum(sub.ranks))
    g.barrier()
    return {"ok": True}


def main():
    mode = sys.argv[1]
    rank, world, _ = init_distributed("gloo", timeout_s=float(os.environ.get("COMM_TIMEOUT", "8")))
    g = Group()
    out = {"rank": rank, "mode": mode}
    if mode == "exact":
        out.update(exact(g))
    elif mode in ("leaver", "absent"):
        # rank 1 fails on the host before the collective (raises and exits, or just never calls it);
        # every other rank must get a "[comm]" error within the group's deadline, never hang
        g.barrier()
        if rank == 1:
            if mode == "leaver":
                print(json.dumps(dict(out, left=True)), flush=True)
                os._exit(3)
            time.sleep(float(os.environ.get("COMM_TIMEOUT", "8")) + 4)
            print(json.dumps(dict(out, slept=True)), flush=True)
            os._exit(0)
        t0 = time.monotonic()
        try:
            g.all_reduce(torch.ones(4))
            out["error"] = None
        except CommError as e:
            out["error"] = str(e)[:200]
        out["seconds"] = time.monotonic() - t0
    print(json.dumps(out), flush=True)
    os._exit(0)              # a broken group cannot be torn down cleanly: leave without the destructor


if __name__ == "__main__":
    main()
