"""Child process of the multi-rank serving tests (gloo ranks on CPU). Rank 0 builds the HTTP app with a
step controller and drives it in-process; the other ranks run the follower loop. Modes:

    tokens   rank 0 posts completions; the tokens must equal, exactly, what the same two-rank engine produced
             when both ranks were handed the prompts directly (the SPMD path the tensor-parallel tests pin
             against a single-rank engine)
    leaver   rank 1 leaves between two steps (no collective in flight); rank 0's next request must end with
             503 inside the control deadline and readiness must turn false
"""
import json
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from fllm_b200.comm import init_distributed, make_tp_pp_groups  # noqa: E402
from fllm_b200.config import EngineConfig, ParallelConfig, preset  # noqa: E402
from fllm_b200.parallel.tp import LibraryTP  # noqa: E402
from fllm_b200.runtime import LLMEngine, SamplingParams  # noqa: E402
from fllm_b200.runtime.step_control import ControlChannel, StepController  # noqa: E402


def main():
    mode = sys.argv[1]
    rank, world, _ = init_distributed("gloo", timeout_s=60)
    cfg = preset("qwen3-tiny")
    cfg.vocab_size = 512
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=48, max_model_len=256, num_kv_blocks=96, use_cuda_graphs=False)
    grp, _, _, tp_rank = make_tp_pp_groups(world, 1)
    eng = LLMEngine(cfg, ec, ParallelConfig(tp=world), device="cpu", tp_group=LibraryTP(grp), tp_rank=tp_rank, seed=3,
                    eos_token_id=None)
    prompts = [[5, 6, 7, 8, 9, 10, 11], list(range(20, 60)), [3, 1, 4, 1, 5, 9, 2, 6]]
    want = eng.generate(prompts, SamplingParams(max_tokens=6)) if mode == "tokens" else None   # every rank takes part
    from fllm_b200.server.app import make_guided_builder
    from fllm_b200.tokenizer import ByteTokenizer
    ctl = StepController(eng, ControlChannel(timeout_s=float(os.environ.get("CONTROL_TIMEOUT", "8"))),
                         guided_builder=make_guided_builder(eng, ByteTokenizer(512), None))
    out = {"rank": rank, "mode": mode}
    if rank != 0:
        if mode == "leaver":
            # follow until the first request has been served, then leave while the group is idle
            while True:
                msg = ctl.ch.bcast()
                ctl.apply(msg)
                if msg["step"]:
                    eng.scheduler.now_override = msg["now"]
                    eng.step()
                if not msg["step"] and ctl.steps_seen > 0 and not eng.has_unfinished():
                    print(json.dumps(dict(out, left=True)), flush=True)
                    os._exit(0)
                ctl.steps_seen += int(msg["step"])
        out["ended"] = ctl.follow()
        out["steps"] = ctl.steps
        print(json.dumps(out), flush=True)
        os._exit(0)
    from fastapi.testclient import TestClient
    from fllm_b200.server.app import create_app
    from fllm_b200.tokenizer import ByteTokenizer
    app = create_app(eng, ByteTokenizer(512), "tiny", controller=ctl)
    with TestClient(app) as c:
        if mode == "tokens":
            got = []
            for p in prompts:
                r = c.post("/v1/completions", json={"prompt": p, "max_tokens": 6, "temperature": 0})
                assert r.status_code == 200, r.text
                got.append(r.json()["choices"][0]["token_ids"])
            out.update(agree=sum(int(a == b) for x, y in zip(got, want) for a, b in zip(x, y)), total=sum(len(w) for w in want),
                       ready=c.get("/ready").status_code)
            # a sampled request goes through the full sampler on every rank (seeded, so identical everywhere)
            r = c.post("/v1/completions", json={"prompt": prompts[0], "max_tokens": 4, "temperature": 0.8, "seed": 7})
            out["sampled_status"] = r.status_code
            # a constrained request: every rank rebuilds the recogniser from the request's fields, so the masks agree
            r = c.post("/v1/completions", json={"prompt": "x", "max_tokens": 12, "temperature": 0, "guided_regex": "[ab]{3}c"})
            out["guided_status"] = r.status_code
            out["guided_text"] = r.json()["choices"][0]["text"] if r.status_code == 200 else r.text
            r = c.post("/v1/completions", json={"prompt": "x", "max_tokens": 4, "guided_regex": "(unclosed"})
            out["bad_grammar_status"] = r.status_code
            r = c.post("/v1/completions", json={"prompt": prompts[2], "max_tokens": 3, "temperature": 0})
            out["after_refusal_status"] = r.status_code
        else:
            r = c.post("/v1/completions", json={"prompt": prompts[0], "max_tokens": 3, "temperature": 0})
            out["first_status"] = r.status_code
            time.sleep(3.5)                        # rank 1 leaves at the next keep-alive; the one after it fails
            t0 = time.monotonic()
            r = c.post("/v1/completions", json={"prompt": prompts[1], "max_tokens": 3, "temperature": 0})
            out.update(second_status=r.status_code, seconds=time.monotonic() - t0, ready=c.get("/ready").status_code,
                       health=c.get("/health").status_code)
    print(json.dumps(out), flush=True)
    os._exit(0)


if __name__ == "__main__":
    main()
