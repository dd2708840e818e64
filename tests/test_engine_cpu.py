"""Engine logic on CPU (reference ops): paged KV, chunked prefill, continuous batching and
prefix caching must reproduce an independent dense decoder token for token."""
import torch

from fllm_b200.config import EngineConfig, preset
from fllm_b200.models.weights import init_random_weights
from fllm_b200.runtime import LLMEngine, SamplingParams

from oracle import dense_forward, greedy_generate


def _prompts(vocab, lens, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def _engine(cfg, **kw):
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=32, max_model_len=256, num_kv_blocks=96, **kw)
    return LLMEngine(cfg, ec, device="cpu")


def test_generate_matches_dense_oracle():
    cfg = preset("qwen3-tiny")
    eng = _engine(cfg)
    prompts = _prompts(cfg.vocab_size, (3, 17, 50, 33))
    outs = eng.generate(prompts, SamplingParams(max_tokens=6))
    for p, o in zip(prompts, outs):
        ref = greedy_generate(cfg, eng.weights, p, 6)
        assert o == ref


def test_chunked_prefill_equals_single_pass():
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu")
    p = _prompts(cfg.vocab_size, (90,))
    small = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=16, max_model_len=256, num_kv_blocks=64), device="cpu", weights=w)
    big = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=256, max_model_len=256, num_kv_blocks=64), device="cpu", weights=w)
    assert small.generate(p, SamplingParams(max_tokens=5)) == big.generate(p, SamplingParams(max_tokens=5))
    assert small.stats.steps > big.stats.steps


def test_prefix_cache_hit_keeps_output():
    cfg = preset("qwen3-tiny")
    eng = _engine(cfg)
    p = _prompts(cfg.vocab_size, (70,))
    a = eng.generate(p, SamplingParams(max_tokens=4))
    b = eng.generate(p, SamplingParams(max_tokens=4))
    assert a == b
    assert eng.blocks.stats["prefix_hits"] >= 1


def test_preemption_by_recompute_keeps_output():
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu")
    prompts = _prompts(cfg.vocab_size, (40, 44, 48, 52))
    roomy = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=64,
                                        enable_prefix_caching=False), device="cpu", weights=w)
    tight = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=13,
                                        enable_prefix_caching=False, watermark=0.0), device="cpu", weights=w)
    sp = SamplingParams(max_tokens=12)
    assert tight.generate(prompts, sp) == roomy.generate(prompts, sp)
    assert tight.scheduler.stats["preemptions"] > 0


def test_llama_and_window_models_match_oracle():
    for name in ("tiny-llama",):
        cfg = preset(name)
        cfg.vocab_size = 512
        eng = _engine(cfg)
        prompts = _prompts(cfg.vocab_size, (9, 30))
        outs = eng.generate(prompts, SamplingParams(max_tokens=5))
        for p, o in zip(prompts, outs):
            assert o == greedy_generate(cfg, eng.weights, p, 5)
    cfg = preset("qwen3-tiny")
    cfg.sliding_window = 24
    eng = _engine(cfg)
    prompts = _prompts(cfg.vocab_size, (60,))
    outs = eng.generate(prompts, SamplingParams(max_tokens=5))
    assert outs[0] == greedy_generate(cfg, eng.weights, prompts[0], 5)


def test_stop_and_max_tokens():
    cfg = preset("qwen3-tiny")
    eng = _engine(cfg)
    p = _prompts(cfg.vocab_size, (10,))
    full = eng.generate(p, SamplingParams(max_tokens=8))[0]
    stop_tok = full[3]
    cut = eng.generate(p, SamplingParams(max_tokens=8, stop_token_ids=(stop_tok,)))[0]
    assert cut == full[: full.index(stop_tok) + 1]


def test_gpt_oss_moe_model_matches_oracle():
    """Sinks, alternating sliding window, biased experts, clamped SwiGLU, top-4 softmax router."""
    cfg = preset("gpt-oss-tiny")
    eng = _engine(cfg)
    prompts = _prompts(cfg.vocab_size, (9, 150))
    outs = eng.generate(prompts, SamplingParams(max_tokens=4))
    for p, o in zip(prompts, outs):
        assert o == greedy_generate(cfg, eng.weights, p, 4)


def test_speculative_ngram_and_draft_model_keep_greedy_output():
    """Speculation must not change greedy text; a draft equal to the target accepts everything."""
    from fllm_b200.runtime.speculative import AdaptiveDraft, NgramProposer
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu")
    prompts = _prompts(cfg.vocab_size, (12, 40))
    prompts[0] = prompts[0][:6] * 4                      # repetition gives the n-gram lookup something to find
    sp = SamplingParams(max_tokens=14)
    base = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=96), device="cpu", weights=w)
    want = base.generate(prompts, sp)
    ng = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=96, speculative="ngram"),
                   device="cpu", weights=w)
    assert ng.generate(prompts, sp) == want
    dm = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=96), device="cpu", weights=w)
    dm.enable_draft_model(cfg, weights=w, k=3)           # draft == target: every draft is accepted
    assert dm.generate(prompts, sp) == want
    assert dm.stats.spec_proposed > 0 and dm.stats.spec_accepted == dm.stats.spec_proposed
    assert dm.stats.steps < base.stats.steps
    other = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=96), device="cpu", weights=w)
    other.enable_draft_model(cfg, k=4, seed=99)          # unrelated draft: mostly rejected, text unchanged
    assert other.generate(prompts, sp) == want
    assert NgramProposer(3).propose([1, 2, 3, 9, 1, 2, 3]) == [9, 1, 2]
    a = AdaptiveDraft(6)
    for _ in range(20):
        a.update(4, 0)
    assert a.length() == 1
    for _ in range(40):
        a.update(4, 4)
    assert a.length() == 6


def test_fp8_kv_cache_stays_close_to_bf16_kv():
    """An e4m3 KV pool (half the bytes) must reproduce the bf16-KV logits within fp8 precision."""
    import torch
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("qwen3-tiny")
    outs = []
    for kvd in ("bf16", "fp8_e4m3"):
        ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=32, kv_cache_dtype=kvd)
        eng = LLMEngine(cfg, ec, device="cpu", seed=1)
        assert eng.kv.store.element_size() == (2 if kvd == "bf16" else 1)
        g = torch.Generator().manual_seed(0)
        p = torch.randint(0, cfg.vocab_size, (70,), generator=g).tolist()
        eng.add_request(p, SamplingParams(max_tokens=1))
        rows = []
        while eng.has_unfinished():
            step = eng.scheduler.schedule()
            batch = eng._build_batch(step)
            logits = eng.decoder.forward(batch)
            if logits.shape[0]:
                rows.append(logits[-1].float())
            eng._commit(step, eng.decoder.greedy_tokens(logits).tolist())
        outs.append(rows[-1])
    err = (outs[0] - outs[1]).abs().max().item() / (outs[0].abs().max().item() + 1e-6)
    assert 0 < err < 0.08, err


def test_disaggregated_prefill_then_decode_matches_one_engine():
    """Prompt processed on engine A, KV handed to engine B, decoding continued there: same tokens as one
    engine doing both; B's pool, prefix cache and limits stay consistent; layout mismatches are refused."""
    import pytest
    import torch
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("qwen3-tiny")
    ec = lambda **kw: EngineConfig(max_num_seqs=4, max_num_batched_tokens=32, max_model_len=160, num_kv_blocks=40, **kw)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (50, 9)]
    sp = SamplingParams(max_tokens=12)
    ref = LLMEngine(cfg, ec(), device="cpu", seed=2)
    want = [ref.generate([p], sp)[0] for p in prompts]        # one at a time, like the hand-over below
    a, b = LLMEngine(cfg, ec(), device="cpu", seed=2), LLMEngine(cfg, ec(), device="cpu", seed=2)
    got = []
    for p in prompts:
        blob, others = a.prefill_only(p, SamplingParams(max_tokens=12))
        assert others == [] and len(blob["output"]) == 1 and blob["num_computed"] == len(p)
        assert not a.requests and a.blocks.num_used() <= a.blocks.blocks_needed(len(p))     # only cached blocks remain
        rid = b.import_request(blob)
        toks = list(blob["output"])
        while b.has_unfinished():
            for ev in b.step():
                if ev.request_id == rid:
                    toks.extend(ev.token_ids)
        got.append(toks)
    assert got == want
    c = LLMEngine(cfg, ec(kv_cache_dtype="fp8_e4m3"), device="cpu", seed=2)
    blob, _ = a.prefill_only(prompts[1], SamplingParams(max_tokens=4))
    with pytest.raises(ValueError):
        c.import_request(blob)


def test_preemption_by_swap_parks_kv_on_the_host_and_keeps_output():
    """With a pool too small for all sequences, decode sequences that get preempted have their KV copied
    to host memory and back instead of being recomputed; output must equal the roomy run, the host tier
    must have been used and must be empty at the end; a zero-byte tier falls back to recompute."""
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu")
    prompts = _prompts(cfg.vocab_size, (40, 44, 48, 52))
    mk = lambda blocks, **kw: LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=blocks,
                                                          enable_prefix_caching=False, watermark=0.0, **kw),
                                        device="cpu", weights=w)
    sp = SamplingParams(max_tokens=12)
    want = mk(64).generate(prompts, sp)
    tight = mk(13, preemption="swap", swap_space_gb=0.25)
    assert tight.generate(prompts, sp) == want
    sw = tight.scheduler.swapper
    assert sw.stats["swapped_out"] > 0 and sw.stats["swapped_in"] == sw.stats["swapped_out"]
    assert not sw.parked and sw.bytes == 0
    none = mk(13, preemption="swap", swap_space_gb=0.0)
    assert none.generate(prompts, sp) == want
    assert none.scheduler.swapper.stats["swapped_out"] == 0 and none.scheduler.stats["preemptions"] > 0


def test_beam_search_matches_a_brute_force_search_on_the_oracle():
    """Width 1 is greedy decoding; width 3 returns sorted hypotheses whose scores are the oracle's summed
    log-probabilities, and its best hypothesis scores like the best one of an independent beam search over
    the dense oracle; an end-of-sequence token closes a hypothesis."""
    cfg = preset("qwen3-tiny")
    eng = _engine(cfg)
    prompt = _prompts(cfg.vocab_size, (9,), seed=4)[0]
    n = 5
    greedy = greedy_generate(cfg, eng.weights, prompt, n)
    one = eng.beam_search(prompt, beam_width=1, max_tokens=n, length_penalty=0.0)
    assert one[0][0] == greedy

    def logp(tokens):
        return torch.log_softmax(dense_forward(cfg, eng.weights, tokens)[-1].float(), -1)

    def seq_score(toks):
        return sum(float(logp(prompt + toks[:i])[toks[i]]) for i in range(len(toks)))
    W = 3
    got = eng.beam_search(prompt, beam_width=W, max_tokens=n, length_penalty=0.0)
    assert len(got) == W and all(len(t) == n for t, _ in got)
    assert [s for _, s in got] == sorted((s for _, s in got), reverse=True)
    for toks, score in got:
        assert abs(score - seq_score(toks)) < 0.05 * n
    beams = [([], 0.0)]
    for _ in range(n):                                   # independent reference search
        cands = []
        for toks, lp in beams:
            top = logp(prompt + toks).topk(2 * W)
            cands += [(toks + [int(t)], lp + float(l)) for l, t in zip(top.values, top.indices)]
        beams = sorted(cands, key=lambda c: -c[1])[:W]
    assert abs(got[0][1] - beams[0][1]) < 0.05 * n
    assert got[0][0] == beams[0][0] or abs(seq_score(got[0][0]) - beams[0][1]) < 0.05
    # with a length penalty the score is the mean log-probability; an EOS ends a hypothesis early
    eos = got[0][0][1]
    ended = eng.beam_search(prompt, beam_width=W, max_tokens=n, length_penalty=1.0, eos_token_id=eos)
    assert any(t[-1] == eos and len(t) < n for t, _ in ended) or all(eos not in t[:-1] for t, _ in ended)
    for t, s in ended:
        assert eos not in t[:-1]
        assert abs(s - seq_score(t) / len(t)) < 0.05
    assert eng.blocks.num_used() <= eng.blocks.blocks_needed(len(prompt) + n) * 4       # nothing leaks: only cached blocks stay
    assert not eng.requests


def test_evicted_prefix_blocks_come_back_from_the_host_and_disk_tiers(tmp_path):
    """A pool too small to keep every prompt cached: evicted prefix blocks go to host memory, overflow to files,
    and are restored when their prompt returns: same tokens, prompt tokens served from the cache, and a new
    engine on the same directory finds the files (re-warm after restart); a different KV layout ignores them."""
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu")
    prompts = _prompts(cfg.vocab_size, (70, 66, 75, 68), seed=9)
    sp = SamplingParams(max_tokens=3)
    kb = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=96, max_model_len=128, num_kv_blocks=8), device="cpu", weights=w)
    block_bytes = kb.kv.store[:, :, 0].numel() * kb.kv.store.element_size()
    mk = lambda **kw: LLMEngine(cfg, EngineConfig(max_num_batched_tokens=96, max_model_len=128, num_kv_blocks=8, watermark=0.0,
                                                  **kw), device="cpu", weights=w)
    plain = mk()
    want = [plain.generate([p], sp)[0] for p in prompts]
    # host tier with room for 6 blocks, the rest spills to disk
    eng = mk(kv_tier_host_gb=6.5 * block_bytes / (1 << 30), kv_tier_disk_dir=str(tmp_path), kv_tier_disk_gb=1.0)
    assert eng.kv_tier is not None and eng.kv_tier.enabled
    assert [eng.generate([p], sp)[0] for p in prompts] == want          # 4 prompts x 4 full blocks through an 8-block pool
    t = eng.kv_tier
    assert t.stats["stored"] >= 8 and t.stats["spilled"] >= 1 and len(t.host) <= 6
    before = eng.blocks.stats["tier_restored"]
    again = [eng.generate([p], sp)[0] for p in prompts]
    assert again == want
    assert eng.blocks.stats["tier_restored"] - before >= 8 and t.stats["host_hits"] + t.stats["disk_hits"] >= 8
    assert t.stats["disk_hits"] >= 1
    # restart: a fresh engine indexes the files and serves the first prompt's blocks from disk
    on_disk = len(t.disk)
    eng2 = mk(kv_tier_host_gb=0.0, kv_tier_disk_dir=str(tmp_path), kv_tier_disk_gb=1.0)
    assert eng2.kv_tier.stats["rewarmed"] == on_disk >= 1
    hit_prompt = next(p for p in prompts if eng2.blocks.tier_has(
        __import__("fllm_b200.runtime.block_manager", fromlist=["chain_hash"]).chain_hash(b"", p[:16], b"")))
    assert eng2.generate([hit_prompt], sp)[0] == want[prompts.index(hit_prompt)]
    assert eng2.blocks.stats["tier_restored"] >= 1 and eng2.kv_tier.stats["disk_hits"] >= 1
    other = LLMEngine(cfg, EngineConfig(max_num_batched_tokens=96, max_model_len=128, num_kv_blocks=8, kv_cache_dtype="fp8_e4m3",
                                        kv_tier_disk_dir=str(tmp_path), kv_tier_disk_gb=1.0), device="cpu", weights=w)
    assert other.kv_tier.stats["rewarmed"] == 0
    # a disk budget of two blocks keeps two files
    small = mk(kv_tier_host_gb=0.0, kv_tier_disk_dir=str(tmp_path / "small"), kv_tier_disk_gb=2.2 * (block_bytes + 32) / (1 << 30))
    for p in prompts:
        small.generate([p], sp)
    assert len(small.kv_tier.disk) == 2 and len([f for f in (tmp_path / "small").iterdir() if f.suffix == ".kv"]) == 2


def test_kv_tier_keeps_its_byte_budgets_and_returns_what_was_stored(tmp_path):
    from fllm_b200.runtime.kv_tier import KvTier
    nb = 256
    t = KvTier("sig", nb, host_bytes=3 * nb, disk_dir=str(tmp_path), disk_bytes=4 * (nb + 32))
    blobs = {bytes([i]) * 8: torch.full((nb,), i, dtype=torch.uint8) for i in range(12)}
    for h, b in blobs.items():
        t.put(h, b)
        assert t.host_used() <= 3 * nb and t.disk_used() <= 4 * (nb + 32)
    assert len(t.host) == 3 and len(t.disk) == 4 and t.stats["dropped"] == 12 - 7
    newest, oldest_kept = bytes([11]) * 8, bytes([5]) * 8
    assert torch.equal(t.get(newest), blobs[newest]) and torch.equal(t.get(oldest_kept), blobs[oldest_kept])
    assert t.get(bytes([0]) * 8) is None and not t.has(bytes([0]) * 8)
    t.put(newest, blobs[newest])                                 # already present: no double count
    assert t.stats["stored"] == 12
    again = KvTier("sig", nb, host_bytes=0, disk_dir=str(tmp_path), disk_bytes=4 * (nb + 32))
    assert again.stats["rewarmed"] == 4 and torch.equal(again.get(oldest_kept), blobs[oldest_kept])
    assert KvTier("other", nb, 0, str(tmp_path), 10 * nb).stats["rewarmed"] == 0
    again.clear()
    assert not [f for f in tmp_path.iterdir() if f.suffix == ".kv"]
    off = KvTier("sig", nb)
    off.put(newest, blobs[newest])
    assert not off.enabled and not off.has(newest)


def test_launch_ahead_commit_survives_two_preemptions_in_one_schedule():
    """The launch-ahead protocol (placeholder commit -> schedule -> patch) when the scheduler evicts two
    sequences of the step that is still in flight: their tokens are patched, nothing is registered for
    a sequence that lost its blocks, and the step loop keeps running."""
    from fllm_b200.runtime.request import RequestStatus
    from fllm_b200.runtime.scheduler import ScheduledSeq, ScheduledStep

    class _Done:
        def synchronize(self):
            pass

    cfg = preset("qwen3-tiny")
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=64, num_kv_blocks=4,
                                      block_size=4, enable_prefix_caching=False, watermark=0.0), device="cpu")
    for p in _prompts(cfg.vocab_size, (3, 3, 3, 3)):
        eng.add_request(p, SamplingParams(max_tokens=8))
    eng.step()                                            # prefill: every sequence now holds 3 + 1 tokens in one block
    running = list(eng.scheduler.running)
    assert len(running) == 4 and all(r.is_decode for r in running)
    step = ScheduledStep(seqs=[ScheduledSeq(r, r.num_computed, 1, True) for r in running])
    fl = {"step": step, "event": _Done(), "out": torch.tensor([11, 12, 13, 14], dtype=torch.int32), "n": 4, "slots": []}
    eng._precommit(fl)                                    # all four now need a second block; the pool has none
    nxt = eng.scheduler.schedule()
    victims = [r for r in running if r.status == RequestStatus.PREEMPTED]
    assert len(victims) >= 2, "the tight pool must evict at least two sequences inside one schedule()"
    events = eng._finalize(fl)                            # must not raise for sequences without a block table
    assert len(events) == 4
    for r, t in zip(running, (11, 12, 13, 14)):
        assert r.output[-1] == t
    assert sum(s.count for s in nxt.seqs) <= eng.cfg.max_num_batched_tokens


def test_preempted_victim_gives_back_rows_budget_and_cow_pairs():
    from fllm_b200.runtime.block_manager import BlockManager
    from fllm_b200.runtime.request import Request
    from fllm_b200.runtime.scheduler import ScheduledSeq, ScheduledStep, Scheduler
    ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=8, max_model_len=64, num_kv_blocks=4, block_size=4,
                      enable_prefix_caching=False, watermark=0.0)
    bm = BlockManager(4, 4, False, 0.0)
    sch = Scheduler(ec, bm)
    a, b = Request("a", 0, [1, 2, 3], SamplingParams()), Request("b", 1, [4, 5, 6], SamplingParams())
    dropped = []
    sch.on_drop = dropped.append
    for r in (a, b):
        bm.allocate(r.seq_id, [])
        bm.ensure_capacity(r.seq_id, 3)
        sch.running.append(r)
    step = ScheduledStep(seqs=[ScheduledSeq(b, 0, 3, True)], cow=[(0, 1)], cow_owner=[b])
    assert sch._preempt_one(step, protect=a)
    assert step.seqs == [] and step.cow == [] and step.cow_owner == []
    assert sch._take_refund() == 3 and sch._take_refund() == 0
    assert dropped == [b] and b in sch.waiting
