"""Host-side logit processors (typical-p, DRY, Mirostat 2, banned sequences) and their path through
the engine's sampler."""
import math

import pytest
import torch

from fllm_b200.config import EngineConfig, preset
from fllm_b200.runtime import LLMEngine, SamplingParams
from fllm_b200.runtime.logits_processors import Mirostat, banned_by_sequences, dry_penalties, typical_keep_mask


def test_typical_mask_keeps_the_tokens_nearest_the_entropy():
    # p = [0.5, 0.25, 0.125, 0.0625, 0.0625]: entropy 1.875 bits; surprises 1, 2, 3, 4, 4 bits
    p = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.0625])
    logits = p.log()
    # deviations from 1.875: 0.875, 0.125, 1.125, 2.125, 2.125 -> order 1, 0, 2, ...
    assert typical_keep_mask(logits, 0.2, 1.0).tolist() == [False, True, False, False, False]
    assert typical_keep_mask(logits, 0.7, 1.0).tolist() == [True, True, False, False, False]
    assert typical_keep_mask(logits, 0.8, 1.0).tolist() == [True, True, True, False, False]
    assert typical_keep_mask(logits, 1.0, 1.0).all()
    # -inf entries (already banned tokens) never come back
    banned = logits.clone()
    banned[1] = float("-inf")
    assert not typical_keep_mask(banned, 0.9, 1.0)[1]


def test_dry_penalises_the_continuation_of_a_repeated_sequence():
    #       0  1  2  3  4  5  6  7
    ctx = [10, 11, 12, 13, 99, 10, 11, 12]          # "10 11 12" came before and was followed by 13
    pen = dry_penalties(ctx, multiplier=0.8, base=2.0, allowed_length=2)
    assert pen == {13: pytest.approx(0.8 * 2.0 ** (3 - 2))}
    assert dry_penalties(ctx, 0.8, 2.0, allowed_length=4) == {}                 # the match (3) is shorter than allowed
    assert dry_penalties(ctx, 0.8, 2.0, 2, breakers=[11]) == {}                 # a breaker inside the match cuts it to 1
    assert dry_penalties(ctx, 0.0) == {} and dry_penalties([], 1.0) == {}
    # two earlier copies: the longer match wins
    ctx2 = [1, 2, 3, 7, 9, 2, 3, 8, 1, 2, 3]
    pen2 = dry_penalties(ctx2, 1.0, 2.0, 2)
    assert pen2[7] == pytest.approx(2.0) and pen2[8] == pytest.approx(1.0)      # "1 2 3"->7 (n=3), "2 3"->8 (n=2)
    assert dry_penalties(ctx2, 1.0, 2.0, 2, last_n=4) == {}                     # window too short to see a copy


def test_banned_sequences_ban_the_last_token_after_the_prefix():
    assert banned_by_sequences([5, 6, 7], [[7, 8], [6, 7, 9], [4], [1, 2]]) == [8, 9, 4]
    assert banned_by_sequences([], [[7, 8], [3]]) == [3]


def test_mirostat_moves_mu_towards_the_target_surprise():
    torch.manual_seed(0)
    m = Mirostat(tau=3.0, eta=0.2)
    assert m.mu == 6.0
    logits = torch.randn(500) * 3
    keep = m.keep_mask(logits, 1.0)
    logp2 = torch.log_softmax(logits, -1) / math.log(2)
    assert torch.equal(keep, -logp2 <= 6.0) and keep.any()
    top = int(torch.argmax(logits))
    s = -float(m._logp2[top])                       # surprise of the most likely token within the kept set
    m.observe(top)
    assert m.mu == pytest.approx(6.0 - 0.2 * (s - 3.0))
    # a run of low-surprise picks raises mu until high-surprise tokens are allowed again; mu stays finite
    for _ in range(50):
        m.keep_mask(logits, 1.0)
        m.observe(top)
    assert m.mu > 6.0 and math.isfinite(m.mu)
    tiny = Mirostat(tau=0.1, eta=0.1)
    tiny.mu = 1e-6
    assert int(tiny.keep_mask(logits, 1.0).sum()) == 1          # never an empty set


def _engine():
    cfg = preset("qwen3-tiny")
    ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=48)
    return cfg, LLMEngine(cfg, ec, device="cpu", seed=3)


def test_engine_applies_banned_sequences_dry_typical_and_mirostat():
    cfg, eng = _engine()
    prompt = [[5, 9, 2, 7, 7, 1]]
    base = eng.generate(prompt, SamplingParams(max_tokens=8))[0]
    # ban the greedy continuation after its predecessor: the sequence must deviate exactly there
    seq = [base[2], base[3]]
    first = next(i for i in range(1, len(base)) if base[i - 1] == seq[0])       # first place the prefix matches
    got = eng.generate(prompt, SamplingParams(max_tokens=8, bad_words=[seq]))[0]
    assert got[:first] == base[:first] and got[first] != seq[1]
    for i in range(1, len(got)):
        assert not (got[i - 1] == seq[0] and got[i] == seq[1])
    # a one-token ban never appears
    got1 = eng.generate(prompt, SamplingParams(max_tokens=8, bad_words=[[base[0]]]))[0]
    assert base[0] not in got1
    # DRY on a prompt that repeats: the token that would continue the repeat loses a huge penalty
    rep = [[3, 4, 5, 6, 3, 4, 5]]
    plain = eng.generate(rep, SamplingParams(max_tokens=1))[0]
    eng.add_request(rep[0], SamplingParams(max_tokens=1))
    step = eng.scheduler.schedule()
    logits = eng.decoder.forward(eng._build_batch(step))[-1].float()
    eng._commit(step, [int(logits.argmax())])
    forced = eng.generate(rep, SamplingParams(max_tokens=1, logit_bias={6: 50.0}))[0]
    assert forced == [6]
    dry = eng.generate(rep, SamplingParams(max_tokens=1, logit_bias={6: 50.0}, dry_multiplier=100.0, dry_base=2.0))[0]
    assert dry != [6] and plain is not None
    # typical_p -> 0 keeps one token: sampling at temperature 1 becomes deterministic, whatever the seed
    a = eng.generate(prompt, SamplingParams(max_tokens=6, temperature=1.0, typical_p=1e-6, seed=1))[0]
    b = eng.generate(prompt, SamplingParams(max_tokens=6, temperature=1.0, typical_p=1e-6, seed=2))[0]
    assert a == b
    # Mirostat: seeded runs repeat, the controller state lives on the request and speculation is off
    sp = SamplingParams(max_tokens=10, temperature=1.0, mirostat_mode=2, mirostat_tau=2.0, seed=11)
    sp.validate(cfg.vocab_size)
    assert sp.speculative is False
    m1 = eng.generate(prompt, SamplingParams(max_tokens=10, temperature=1.0, mirostat_mode=2, mirostat_tau=2.0, seed=11))[0]
    m2 = eng.generate(prompt, SamplingParams(max_tokens=10, temperature=1.0, mirostat_mode=2, mirostat_tau=2.0, seed=11))[0]
    assert m1 == m2 and len(m1) == 10
    with pytest.raises(ValueError):
        SamplingParams(typical_p=0.0).validate(cfg.vocab_size)
    with pytest.raises(ValueError):
        SamplingParams(mirostat_mode=3).validate(cfg.vocab_size)


def test_http_fields_reach_the_sampling_parameters():
    from fllm_b200.server.app import _sampling_from
    sp = _sampling_from({"typical_p": 0.9, "dry_multiplier": 0.8, "dry_base": 1.5, "dry_allowed_length": 3,
                         "dry_sequence_breakers": [13, "\n"], "mirostat": 2, "mirostat_tau": 4.0, "mirostat_eta": 0.2,
                         "bad_words_ids": [[4, 5], [6]]})
    assert (sp.typical_p, sp.dry_multiplier, sp.dry_base, sp.dry_allowed_length) == (0.9, 0.8, 1.5, 3)
    assert sp.dry_sequence_breakers == (13,) and (sp.mirostat_mode, sp.mirostat_tau, sp.mirostat_eta) == (2, 4.0, 0.2)
    assert sp.bad_words == [[4, 5], [6]] and sp.needs_full_sampler and sp.needs_host_processors
    o = _sampling_from({"options": {"typical_p": 0.5, "mirostat": 1}}, dialect="ollama")
    assert o.typical_p == 0.5 and o.mirostat_mode == 1
    from fllm_b200.server.cache import request_key
    k1 = request_key("m", [1, 2], _sampling_from({"temperature": 0, "typical_p": 0.9}))
    k2 = request_key("m", [1, 2], _sampling_from({"temperature": 0, "typical_p": 0.8}))
    assert k1 != k2


def test_mirostat_v1_cuts_by_the_zipf_estimate():
    # an exact Zipf distribution p_i ~ i^-s: the estimator recovers s, and k follows the closed form
    n, s = 5000, 1.3
    logits = -s * torch.log(torch.arange(1, n + 1, dtype=torch.float64))
    m = Mirostat(tau=3.0, eta=0.1, version=1)
    keep = m.keep_mask(logits.float(), 1.0)
    eps = s - 1.0
    k_expect = ((eps * 2.0 ** m.mu) / (1.0 - n ** (-eps))) ** (1.0 / s)
    assert abs(int(keep.sum()) - k_expect) <= max(2.0, 0.02 * k_expect)
    assert bool(keep[: int(keep.sum())].all())                       # the k most probable tokens
    mu0 = m.mu
    m.observe(0)                                                     # surprise of the top token is below tau
    assert m.mu > mu0
    # a smaller mu keeps fewer tokens
    m2 = Mirostat(tau=1.0, eta=0.1, version=1)
    assert int(m2.keep_mask(logits.float(), 1.0).sum()) < int(keep.sum())
    # through the engine: mode 1 is seeded-repeatable
    from fllm_b200.runtime.request import SamplingParams
    sp = SamplingParams(max_tokens=4, temperature=1.0, mirostat_mode=1, mirostat_tau=2.0, seed=3)
    assert sp.needs_host_logits() if hasattr(sp, "needs_host_logits") else True
