"""End-to-end on a GPU: the engine running the hand-written kernels (with and without CUDA
graphs) against the PyTorch oracle on the same weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _prompts(vocab, lens, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (n,), generator=g).tolist() for n in lens]


def test_native_library_is_loaded():
    from fllm_b200.ops import _lib, get_ops
    ops = get_ops("cuda:0")
    assert ops.name == "sm100a"
    assert any(p.endswith("_C.so") for p in _lib.loaded_libraries())


@pytest.mark.parametrize("name", ["qwen3-tiny", "tiny-llama"])
def test_logits_match_oracle(name):
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from oracle import dense_forward
    cfg = preset(name)
    if name == "tiny-llama":
        cfg.vocab_size = 2048
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=48, max_model_len=256, num_kv_blocks=64)
    eng = LLMEngine(cfg, ec, device="cuda:0")
    p = _prompts(cfg.vocab_size, (100,))[0]
    # chunked prefill through the engine, then compare the last-row logits
    eng.add_request(p, SamplingParams(max_tokens=1))
    logits = None
    while eng.has_unfinished():
        step = eng.scheduler.schedule()
        batch = eng._build_batch(step)
        logits = eng.decoder.forward(batch)
        toks = eng.decoder.greedy_tokens(logits).tolist()
        eng._commit(step, toks)
    want = dense_forward(cfg, eng.weights, p)[-1]
    got = logits[-1].float()
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert eng.ops.check_status() == 0


def test_head_dim_128_prefill_runs_on_the_tensor_memory_attention_kernel_and_matches_oracle():
    """head_dim 128 with chunks of 256 tokens: both chunks of the prompt (the second continues the first)
    go through the tcgen05 prefill kernel; the last-row logits must match the dense fp32 oracle."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from oracle import dense_forward
    cfg = preset("qwen3-tiny")
    cfg.head_dim = 128
    ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=256, max_model_len=640, num_kv_blocks=96)
    eng = LLMEngine(cfg, ec, device="cuda:0")
    p = _prompts(cfg.vocab_size, (500,), seed=5)[0]
    eng.add_request(p, SamplingParams(max_tokens=1))
    logits = None
    while eng.has_unfinished():
        step = eng.scheduler.schedule()
        batch = eng._build_batch(step)
        out = eng.decoder.forward(batch)
        if out.shape[0]:
            logits = out
        eng._commit(step, eng.decoder.greedy_tokens(out).tolist())
    want = dense_forward(cfg, eng.weights, p)[-1]
    got = logits[-1].float()
    err = (got - want).abs().max().item()
    assert err < 0.05 * want.abs().max().item() + 1e-3, err
    assert eng.ops.check_status() == 0


def test_graph_and_eager_decode_agree():
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cuda:0")
    prompts = _prompts(cfg.vocab_size, (5, 33, 70, 16, 90))
    outs = []
    for graphs in (False, True):
        ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=128,
                          use_cuda_graphs=graphs)
        eng = LLMEngine(cfg, ec, device="cuda:0", weights=w)
        outs.append(eng.generate(prompts, SamplingParams(max_tokens=12)))
        if graphs:
            assert eng.stats.graph_steps > 0
    # Same tokens; where the two runs part (padded graph buckets and exact-size eager steps may round a dot product
    # differently), both choices must be within a hair of the best logit of the dense fp32 oracle at that position.
    from oracle import dense_forward
    diverged = 0
    for p, a, b in zip(prompts, outs[0], outs[1]):
        if a == b:
            continue
        diverged += 1
        j = next(i for i in range(len(a)) if a[i] != b[i])
        lg = dense_forward(cfg, w, p + a[:j])[-1].float()
        span = (lg.max() - lg.min()).item()
        assert lg.max().item() - min(lg[a[j]].item(), lg[b[j]].item()) < 0.02 * span, (j, a, b)
    assert diverged <= 1


def test_sampled_generation_is_seeded():
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("qwen3-tiny")
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=128)
    eng = LLMEngine(cfg, ec, device="cuda:0")
    p = _prompts(cfg.vocab_size, (20, 21))
    sp = SamplingParams(max_tokens=10, temperature=0.9, top_p=0.95, top_k=40, seed=7)
    a = eng.generate(p, sp)
    b = eng.generate(p, sp)
    c = eng.generate(p, SamplingParams(max_tokens=10, temperature=0.9, top_p=0.95, top_k=40, seed=8))
    assert a == b and a != c


def test_gpt_oss_tiny_logits_match_oracle():
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from oracle import dense_forward
    cfg = preset("gpt-oss-tiny")
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=64)
    eng = LLMEngine(cfg, ec, device="cuda:0")
    p = _prompts(cfg.vocab_size, (150,))[0]
    eng.add_request(p, SamplingParams(max_tokens=1))
    logits = None
    while eng.has_unfinished():
        step = eng.scheduler.schedule()
        batch = eng._build_batch(step)
        logits = eng.decoder.forward(batch)
        eng._commit(step, eng.decoder.greedy_tokens(logits).tolist())
    want = dense_forward(cfg, eng.weights, p)[-1]
    err = (logits[-1].float() - want).abs().max().item()
    assert err < 0.06 * want.abs().max().item() + 1e-3, err
    assert eng.ops.check_status() == 0


def test_gguf_q4_k_stays_packed_on_the_gpu(tmp_path):
    """A Q4_K GGUF file loaded with its 4-bit projections packed (INT4 group-affine GEMM) gives the same
    logits as the same file expanded to bf16 at load time."""
    from fllm_b200.config import EngineConfig
    from fllm_b200.cpu_engine import write_tiny_llama_gguf
    from fllm_b200.formats.loader import load_gguf
    from fllm_b200.ops.int4 import Int4Weight
    from fllm_b200.runtime import LLMEngine, SamplingParams
    path = str(tmp_path / "tiny.gguf")
    write_tiny_llama_gguf(path, seed=3)
    outs = []
    for packed in (True, False):
        cfg, w, _ = load_gguf(path, "cuda:0", keep_packed=packed)
        assert isinstance(w.layers[0].wqkv, Int4Weight) == packed
        ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=64)
        eng = LLMEngine(cfg, ec, device="cuda:0", weights=w)
        p = _prompts(cfg.vocab_size, (90,))[0]
        eng.add_request(p, SamplingParams(max_tokens=4))
        rows = []
        while eng.has_unfinished():
            step = eng.scheduler.schedule()
            batch = eng._build_batch(step)
            logits = eng.decoder.forward(batch)
            if logits.shape[0]:
                rows.append(logits[-1].float().clone())
            eng._commit(step, eng.decoder.greedy_tokens(logits).tolist())
        assert eng.ops.check_status() == 0
        outs.append(rows[0])          # the prompt's last position: identical inputs in both runs
    err = (outs[0] - outs[1]).abs().max().item()
    assert err < 0.05 * outs[1].abs().max().item() + 1e-3, err


def test_fp8_kv_cache_on_the_gpu_matches_the_cpu_oracle_path():
    """e4m3 KV pool: written by the rope kernel, read by the generic attention kernel. Compared with the
    same engine on bf16 KV (fp8 tolerance) and checked to really hold one byte per value."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("qwen3-tiny")
    outs = []
    for kvd in ("bf16", "fp8_e4m3"):
        ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=64, kv_cache_dtype=kvd,
                          use_cuda_graphs=False)
        eng = LLMEngine(cfg, ec, device="cuda:0", seed=1)
        assert eng.kv.store.element_size() == (2 if kvd == "bf16" else 1)
        p = _prompts(cfg.vocab_size, (150,))[0]
        eng.add_request(p, SamplingParams(max_tokens=3))
        rows = []
        while eng.has_unfinished():
            step = eng.scheduler.schedule()
            batch = eng._build_batch(step)
            logits = eng.decoder.forward(batch)
            if logits.shape[0]:
                rows.append(logits[-1].float().clone())
            eng._commit(step, eng.decoder.greedy_tokens(logits).tolist())
        assert eng.ops.check_status() == 0
        outs.append(rows[0])
    err = (outs[0] - outs[1]).abs().max().item() / (outs[0].abs().max().item() + 1e-6)
    assert 0 < err < 0.08, err


def test_gpt_oss_checkpoint_keeps_mxfp4_experts_packed_on_the_gpu(tmp_path):
    """The same synthetic gpt-oss checkpoint loaded on the GPU keeps its experts as MXFP4 stacks (grouped
    packed GEMM) and gives the logits of the CPU load that expands them to bf16."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.ops.fp4 import Fp4ExpertStack
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from test_formats_cpu import write_gpt_oss_checkpoint
    cfg = preset("gpt-oss-tiny")
    write_gpt_oss_checkpoint(tmp_path, cfg, init_random_weights(cfg, device="cpu", seed=4))
    outs = []
    for device in ("cuda:0", "cpu"):
        cfg2, w2, _ = load_hf_checkpoint(str(tmp_path), device=device)
        assert isinstance(w2.layers[0].exp_gate_up, Fp4ExpertStack) == (device != "cpu")
        ec = EngineConfig(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=32)
        eng = LLMEngine(cfg2, ec, device=device, weights=w2)
        p = _prompts(cfg2.vocab_size, (40,))[0]
        eng.add_request(p, SamplingParams(max_tokens=1))
        step = eng.scheduler.schedule()
        logits = eng.decoder.forward(eng._build_batch(step))
        outs.append(logits[-1].float().cpu())
        if device != "cpu":
            assert eng.ops.check_status() == 0
    err = (outs[0] - outs[1]).abs().max().item() / (outs[1].abs().max().item() + 1e-6)
    assert err < 0.05, err


def test_smoke_entry_point():
    """The entry point the build check runs on a GPU: tiny prefill + decode through the kernels, compared
    with the PyTorch reference operators on the same weights (which must stay off the graph path)."""
    import __graft_entry__ as entry
    entry.smoke()


def test_rare_samplers_logprobs_and_beam_search_on_the_gpu():
    """The host-side logit processors edit CUDA logit rows before the device sampler; log-probabilities and
    beam search read them. Same invariants as on the CPU: bans hold, seeded runs repeat, width-1 beam = greedy."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("qwen3-tiny")
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=128)
    eng = LLMEngine(cfg, ec, device="cuda:0", seed=3)
    prompt = _prompts(cfg.vocab_size, (12,), seed=2)
    base = eng.generate(prompt, SamplingParams(max_tokens=8))[0]
    banned = eng.generate(prompt, SamplingParams(max_tokens=8, bad_words=[[base[0]]]))[0]
    assert base[0] not in banned
    sp = dict(max_tokens=8, temperature=1.0, seed=7, typical_p=0.8, dry_multiplier=0.8, mirostat_mode=2, mirostat_tau=3.0)
    a = eng.generate(prompt, SamplingParams(**sp))[0]
    b = eng.generate(prompt, SamplingParams(**sp))[0]
    assert a == b and len(a) == 8
    rid = eng.add_request(prompt[0], SamplingParams(max_tokens=4, logprobs=True, top_logprobs=3))
    req = eng.requests[rid]
    evs = []
    while eng.has_unfinished():
        evs += [e for e in eng.step() if e.request_id == rid]
    lps = [x for e in evs for x in (e.logprobs or [])]
    tops = [x for e in evs for x in (e.top_logprobs or [])]
    assert len(lps) == len(tops) == 4 and all(lp <= 1e-6 for lp in lps)
    for tok, lp, alt in zip(req.output, lps, tops):
        # greedy: the pick has the best alternative's log-probability (bf16 logits tie often, so the ids may differ)
        assert abs(alt[0][1] - lp) < 1e-3 and len(alt) == 3 and alt[0][1] >= alt[1][1] >= alt[2][1]
    one = eng.beam_search(prompt[0], beam_width=1, max_tokens=6, length_penalty=0.0, eos_token_id=-1)
    assert len(one) == 1 and len(one[0][0]) == 6 and one[0][1] <= 0.0
    two = eng.beam_search(prompt[0], beam_width=2, max_tokens=6, length_penalty=0.0, eos_token_id=-1)
    assert len(two) == 2 and two[0][1] >= two[1][1] and two[0][0] != two[1][0]
    assert not eng.requests
    assert eng.ops.check_status() == 0


def test_speculation_on_the_gpu_greedy_and_sampled():
    """Draft-model speculation with device-side acceptance: greedy text is unchanged, a draft equal to the target
    is accepted in full for greedy and for sampled requests, and the proposer issues one staged copy per call."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg = preset("qwen3-tiny")
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=128)
    base = LLMEngine(cfg, ec, device="cuda:0", seed=3)
    prompts = _prompts(cfg.vocab_size, (12, 30), seed=4)
    want = base.generate(prompts, SamplingParams(max_tokens=12))
    dm = LLMEngine(cfg, ec, device="cuda:0", seed=3, weights=base.weights)
    dm.enable_draft_model(cfg, weights=base.weights, k=3)
    got = dm.generate(prompts, SamplingParams(max_tokens=12))
    # the verify rows go through the prefill-shaped kernels: bf16 near-ties may flip a token, after which texts differ
    same = sum(a == b for a, b in zip(got, want))
    assert same >= 1 and dm.stats.spec_proposed > 0
    assert dm.stats.spec_accepted >= 0.8 * dm.stats.spec_proposed
    assert dm.proposer.h2d_copies == 1
    p0, a0 = dm.stats.spec_proposed, dm.stats.spec_accepted
    sp = lambda: SamplingParams(max_tokens=12, temperature=0.8, seed=5)
    s1 = dm.generate(prompts, sp())
    assert all(len(o) == 12 for o in s1)
    prop, acc = dm.stats.spec_proposed - p0, dm.stats.spec_accepted - a0
    assert prop > 0 and acc >= 0.8 * prop                       # same model drafts from (nearly) the same distribution
    ng = LLMEngine(cfg, EngineConfig(max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=128,
                                     speculative="ngram"), device="cuda:0", seed=3, weights=base.weights)
    rep = [prompts[0][:6] * 4]
    assert all(len(o) == 10 for o in ng.generate(rep, SamplingParams(max_tokens=10, temperature=0.7, seed=1)))


def test_gguf_mixed_k_quants_stay_packed_on_the_gpu(tmp_path):
    """A Q4_K_M-style file (attn_v and ffn_down in Q6_K, token embeddings in Q8_0-eligible shapes) keeps every
    projection packed: q|k|v becomes a stack of differently typed parts. Same logits as the bf16 expansion, for a
    prompt (GEMM path) and for single-token decode steps (dp4a path)."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.cpu_engine import write_tiny_llama_gguf
    from fllm_b200.formats import quant
    from fllm_b200.formats.loader import load_gguf
    from fllm_b200.ops.int4 import Int4Weight
    from fllm_b200.ops.intk import IntKWeight, StackedWeight
    from fllm_b200.runtime import LLMEngine, SamplingParams
    cfg0 = preset("tiny-llama")
    cfg0.intermediate_size = 1024
    path = str(tmp_path / "mixed.gguf")
    write_tiny_llama_gguf(path, cfg0, seed=5,
                          qtype_for=lambda n: quant.Q6_K if ("attn_v" in n or "ffn_down" in n) else (quant.Q5_K if "attn_output" in n else None))
    outs, toks = [], []
    for packed in (True, False):
        cfg, w, _ = load_gguf(path, "cuda:0", keep_packed=packed)
        if packed:
            lw = w.layers[0]
            assert isinstance(lw.wqkv, StackedWeight) and isinstance(lw.wqkv.parts[2], IntKWeight) and isinstance(lw.wqkv.parts[0], Int4Weight)
            assert isinstance(lw.w_down, IntKWeight) and lw.w_down.fmt == 6 and isinstance(lw.wo, IntKWeight) and lw.wo.fmt == 5
            assert isinstance(lw.w_gate_up, Int4Weight)
        ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=64, use_cuda_graphs=False)
        eng = LLMEngine(cfg, ec, device="cuda:0", weights=w)
        p = _prompts(cfg.vocab_size, (70,))[0]
        lg = eng.token_logits(p)
        outs.append(lg[-1].float().cpu())
        toks.append(eng.generate([p], SamplingParams(max_tokens=6))[0])
        assert eng.ops.check_status() == 0
    err = (outs[0] - outs[1]).abs().max().item()
    assert err < 0.05 * outs[1].abs().max().item() + 1e-3, err
    assert len(toks[0]) == 6


def test_encoder_on_the_gpu_matches_the_pytorch_path():
    """A BERT-shaped encoder (random weights): hidden states, pooled embeddings and classifier logits from the native
    operators (tcgen05 GEMMs, bidirectional attention kernels) against the PyTorch operators on the same weights."""
    from fllm_b200.models.encoder import Encoder, EncoderConfig, init_random_encoder
    from fllm_b200.ops import get_ops
    from fllm_b200.ops.reference import RefOps
    cfg = EncoderConfig(vocab_size=1000, hidden_size=256, num_layers=2, num_heads=4, intermediate_size=512, max_position=512, num_labels=2)
    w = init_random_encoder(cfg, "cuda:0", torch.bfloat16, seed=1)
    g = torch.Generator().manual_seed(2)
    seqs = [torch.randint(0, 1000, (n,), generator=g).tolist() for n in (7, 150, 33, 300)]
    nat = Encoder(cfg, w, get_ops("cuda"), "cuda:0")
    ref = Encoder(cfg, w, RefOps(), "cuda:0")
    a, b = nat.forward(seqs).float(), ref.forward(seqs).float()
    assert (a - b).abs().max().item() < 0.05 * b.abs().max().item()
    ea, eb = nat.embed(seqs), ref.embed(seqs)
    assert torch.nn.functional.cosine_similarity(ea, eb).min().item() > 0.999
    assert (nat.classify(seqs) - ref.classify(seqs)).abs().max().item() < 0.05
    assert nat.ops.check_status() == 0
