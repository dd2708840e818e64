"""Speculative decoding beyond the greedy chain: the exact accept / residual rule for sampled requests
(rust/engine/src/speculative.rs:103), its wiring into the engine, and the draft proposer's batching."""
import numpy as np
import torch

from fllm_b200.config import EngineConfig, preset
from fllm_b200.models.weights import init_random_weights
from fllm_b200.ops.reference import RefOps, philox_uniform, philox_uniform_np
from fllm_b200.runtime.engine import LLMEngine
from fllm_b200.runtime.request import SamplingParams


def _row(temp, draw, seed):
    return (temp, 1.0, 0.0, 1.0, 0.0, 0.0, 0, draw, seed)


def test_vector_philox_equals_the_scalar_one():
    idx = np.array([0, 1, 77, 0xFFFFFFFF, 123456], dtype=np.uint64)
    a = philox_uniform_np(0xABCDEF012345, 9, idx)
    assert np.allclose(a, [philox_uniform(0xABCDEF012345, 9, int(i)) for i in idx])


def test_sampled_rule_emits_the_target_distribution():
    """Whatever the draft distribution, the first emitted token is distributed as the target's p."""
    ops = RefOps()
    V, n = 6, 6000
    g = torch.Generator().manual_seed(0)
    tl = torch.randn(2, V, generator=g) * 1.5                     # rows: position 0 and the bonus row
    dl = torch.randn(1, V, generator=g) * 1.5
    p = torch.softmax(tl[0], -1).numpy()
    q = torch.softmax(dl[0], -1).numpy()
    rng = np.random.default_rng(1)
    xs = rng.choice(V, size=n, p=q / q.sum())                     # drafts drawn from q
    counts = np.zeros(V)
    acc = 0
    for t in range(n):
        n_acc, out = ops.spec_verify_sampled(tl, dl, torch.tensor([[int(xs[t])]], dtype=torch.int32), [_row(1.0, 0, 1000 + t)])
        counts[int(out[0, 0])] += 1
        acc += int(n_acc[0])
    emp = counts / n
    assert np.abs(emp - p).max() < 0.03, (emp, p)
    expect_acc = np.minimum(p, q).sum()                           # 1 - total variation distance
    assert abs(acc / n - expect_acc) < 0.03
    # point-mass drafts (no draft logits): accepted with probability p(x), otherwise a draw from p without x
    counts[:] = 0
    x = int(np.argmax(p))
    for t in range(n):
        _, out = ops.spec_verify_sampled(tl, None, torch.tensor([[x]], dtype=torch.int32), [_row(1.0, 0, 5000 + t)])
        counts[int(out[0, 0])] += 1
    assert np.abs(counts / n - p).max() < 0.03


def test_ragged_rows_and_greedy_rule():
    ops = RefOps()
    draft = torch.tensor([[5, 6, 7], [1, 2, -1]], dtype=torch.int32)
    flat = torch.tensor([9, 5, 6, 8, 0, 1, 2, 3], dtype=torch.int32)   # seq 0 rows 1..4, seq 1 rows 5..7
    n_acc, out = ops.spec_verify_greedy(draft, flat, torch.tensor([3, 2], dtype=torch.int32), torch.tensor([1, 5], dtype=torch.int32))
    assert n_acc.tolist() == [2, 2]
    assert out[0, :3].tolist() == [5, 6, 8] and out[1].tolist()[:3] == [1, 2, 3]
    # temperature 0 through the sampled rule is the greedy rule
    tl = torch.full((8, 12), -5.0)
    for r, t in enumerate(flat.tolist()):
        tl[r, t] = 3.0
    n2, out2 = ops.spec_verify_sampled(tl, None, draft, [_row(0.0, 0, 1), _row(0.0, 0, 2)],
                                       torch.tensor([3, 2], dtype=torch.int32), torch.tensor([1, 5], dtype=torch.int32))
    assert n2.tolist() == [2, 2] and out2[0, :3].tolist() == [5, 6, 8] and out2[1, :3].tolist() == [1, 2, 3]


def _eng(cfg, w, **kw):
    return LLMEngine(cfg, EngineConfig(max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=96, **kw), device="cpu", weights=w)


def test_engine_speculates_sampled_requests():
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu")
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (10, 23)]
    prompts[0] = prompts[0][:5] * 4
    sp = lambda: SamplingParams(max_tokens=12, temperature=0.8, seed=21)
    assert sp().spec_mode == "sampled" and SamplingParams(temperature=0.8, top_k=5).spec_mode is None
    # a draft equal to the target proposes from the same distribution: everything is accepted
    dm = _eng(cfg, w)
    dm.enable_draft_model(cfg, weights=w, k=3)
    out1 = dm.generate(prompts, sp())
    assert dm.stats.spec_proposed > 0 and dm.stats.spec_accepted == dm.stats.spec_proposed
    assert dm.proposer.h2d_copies == 1                      # one staged copy per call, whatever k is
    assert all(len(o) == 12 for o in out1)
    dm2 = _eng(cfg, w)
    dm2.enable_draft_model(cfg, weights=w, k=3)
    assert dm2.generate(prompts, sp()) == out1              # seeded: repeatable
    # an unrelated draft and the n-gram lookup (point-mass drafts) still produce valid seeded output
    other = _eng(cfg, w)
    other.enable_draft_model(cfg, k=4, seed=99)
    o2 = other.generate(prompts, sp())
    assert all(len(o) == 12 and all(0 <= t < cfg.vocab_size for t in o) for o in o2)
    assert other.stats.spec_accepted < other.stats.spec_proposed
    ng = _eng(cfg, w, speculative="ngram")
    o3 = ng.generate(prompts, sp())
    assert all(len(o) == 12 for o in o3)
    # greedy and sampled requests verified in the same step
    mixed = _eng(cfg, w)
    mixed.enable_draft_model(cfg, weights=w, k=3)
    base = _eng(cfg, w)
    want = base.generate([prompts[1]], SamplingParams(max_tokens=10))[0]
    ids = [mixed.add_request(prompts[0], sp()), mixed.add_request(prompts[1], SamplingParams(max_tokens=10))]
    got = {}
    while mixed.has_unfinished():
        for ev in mixed.step():
            got.setdefault(ev.request_id, []).extend(ev.token_ids)
    assert got[ids[1]] == want and len(got[ids[0]]) == 12


def test_draft_tree_masks_and_greedy_verification():
    from fllm_b200.runtime.speculative import DraftTree
    tree = DraftTree.from_chains([[5, 6, 7], [5, 9], [4, 4, 4]])
    assert tree.tokens == [5, 6, 7, 9, 4, 4, 4] and tree.parents == [-1, 0, 1, 0, -1, 4, 5]
    assert tree.depths() == [0, 1, 2, 1, 0, 1, 2]
    assert tree.masks() == [0b1, 0b11, 0b111, 0b1001, 0b10000, 0b110000, 0b1110000]
    # the target wants 5, then 9 after node 0, then 2 after node 3: path [0, 3], bonus token 2
    assert tree.verify_greedy(5, [9, 0, 0, 2, 0, 0, 0]) == ([0, 3], 2)
    assert tree.verify_greedy(8, [0] * 7) == ([], 8)
    assert tree.verify_greedy(4, [0, 0, 0, 0, 4, 4, 1]) == ([4, 5, 6], 1)
    import pytest
    with pytest.raises(ValueError):
        DraftTree([1, 2], [0, -1])


def test_tree_attention_reference_equals_chain_attention_on_each_path():
    """A node of a draft tree must see exactly what it would see if its root-to-node path were a plain sequence."""
    from fllm_b200.runtime.speculative import DraftTree
    ops = RefOps()
    g = torch.Generator().manual_seed(0)
    hq, hkv, D, bs, ctx = 4, 2, 64, 16, 21
    tree = DraftTree.from_chains([[5, 6, 7], [5, 9], [4, 4]])
    M = len(tree)
    nblk = (ctx + M + bs - 1) // bs
    kc = torch.randn(nblk, hkv, bs, D, generator=g)
    vc = torch.randn(nblk, hkv, bs, D, generator=g)
    tables = torch.arange(nblk, dtype=torch.int32).view(1, nblk)
    q = torch.randn(M, hq * D, generator=g)
    rs = torch.zeros(M, dtype=torch.int32)
    pos = torch.full((M,), ctx + M - 1, dtype=torch.int32)
    y = ops.attention_tree(q, kc, vc, tables, rs, pos, torch.tensor(tree.masks_i64()), torch.full((M,), ctx, dtype=torch.int32),
                           hq, hkv, D, D ** -0.5)
    flat_k = kc.permute(1, 0, 2, 3).reshape(hkv, nblk * bs, D)
    flat_v = vc.permute(1, 0, 2, 3).reshape(hkv, nblk * bs, D)
    for i in range(M):
        path, p = [i], tree.parents[i]
        while p >= 0:
            path.append(p)
            p = tree.parents[p]
        idx = list(range(ctx)) + [ctx + j for j in sorted(path)]
        k = flat_k[:, idx].repeat_interleave(hq // hkv, 0)
        v = flat_v[:, idx].repeat_interleave(hq // hkv, 0)
        s = torch.einsum("hd,hnd->hn", q[i].view(hq, D), k) * D ** -0.5
        want = torch.einsum("hn,hnd->hd", torch.softmax(s, -1), v).reshape(-1)
        assert (y[i] - want).abs().max().item() < 1e-4


def test_suffix_proposer_drafts_from_earlier_requests():
    from fllm_b200.runtime.speculative import SuffixProposer
    p = SuffixProposer(k=4, max_n=3, min_n=2)
    assert p.propose([1, 2, 3, 4]) == []
    p.observe([9, 8, 7, 6, 5, 4, 3])
    assert p.propose([100, 8, 7]) == [6, 5, 4, 3]            # a different request ends in a known 2-gram
    assert p.propose([8, 7, 6, 50, 8, 7]) == [6, 50, 8, 7]   # its own context wins over the shared index
    # through the engine: the second, identical request is drafted from the first one's text and keeps it
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cpu")
    g = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, cfg.vocab_size, (17,), generator=g).tolist()
    base = _eng(cfg, w).generate([prompt], SamplingParams(max_tokens=12))[0]
    eng = _eng(cfg, w, speculative="suffix")
    first = eng.generate([prompt], SamplingParams(max_tokens=12))[0]
    steps0, acc0 = eng.stats.steps, eng.stats.spec_accepted
    second = eng.generate([prompt], SamplingParams(max_tokens=12))[0]
    assert first == base and second == base
    assert eng.stats.spec_accepted - acc0 >= 6 and eng.stats.steps - steps0 < steps0


def test_suffix_index_survives_a_restart(tmp_path, monkeypatch):
    """The suffix source keeps its documents in $FLLM_SUFFIX_DIR under the model's digest: a second engine drafts from the
    first one's outputs; a file of another model or a damaged file counts as absent."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from fllm_b200.runtime.speculative import SuffixProposer
    monkeypatch.setenv("FLLM_SUFFIX_DIR", str(tmp_path))
    cfg = preset("tiny-llama")
    cfg.vocab_size = 512
    ec = EngineConfig(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=32, speculative="suffix", draft_tokens=3)
    a = LLMEngine(cfg, ec, device="cpu", seed=2)
    prompt = [5, 9, 2, 7, 11, 3]
    out = a.generate([prompt], SamplingParams(max_tokens=12, temperature=0.0))[0]
    a.close()
    files = list(tmp_path.glob("suffix-*.bin"))
    assert len(files) == 1
    b = LLMEngine(cfg, ec, device="cpu", seed=2)
    assert b.proposer.documents == [prompt + out]
    assert b.proposer.propose([99, 98, 5, 9]) == [2, 7, 11]            # drafts come from the other engine's text
    other = SuffixProposer(3)
    assert other.load(str(files[0]), b"another model") == 0
    files[0].write_bytes(files[0].read_bytes()[:-5])
    assert SuffixProposer(3).load(str(files[0]), b._suffix_digest) == 0
