"""Hybrid and recurrent models through the engine on a GPU: the sm_100a kernels against the PyTorch statement of the
same ops on the same weights, chunked prefill against one shot, and captured decode steps against eager ones."""
import pytest
import torch

from fllm_b200.config import EngineConfig, ModelConfig, preset
from fllm_b200.runtime.engine import LLMEngine
from fllm_b200.runtime.request import SamplingParams

pytestmark = pytest.mark.gpu


def _cfg(kinds, ssm):
    return ModelConfig(vocab_size=512, hidden_size=256, num_layers=len(kinds), num_heads=4, num_kv_heads=2, head_dim=64,
                       intermediate_size=512, layer_kinds=kinds, ffn_kinds=["none" if k == "mamba1" else "glu" for k in kinds],
                       ssm=ssm, tie_embeddings=True)


CASES = [
    (["mamba2", "attention", "mamba2"], dict(d_inner=512, d_state=128, d_conv=4, n_groups=2, head_dim=64, n_heads=8, norm_groups=1, conv_bias=True)),
    (["mamba1", "mamba1"], dict(d_inner=512, d_state=16, d_conv=4, dt_rank=16, conv_bias=True)),
    (["gated_delta", "attention", "gated_delta"], dict(num_k_heads=2, num_v_heads=4, head_k_dim=128, head_v_dim=128, d_conv=4)),
    (["shortconv", "attention", "shortconv"], dict(d_conv=3, conv_bias=True)),
]


def _engine(cfg, ops=None, chunk=64, graphs=False, weights=None, max_len=512):
    ec = EngineConfig(max_num_seqs=8, max_num_batched_tokens=chunk, max_model_len=max_len, num_kv_blocks=max_len // 2, block_size=16,
                      use_cuda_graphs=graphs)
    return LLMEngine(cfg, ec, device="cuda:0", seed=3, ops=ops, weights=weights)


@pytest.mark.parametrize("kinds,ssm", CASES)
def test_native_kernels_match_reference_ops(kinds, ssm):
    from fllm_b200.ops.reference import RefOps
    cfg = _cfg(kinds, ssm)
    nat = _engine(cfg)
    assert type(nat.ops).__name__ == "NativeOps"
    ref = _engine(cfg, ops=RefOps(), weights=nat.weights)
    toks = torch.randint(0, 512, (150,), generator=torch.Generator().manual_seed(5)).tolist()
    a, b = nat.token_logits(toks), ref.token_logits(toks)                   # three steps: states cross two boundaries
    err = float((a - b).norm() / b.norm())
    assert err < 2e-2, err
    assert int(nat.ops.status.item()) == 0


@pytest.mark.parametrize("kinds,ssm", CASES)
def test_schedule_and_graphs_do_not_change_tokens(kinds, ssm):
    cfg = _cfg(kinds, ssm)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 512, (n,), generator=g).tolist() for n in (37, 5, 150, 64)]
    sp = SamplingParams(max_tokens=12, temperature=0.0)
    base = _engine(cfg, chunk=512)
    want = base.generate(prompts, sp)
    w = base.weights
    assert _engine(cfg, chunk=48, weights=w).generate(prompts, sp) == want
    eng = _engine(cfg, chunk=512, graphs=True, weights=w)
    assert eng.generate(prompts, sp) == want
    assert eng.generate(prompts[:2], sp) == want[:2]                        # rows are reused by later requests
    assert len(eng.blocks.state_free) == eng.rstate.slots - 1


def test_latent_attention_engine():
    """The latent-attention kernel inside the engine against the PyTorch statement on the same weights, and captured
    decode steps against eager ones."""
    from fllm_b200.ops.reference import RefOps
    cfg = preset("mla-tiny")
    nat = _engine(cfg)
    ref = _engine(cfg, ops=RefOps(), weights=nat.weights)
    toks = torch.randint(0, 4096, (150,), generator=torch.Generator().manual_seed(5)).tolist()
    a, b = nat.token_logits(toks), ref.token_logits(toks)
    assert float((a - b).norm() / b.norm()) < 2e-2
    prompts = [toks[:37], toks[40:45], toks]
    sp = SamplingParams(max_tokens=10, temperature=0.0)
    want = _engine(cfg, chunk=512, weights=nat.weights).generate(prompts, sp)
    assert _engine(cfg, chunk=512, graphs=True, weights=nat.weights).generate(prompts, sp) == want


def test_deepseek_moe_engine():
    """Latent attention + routed experts (family router in tensor ops, grouped GEMMs) + shared experts on the GPU against
    the PyTorch statement on the same weights."""
    from fllm_b200.ops.reference import RefOps
    cfg = preset("deepseek-moe-tiny")
    nat = _engine(cfg)
    ref = _engine(cfg, ops=RefOps(), weights=nat.weights)
    toks = torch.randint(0, 4096, (100,), generator=torch.Generator().manual_seed(5)).tolist()
    a, b = nat.token_logits(toks), ref.token_logits(toks)
    err = (a - b).norm(dim=1) / b.norm(dim=1)
    assert float(err.median()) < 2e-2 and int((err > 0.1).sum()) <= 3, err          # a near-tie in the router may flip a row
    out = _engine(cfg, chunk=512, graphs=True, weights=nat.weights).generate([toks[:20], toks[30:70]], SamplingParams(max_tokens=8, temperature=0.0))
    assert [len(o) for o in out] == [8, 8]


@pytest.mark.parametrize("name", ["rwkv7-tiny", "rwkv6-tiny"])
def test_rwkv_engine(name):
    from fllm_b200.ops.reference import RefOps
    cfg = preset(name)
    nat = _engine(cfg)
    ref = _engine(cfg, ops=RefOps(), weights=nat.weights)
    toks = torch.randint(0, 4096, (150,), generator=torch.Generator().manual_seed(5)).tolist()
    a, b = nat.token_logits(toks), ref.token_logits(toks)
    assert float((a - b).norm() / b.norm()) < 3e-2
    prompts = [toks[:37], toks[40:45], toks]
    sp = SamplingParams(max_tokens=10, temperature=0.0)
    want = _engine(cfg, chunk=512, weights=nat.weights).generate(prompts, sp)
    assert _engine(cfg, chunk=512, graphs=True, weights=nat.weights).generate(prompts, sp) == want


def test_long_prompt_chunks_take_the_matrix_form(monkeypatch):
    """With the switch on, prompt chunks of 512 tokens or more run the Mamba-2 layers in their matrix form; a decode row
    of another sequence in the same step stays on the scan kernel. Logits against the PyTorch operators, tokens against
    a run whose chunks are too short for the matrix form."""
    import fllm_b200.ops.recurrent as rec
    from fllm_b200.ops.reference import RefOps
    monkeypatch.setattr(rec, "SSD_MIN_TOKENS", 512)
    cfg = preset("bamba-tiny")
    nat = _engine(cfg, chunk=1024, max_len=1024)
    ref = _engine(cfg, ops=RefOps(), chunk=1024, weights=nat.weights, max_len=1024)
    toks = torch.randint(0, 4096, (400,), generator=torch.Generator().manual_seed(5)).tolist() * 2       # 800 tokens
    a, b = nat.token_logits(toks[:500] + toks[:200]), ref.token_logits(toks[:500] + toks[:200])
    assert float((a - b).norm() / b.norm()) < 2e-2
    sp = SamplingParams(max_tokens=8, temperature=0.0)
    prompts = [toks[:300], toks, toks[100:140]]
    want = _engine(cfg, chunk=256, weights=nat.weights, max_len=1024).generate(prompts, sp)
    assert _engine(cfg, chunk=1024, weights=nat.weights, max_len=1024).generate(prompts, sp) == want


def test_hybrid_presets_decode():
    for name in ("mamba2-tiny", "bamba-tiny", "mamba1-tiny"):
        eng = _engine(preset(name), chunk=256, graphs=True)
        out = eng.generate([[1, 2, 3, 4, 5] * 9, [7] * 20], SamplingParams(max_tokens=8, temperature=0.0))
        assert [len(o) for o in out] == [8, 8]


def test_mamba1_long_prompt_sequence_parallel():
    """A prompt long enough for the segmented Mamba-1 scan gives the chunk-by-chunk walk's tokens and the fp32
    reference's logits."""
    from fllm_b200.ops.reference import RefOps
    cfg = preset("mamba1-tiny")
    nat = _engine(cfg, chunk=1024, max_len=1024)
    ref = _engine(cfg, ops=RefOps(), chunk=1024, weights=nat.weights, max_len=1024)
    toks = torch.randint(0, 4096, (800,), generator=torch.Generator().manual_seed(6)).tolist()
    a, b = nat.token_logits(toks[:700]), ref.token_logits(toks[:700])
    assert float((a - b).norm() / b.norm()) < 2e-2
    sp = SamplingParams(max_tokens=8, temperature=0.0)
    prompts = [toks[:300], toks, toks[100:140]]
    want = _engine(cfg, chunk=256, weights=nat.weights, max_len=1024).generate(prompts, sp)
    assert _engine(cfg, chunk=1024, weights=nat.weights, max_len=1024).generate(prompts, sp) == want
