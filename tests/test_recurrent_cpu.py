"""Recurrent and hybrid families on CPU: teacher-forced logits of tiny random checkpoints against Hugging Face
`transformers` (fp32, chunked prefill so that states cross step boundaries), and scheduling invariants of the state
rows (chunked = one shot = one sequence at a time; rows are returned when sequences finish)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from fllm_b200.config import EngineConfig, ModelConfig
from fllm_b200.runtime.engine import LLMEngine
from fllm_b200.runtime.request import SamplingParams


def _tiny(kind):
    torch.manual_seed(0)
    if kind == "mamba":
        from transformers import MambaConfig, MambaForCausalLM
        return MambaForCausalLM(MambaConfig(vocab_size=300, hidden_size=64, state_size=16, num_hidden_layers=2, expand=2,
                                            conv_kernel=4, time_step_rank=4, use_mambapy=False))
    if kind == "mamba2":
        from transformers import Mamba2Config, Mamba2ForCausalLM
        return Mamba2ForCausalLM(Mamba2Config(vocab_size=300, hidden_size=64, state_size=16, num_hidden_layers=2, num_heads=4,
                                              head_dim=32, n_groups=2, expand=2, conv_kernel=4, chunk_size=8))
    if kind == "bamba":
        from transformers import BambaConfig, BambaForCausalLM
        return BambaForCausalLM(BambaConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                                            num_attention_heads=4, num_key_value_heads=2, attn_layer_indices=[1], mamba_n_heads=4,
                                            mamba_d_head=32, mamba_n_groups=1, mamba_d_state=16, mamba_d_conv=4, mamba_expand=2,
                                            mamba_chunk_size=8, max_position_embeddings=256))
    if kind == "lfm2":
        from transformers import Lfm2Config, Lfm2ForCausalLM
        return Lfm2ForCausalLM(Lfm2Config(vocab_size=300, hidden_size=64, intermediate_size=192, num_hidden_layers=3,
                                          num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=256,
                                          layer_types=["conv", "full_attention", "conv"], conv_L_cache=3, block_multiple_of=16))
    if kind == "jamba":
        from transformers import JambaConfig, JambaForCausalLM
        return JambaForCausalLM(JambaConfig(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=4,
                                            num_attention_heads=4, num_key_value_heads=2, num_experts=4, num_experts_per_tok=2,
                                            expert_layer_period=2, expert_layer_offset=1, attn_layer_period=2, attn_layer_offset=1,
                                            mamba_d_state=16, mamba_d_conv=4, mamba_expand=2, mamba_dt_rank=8, use_mamba_kernels=False,
                                            max_position_embeddings=256))
    if kind in ("granite_dense", "granite_moe"):
        from transformers import GraniteMoeHybridConfig, GraniteMoeHybridForCausalLM
        return GraniteMoeHybridForCausalLM(GraniteMoeHybridConfig(
            vocab_size=300, hidden_size=64, intermediate_size=48, shared_intermediate_size=96, num_hidden_layers=3,
            num_attention_heads=4, num_key_value_heads=2, num_local_experts=0 if kind == "granite_dense" else 4, num_experts_per_tok=2,
            layer_types=["mamba", "attention", "mamba"], mamba_n_heads=4, mamba_d_head=32, mamba_n_groups=1, mamba_d_state=16,
            mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=8, embedding_multiplier=3.0, logits_scaling=2.0, residual_multiplier=0.5,
            attention_multiplier=0.2, position_embedding_type="nope" if kind == "granite_dense" else "rope",
            max_position_embeddings=256))
    if kind in ("granitemoe", "granitemoeshared"):
        import transformers as tf
        common = dict(vocab_size=300, hidden_size=64, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      num_local_experts=4, num_experts_per_tok=2, embedding_multiplier=3.0, logits_scaling=2.0, residual_multiplier=0.5,
                      attention_multiplier=0.2, max_position_embeddings=256)
        if kind == "granitemoe":
            return tf.GraniteMoeForCausalLM(tf.GraniteMoeConfig(**common))
        return tf.GraniteMoeSharedForCausalLM(tf.GraniteMoeSharedConfig(**common, shared_intermediate_size=96))
    if kind == "falcon_mamba":
        from transformers import FalconMambaConfig, FalconMambaForCausalLM
        return FalconMambaForCausalLM(FalconMambaConfig(vocab_size=300, hidden_size=64, state_size=16, num_hidden_layers=2, expand=2,
                                                        conv_kernel=4, time_step_rank=8, use_mambapy=False))
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["mamba", "mamba2", "bamba", "lfm2", "jamba", "falcon_mamba", "granite_dense", "granite_moe",
                                  "granitemoe", "granitemoeshared"])
def test_recurrent_families_match_transformers(tmp_path, kind):
    from fllm_b200.formats.loader import load_hf_checkpoint
    m = _tiny(kind).eval().float()
    with torch.no_grad():                      # spread the parameters a trained model would not leave at their init
        for n, p in m.named_parameters():
            if n.endswith(("norm.weight", "layernorm.weight", "norm_f.weight", ".D", "dt_bias")):
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith(("router.weight", "router.layer.weight")):
                p.mul_(20.0)                                  # clear routing decisions
            if n.endswith(("q_proj.weight", "k_proj.weight")):
                p.mul_(12.0)                                  # peaked attention: a wrong rotation or mask moves the logits
    d = str(tmp_path / kind)
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.has_recurrent or kind.startswith("granitemoe")
    if kind == "bamba":
        # The config rotates half of each head (as the published checkpoints were trained and as the engine does); this
        # version of the oracle rotates the whole head whatever the config says, so the width follows the oracle here.
        assert cfg.rot_dim == cfg.head_dim // 2
        cfg.rotary_dim = None
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)               # three steps of at most 16 rows: the states cross two boundaries
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    scale = float(want.abs().max())
    err = (got - want).abs().max(dim=1).values / scale
    # fp32 end to end; routed layers round their router scores to bf16, which may flip a near-tie for a token
    routed = bool(cfg.ffn_kinds) and "moe" in cfg.ffn_kinds
    assert float(err.median()) < (1e-2 if routed else 2e-3) and int((err > (5e-2 if routed else 1e-2)).sum()) <= (2 if routed else 0), err
    assert not eng.blocks.seqs and (eng.rstate is None or len(eng.blocks.state_free) == eng.rstate.slots - 1)


def _synthetic(kinds, ssm):
    return ModelConfig(vocab_size=200, hidden_size=64, num_layers=len(kinds), num_heads=2, num_kv_heads=1, head_dim=32,
                       intermediate_size=128, layer_kinds=kinds, ffn_kinds=["none" if k == "mamba1" else "glu" for k in kinds],
                       ssm=ssm, tie_embeddings=True)


SYNTHETIC = [
    (["mamba2", "attention", "mamba2"], dict(d_inner=128, d_state=16, d_conv=4, n_groups=1, head_dim=32, n_heads=4, norm_groups=1)),
    (["mamba1", "mamba1"], dict(d_inner=128, d_state=16, d_conv=4, dt_rank=4)),
    (["gated_delta", "attention"], dict(num_k_heads=2, num_v_heads=4, head_k_dim=32, head_v_dim=32, d_conv=4)),
    (["shortconv", "attention"], dict(d_conv=3, conv_bias=True)),
]


@pytest.mark.parametrize("kinds,ssm", SYNTHETIC)
def test_state_rows_follow_the_schedule(kinds, ssm):
    """The same prompts through one big step, through 16-token chunks interleaved with other sequences' decode
    steps, and one sequence at a time give the same greedy tokens; every state row comes back."""
    cfg = _synthetic(kinds, ssm)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 200, (n,), generator=g).tolist() for n in (37, 5, 70)]

    def run(chunk, ps):
        ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=chunk, max_model_len=256, num_kv_blocks=64, block_size=16)
        eng = LLMEngine(cfg, ec, device="cpu", seed=1)
        assert not eng.cfg.enable_prefix_caching and eng.cfg.speculative == "off"
        out = eng.generate(ps, SamplingParams(max_tokens=6, temperature=0.0))
        assert len(eng.blocks.state_free) == eng.rstate.slots - 1
        return out
    one = run(256, prompts)
    assert run(16, prompts) == one
    assert [run(256, [p])[0] for p in prompts] == one


def test_gated_delta_mixer_matches_transformers():
    """The gated delta rule layer against the Qwen3-Next module of `transformers` (its plain PyTorch path) with the
    module's interleaved projection rows re-ordered into [q | k | v | z | beta | a]."""
    from transformers.models.qwen3_next.configuration_qwen3_next import Qwen3NextConfig
    from transformers.models.qwen3_next.modeling_qwen3_next import Qwen3NextGatedDeltaNet
    from fllm_b200.models.recurrent import RecurrentState, gated_delta_mixer, pack_gated_delta
    from fllm_b200.ops.reference import RefOps
    torch.manual_seed(0)
    Hk, Hv, Dk, Dv, H = 2, 4, 32, 32, 64
    hc = Qwen3NextConfig(hidden_size=H, linear_num_key_heads=Hk, linear_num_value_heads=Hv, linear_key_head_dim=Dk,
                         linear_value_head_dim=Dv, linear_conv_kernel_dim=4, num_hidden_layers=1, vocab_size=100, rms_norm_eps=1e-6)
    mod = Qwen3NextGatedDeltaNet(hc, 0).eval().float()
    with torch.no_grad():
        mod.norm.weight.add_(0.3 * torch.randn_like(mod.norm.weight))
        mod.dt_bias.add_(0.3 * torch.randn_like(mod.dt_bias))
    r = Hv // Hk
    qkvz = mod.in_proj_qkvz.weight.detach().view(Hk, 2 * Dk + 2 * r * Dv, H)      # per key head: q | k | v (r heads) | z (r heads)
    ba = mod.in_proj_ba.weight.detach().view(Hk, 2 * r, H)
    q, k = qkvz[:, :Dk].reshape(-1, H), qkvz[:, Dk:2 * Dk].reshape(-1, H)
    v, z = qkvz[:, 2 * Dk:2 * Dk + r * Dv].reshape(-1, H), qkvz[:, 2 * Dk + r * Dv:].reshape(-1, H)
    b, a = ba[:, :r].reshape(-1, H), ba[:, r:].reshape(-1, H)
    mixer = pack_gated_delta(q, k, v, z, b, a, mod.conv1d.weight.detach(), mod.dt_bias.detach(), mod.A_log.detach(),
                             mod.norm.weight.detach(), mod.out_proj.weight.detach(), torch.float32, "cpu")
    cfg = _synthetic(["gated_delta"], dict(num_k_heads=Hk, num_v_heads=Hv, head_k_dim=Dk, head_v_dim=Dv, d_conv=4, norm_eps=1e-6))

    class Dec:
        pass
    dec = Dec()
    dec.cfg, dec.ops = cfg, RefOps()
    dec.rstate = RecurrentState(cfg, range(1), 3, "cpu", torch.float32)

    class LW:
        pass
    lw = LW()
    lw.mixer = mixer

    class B:
        pass
    x = torch.randn(1, 21, H)
    with torch.no_grad():
        want = mod(x)[0] if isinstance(mod(x), tuple) else mod(x)
    got = []
    for t0, t1 in ((0, 9), (9, 10), (10, 21)):                    # a chunk, one decode row, another chunk
        bt = B()
        bt.q_starts = torch.tensor([0, t1 - t0], dtype=torch.int32)
        bt.seq_state = torch.tensor([1], dtype=torch.int32)
        bt.positions = torch.arange(t0, t1, dtype=torch.int32)
        got.append(gated_delta_mixer(dec, 0, lw, x[0, t0:t1], bt))
    got = torch.cat(got)
    assert float((got - want.reshape(21, H)).abs().max()) < 1e-4


@pytest.mark.parametrize("version,q_lora", [(2, None), (2, 24), (3, 24)])
def test_latent_attention_matches_transformers(tmp_path, version, q_lora):
    """DeepSeek-V2 / V3 with dense feed-forward layers: absorbed latent attention over the 1-row-per-token cache against
    the expanded attention of `transformers`, with YaRN scaling (V3 also scales the softmax)."""
    from fllm_b200.formats.loader import load_hf_checkpoint
    torch.manual_seed(0)
    common = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                  num_key_value_heads=4, kv_lora_rank=32, q_lora_rank=q_lora, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                  first_k_dense_replace=2, n_routed_experts=4, n_shared_experts=1, num_experts_per_tok=2, moe_intermediate_size=32,
                  max_position_embeddings=256,
                  rope_parameters=dict(rope_type="yarn", rope_theta=10000.0, factor=4.0, original_max_position_embeddings=64,
                                       beta_fast=32.0, beta_slow=1.0, mscale=1.0, mscale_all_dim=0.7))
    if version == 2:
        from transformers import DeepseekV2Config, DeepseekV2ForCausalLM
        m = DeepseekV2ForCausalLM(DeepseekV2Config(**common))
    else:
        from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
        m = DeepseekV3ForCausalLM(DeepseekV3Config(n_group=1, topk_group=1, **common))
    m = m.eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "layernorm" in n or n.endswith("norm.weight"):
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith(("q_proj.weight", "q_b_proj.weight", "kv_b_proj.weight", "kv_a_proj_with_mqa.weight")):
                p.mul_(6.0)                                   # peaked attention
    d = str(tmp_path / f"ds{version}")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.has_mla and not cfg.has_recurrent and cfg.rope_scaling.kind == "yarn"
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=256, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (150,), generator=torch.Generator().manual_seed(1)).tolist()      # beyond the original 64 positions
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) < 2e-3 * scale, (float((got - want).abs().max()), scale)


def _rwkv7_oracle(sd, cfg, ids):
    """RWKV-7 one token at a time in fp32, with the states in a dictionary: the published recurrence written without
    any of the engine's pieces (no ragged batch, no kernels, no packed weights)."""
    import torch.nn.functional as F
    C, N, eps = cfg.hidden_size, cfg.ssm["head_dim"], cfg.rms_eps
    H = C // N
    ln = lambda x, n: F.layer_norm(x, (C,), sd[n + ".weight"], sd[n + ".bias"], eps)
    st = {}
    out = []
    for tok in ids:
        x = sd["model.embeddings.weight"][tok]
        v_first = None
        for l in range(cfg.num_layers):
            g = lambda n: sd[f"model.layers.{l}.{n}"]
            if l == 0:
                x = ln(x, "model.layers.0.pre_norm")
            h = ln(x, f"model.layers.{l}.attn_norm")
            xx = st.get(("a", l), torch.zeros(C)) - h
            st[("a", l)] = h
            mix = {c: h + xx * g("attn.x_" + c).reshape(-1) for c in "rwkvag"}
            r, k, v = g("attn.r_proj.weight") @ mix["r"], g("attn.k_proj.weight") @ mix["k"], g("attn.v_proj.weight") @ mix["v"]
            low = lambda n, vec, act=lambda t: t: g(f"attn.{n}_lora.lora.2.weight") @ act(g(f"attn.{n}_lora.lora.0.weight") @ vec)
            decay = torch.exp(-0.6065306597126334 * torch.sigmoid(low("w", mix["w"], torch.tanh) + g("attn.w_lora.lora.2.bias")))
            if l == 0:
                v_first = v
            else:
                v = v + (v_first - v) * torch.sigmoid(low("v", mix["v"]) + g("attn.v_lora.lora.2.bias"))
            a = torch.sigmoid(low("a", mix["a"]) + g("attn.a_lora.lora.2.bias"))
            gate = low("g", mix["g"], torch.sigmoid)
            kk = F.normalize((k * g("attn.k_k")).view(H, N), dim=-1).view(-1)
            k = k * (1 + (a - 1) * g("attn.k_a"))
            S = st.get(("s", l), torch.zeros(H, N, N))
            sa = torch.einsum("hvk,hk->hv", S, -kk.view(H, N))
            S = S * decay.view(H, 1, N) + sa[:, :, None] * (kk * a).view(H, 1, N) + v.view(H, N, 1) * k.view(H, 1, N)
            st[("s", l)] = S
            y = torch.einsum("hvk,hk->hv", S, r.view(H, N)).reshape(1, C)
            y = F.group_norm(y, H, g("attn.g_norm.weight"), g("attn.g_norm.bias"), N * eps).reshape(-1)
            y = y + ((r.view(H, N) * k.view(H, N) * g("attn.r_k")).sum(-1, keepdim=True) * v.view(H, N)).reshape(-1)
            x = x + g("attn.o_proj.weight") @ (y * gate)
            h2 = ln(x, f"model.layers.{l}.ffn_norm")
            xx = st.get(("f", l), torch.zeros(C)) - h2
            st[("f", l)] = h2
            x = x + g("ffn.value.weight") @ torch.relu(g("ffn.key.weight") @ (h2 + xx * g("ffn.x_k").reshape(-1))) ** 2
        out.append(sd["lm_head.weight"] @ ln(x, "model.norm"))
    return torch.stack(out)


def test_rwkv7_matches_token_by_token_recurrence(tmp_path):
    import json
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.formats.safetensors_io import save_file
    from fllm_b200.models.rwkv import random_rwkv7_state_dict
    hf = {"model_type": "rwkv7", "architectures": ["RWKV7ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 3, "head_dim": 16,
          "decay_low_rank_dim": 8, "a_low_rank_dim": 8, "v_low_rank_dim": 8, "gate_low_rank_dim": 16, "intermediate_size": 256,
          "norm_eps": 1e-5, "vocab_size": 300}
    cfg = ModelConfig.from_hf_config(hf)
    sd = random_rwkv7_state_dict(cfg, seed=3)
    json.dump(hf, open(tmp_path / "config.json", "w"))
    save_file(sd, str(tmp_path / "model.safetensors"))
    cfg2, w, _ = load_hf_checkpoint(str(tmp_path), device="cpu", dtype=torch.float32)
    assert cfg2.arch == "rwkv7" and cfg2.has_recurrent
    eng = LLMEngine(cfg2, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    got = eng.token_logits(toks)                       # 16 + 16 + 8 rows: every state crosses two step boundaries
    want = _rwkv7_oracle(sd, cfg, toks)
    assert float((got - want).abs().max()) < 1e-3 * float(want.abs().max())
    # decode after a chunked prefill equals decode after a one-shot prefill
    sp = SamplingParams(max_tokens=6, temperature=0.0)
    big = LLMEngine(cfg2, EngineConfig(max_num_seqs=2, max_num_batched_tokens=64, max_model_len=128, num_kv_blocks=32), device="cpu", weights=w)
    assert eng.generate([toks[:37], toks[:5]], sp) == big.generate([toks[:37], toks[:5]], sp)


@pytest.mark.parametrize("version", [2, 3])
def test_deepseek_routed_and_shared_experts_match_transformers(tmp_path, version):
    """First layer dense, then routed experts with shared experts: V2 with softmax scores and plain top-k, V3 with
    sigmoid scores, a selection bias, groups ranked by their two best experts and renormalised weights."""
    from fllm_b200.formats.loader import load_hf_checkpoint
    torch.manual_seed(0)
    common = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                  num_key_value_heads=4, kv_lora_rank=32, q_lora_rank=None, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16,
                  first_k_dense_replace=1, n_routed_experts=8, n_shared_experts=2, num_experts_per_tok=3, moe_intermediate_size=32,
                  n_group=4, topk_group=2, routed_scaling_factor=1.5, max_position_embeddings=256)
    if version == 2:
        from transformers import DeepseekV2Config, DeepseekV2ForCausalLM
        # (the group-limited V2 router of this transformers version reads an attribute it never sets; "greedy" is
        # the router of the published V2-Lite checkpoints)
        m = DeepseekV2ForCausalLM(DeepseekV2Config(topk_method="greedy", norm_topk_prob=False, **common))
    else:
        from transformers import DeepseekV3Config, DeepseekV3ForCausalLM
        m = DeepseekV3ForCausalLM(DeepseekV3Config(norm_topk_prob=True, **common))
    m = m.eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith("gate.weight"):
                p.mul_(20.0)                                     # spread the scores so that the selection is not a coin toss
            if n.endswith("e_score_correction_bias"):
                p.copy_(0.2 * torch.randn_like(p))
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(0.2 * torch.randn_like(b))
    d = str(tmp_path / f"dsmoe{version}")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.ffn_kinds == ["glu", "moe", "moe"] and cfg.shared_intermediate_size == 64
    assert cfg.router_groups == (1 if version == 2 else 4)
    assert w.layers[1].router_w is not None and w.layers[0].router_w is None
    assert (w.layers[1].router_select_b is not None) == (version == 3)
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=32, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (50,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    err = (got - want).abs().max(dim=1).values / float(want.abs().max())
    # bf16 rounding of the router scores can flip a near-tie for a single token; the rest must agree closely
    assert float(err.median()) < 1e-2 and int((err > 5e-2).sum()) <= 2, err


def test_group_limited_router_keeps_the_best_groups():
    """V2 group-limited routing: only experts of the `topk_group` groups with the highest best score can be chosen."""
    from fllm_b200.models.moe import route_deepseek
    cfg = ModelConfig(num_experts=8, experts_per_token=3, router_kind="deepseek_v2", router_groups=4, router_topk_groups=2,
                      router_scale=2.0, router_norm_topk=False)
    logits = torch.tensor([[5.0, 0.1, 0.2, 0.3, 4.0, 3.9, 3.0, 2.9]])       # groups (0,1) (2,3) (4,5) (6,7): best are 0 and 2
    ids, w = route_deepseek(cfg, logits, None)
    assert sorted(ids[0].tolist()) == [0, 4, 5]                             # expert 6 (3.0) loses to 5 although its group is third
    p = torch.softmax(logits, -1)[0]
    assert torch.allclose(w[0].sort().values, (2.0 * p[[0, 4, 5]]).sort().values)


@pytest.mark.parametrize("kinds,ssm", SYNTHETIC[:2])
def test_state_checkpoints_reuse_a_prompt_prefix(kinds, ssm):
    """With state checkpoints a second request that shares a prompt prefix starts behind the last block boundary whose
    state was kept, and generates what it generates without the cache; a preempted-and-recomputed run is covered by
    the same path."""
    cfg = _synthetic(kinds, ssm)
    g = torch.Generator().manual_seed(0)
    shared = torch.randint(0, 200, (70,), generator=g).tolist()
    p1, p2 = shared + [3, 4, 5], shared + [9, 8, 7, 6]
    sp = SamplingParams(max_tokens=6, temperature=0.0)

    def engine(gb):
        ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=256, max_model_len=256, num_kv_blocks=64, block_size=16,
                          state_cache_gb=gb)
        return LLMEngine(cfg, ec, device="cpu", seed=1)
    plain = engine(0.0)
    want = [plain.generate([p], sp)[0] for p in (p1, p2, p1)]
    eng = engine(0.25)
    assert eng.cfg.enable_prefix_caching and eng.scheduler.chunk_align == 16
    got1 = eng.generate([p1], sp)[0]
    assert eng.state_ckpt.stats["saved"] >= 1 and eng.state_ckpt.stats["restored"] == 0
    before = eng.stats.prefill_tokens
    got2 = eng.generate([p2], sp)[0]
    assert eng.state_ckpt.stats["restored"] == 1
    assert eng.stats.prefill_tokens - before <= len(p2) - 64            # the first four blocks were not computed again
    got3 = eng.generate([p1], sp)[0]                                      # the whole aligned prefix of p1 is there: 64 tokens reused
    assert [got1, got2, got3] == want
    assert len(eng.blocks.state_free) == eng.rstate.slots - 1


def test_qwen3_next_matches_transformers(tmp_path):
    """Gated delta rule layers + gated full attention (partial rotary, 1 + w norms) + routed experts with a gated shared
    expert, against `transformers` on a random tiny checkpoint."""
    from transformers import Qwen3NextConfig, Qwen3NextForCausalLM
    from fllm_b200.formats.loader import load_hf_checkpoint
    torch.manual_seed(0)
    hc = Qwen3NextConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=4, num_attention_heads=4,
                         num_key_value_heads=2, head_dim=32, linear_conv_kernel_dim=4, linear_key_head_dim=32, linear_value_head_dim=32,
                         linear_num_key_heads=2, linear_num_value_heads=4, moe_intermediate_size=32, shared_expert_intermediate_size=48,
                         num_experts_per_tok=2, num_experts=8, max_position_embeddings=256, mlp_only_layers=[0])
    m = Qwen3NextForCausalLM(hc).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("norm.weight", "layernorm.weight", "dt_bias")):
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith("mlp.gate.weight"):
                p.mul_(20.0)
    d = str(tmp_path / "q3n")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.layer_kinds == ["gated_delta"] * 3 + ["attention"] and cfg.ffn_kinds == ["glu", "moe", "moe", "moe"]
    assert cfg.rot_dim == 8 and cfg.attn_out_gate and w.layers[3].w_attn_gate is not None and w.layers[1].shared_gate_w is not None
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    err = (got - want).abs().max(dim=1).values / float(want.abs().max())
    assert float(err.median()) < 1e-2 and int((err > 5e-2).sum()) <= 2, err


@pytest.mark.parametrize("n,H,P,G,N,Q,fresh", [(300, 4, 16, 2, 16, 64, True), (129, 6, 8, 1, 32, 128, False), (64, 2, 8, 2, 16, 64, False)])
def test_mamba2_matrix_form_equals_the_walk(n, H, P, G, N, Q, fresh):
    """The chunked matrix form of the Mamba-2 recurrence (prefill path on a GPU) against the token walk: outputs and the
    final state, from zeros or from a carried state, with a ragged last chunk."""
    from fllm_b200.ops.recurrent import ssd_chunked
    from fllm_b200.ops.reference import RefOps
    torch.manual_seed(n)
    x, dt = torch.randn(n, H * P), torch.randn(n, H)
    Bm, Cm = torch.randn(n, G * N), torch.randn(n, G * N)
    A, D, dtb = -torch.exp(torch.randn(H) * 0.5), torch.randn(H), torch.randn(H) * 0.5 - 1
    st = torch.randn(2, H, P, N) * 0.5
    st_ref = st.clone()
    qs, ss = torch.tensor([0, n], dtype=torch.int32), torch.tensor([1], dtype=torch.int32)
    pos = torch.arange(0 if fresh else 5, (0 if fresh else 5) + n, dtype=torch.int32)
    y_ref = RefOps().mamba2_scan(x, dt, Bm, Cm, A, D, dtb, st_ref, qs, ss, pos, H, P, G, N, 0.001, 100.0)
    y, hf = ssd_chunked(x, dt, Bm, Cm, A, D, dtb, None if fresh else st[1], H, P, G, N, 0.001, 100.0, Q)
    assert float((y - y_ref).abs().max()) < 1e-4 * float(y_ref.abs().max())
    assert float((hf - st_ref[1]).abs().max()) < 1e-4 * float(st_ref[1].abs().max())


def _rwkv6_oracle(sd, cfg, ids):
    """RWKV-6 one token at a time in fp32 with the states in a dictionary (the published recurrence, state [head, key,
    value]), written without any of the engine's pieces."""
    import torch.nn.functional as F
    C, N, eps = cfg.hidden_size, cfg.ssm["head_dim"], cfg.rms_eps
    H = C // N
    ln = lambda x, n: F.layer_norm(x, (C,), sd[n + ".weight"], sd[n + ".bias"], eps)
    st, out = {}, []
    for tok in ids:
        x = sd["rwkv.embeddings.weight"][tok]
        for l in range(cfg.num_layers):
            p = f"rwkv.blocks.{l}."
            a = lambda n: sd[p + "attention." + n]
            if l == 0:
                x = ln(x, p + "pre_ln")
            h = ln(x, p + "ln1")
            xx = st.get(("a", l), torch.zeros(C)) - h
            st[("a", l)] = h
            xxx = h + xx * a("time_maa_x").reshape(-1)
            d = a("time_maa_w2").shape[1]
            lo = torch.tanh(xxx @ a("time_maa_w1")).reshape(5, 1, d)
            mix = torch.bmm(lo, a("time_maa_w2")).reshape(5, -1)
            xw, xk, xv, xr, xg = (h + xx * (a("time_maa_" + c).reshape(-1) + mix[j]) for j, c in enumerate("wkvrg"))
            r, k, v = a("receptance.weight") @ xr, a("key.weight") @ xk, a("value.weight") @ xv
            gate = F.silu(a("gate.weight") @ xg)
            w = a("time_decay").reshape(-1) + torch.tanh(xw @ a("time_decay_w1")) @ a("time_decay_w2")
            decay = torch.exp(-torch.exp(w)).view(H, N)
            S = st.get(("s", l), torch.zeros(H, N, N))
            kv = k.view(H, N, 1) * v.view(H, 1, N)
            y = torch.einsum("hk,hkv->hv", r.view(H, N), a("time_faaaa")[:, :, None] * kv + S).reshape(1, C)
            st[("s", l)] = kv + decay[:, :, None] * S
            y = F.group_norm(y, H, a("ln_x.weight"), a("ln_x.bias"), 1e-5 * cfg.ssm["head_size_divisor"] ** 2).reshape(-1)
            x = x + a("output.weight") @ (y * gate)
            h2 = ln(x, p + "ln2")
            xx = st.get(("f", l), torch.zeros(C)) - h2
            st[("f", l)] = h2
            f = lambda n: sd[p + "feed_forward." + n]
            kk = torch.relu(f("key.weight") @ (h2 + xx * f("time_maa_k").reshape(-1))) ** 2
            x = x + torch.sigmoid(f("receptance.weight") @ (h2 + xx * f("time_maa_r").reshape(-1))) * (f("value.weight") @ kk)
        out.append(sd["head.weight"] @ ln(x, "rwkv.ln_out"))
    return torch.stack(out)


def test_rwkv6_matches_token_by_token_recurrence(tmp_path):
    import json
    from fllm_b200.formats.loader import load_hf_checkpoint
    from fllm_b200.formats.safetensors_io import save_file
    from fllm_b200.models.rwkv import random_rwkv6_state_dict
    hf = {"model_type": "rwkv6", "architectures": ["Rwkv6ForCausalLM"], "hidden_size": 64, "num_hidden_layers": 3, "head_size": 16,
          "head_size_divisor": 8, "intermediate_size": 224, "layer_norm_epsilon": 1e-5, "vocab_size": 300, "time_mix_extra_dim": 8,
          "time_decay_extra_dim": 16}
    cfg = ModelConfig.from_hf_config(hf)
    sd = random_rwkv6_state_dict(cfg, seed=4)
    json.dump(hf, open(tmp_path / "config.json", "w"))
    save_file(sd, str(tmp_path / "model.safetensors"))
    cfg2, w, _ = load_hf_checkpoint(str(tmp_path), device="cpu", dtype=torch.float32)
    assert cfg2.arch == "rwkv6"
    eng = LLMEngine(cfg2, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (40,), generator=torch.Generator().manual_seed(2)).tolist()
    got = eng.token_logits(toks)
    want = _rwkv6_oracle(sd, cfg, toks)
    assert float((got - want).abs().max()) < 1e-3 * float(want.abs().max())


@pytest.mark.parametrize("moe", [False, True])
def test_qwen3_5_text_matches_transformers(tmp_path, moe):
    """Qwen3.5 (text): the Qwen3-Next layer kinds with the delta-rule projections stored apart (q | k | v, z, beta, a), dense
    or routed feed-forward layers."""
    import transformers as tf
    from fllm_b200.formats.loader import load_hf_checkpoint
    torch.manual_seed(0)
    common = dict(vocab_size=300, hidden_size=64, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                  linear_conv_kernel_dim=4, linear_key_head_dim=32, linear_value_head_dim=32, linear_num_key_heads=2, linear_num_value_heads=4,
                  max_position_embeddings=256, pad_token_id=0)
    if moe:
        m = tf.Qwen3_5MoeForCausalLM(tf.Qwen3_5MoeTextConfig(**common, moe_intermediate_size=32, shared_expert_intermediate_size=48,
                                                             num_experts_per_tok=2, num_experts=8))
    else:
        m = tf.Qwen3_5ForCausalLM(tf.Qwen3_5TextConfig(**common, intermediate_size=128))
    m = m.eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if n.endswith(("q_proj.weight", "k_proj.weight")):
                p.mul_(12.0)
            if "norm" in n or n.endswith("dt_bias"):
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith("mlp.gate.weight"):
                p.mul_(20.0)
    d = str(tmp_path / "q35")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.layer_kinds == ["gated_delta"] * 3 + ["attention"] and cfg.ffn_kinds == (["moe"] * 4 if moe else ["glu"] * 4)
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    err = (got - want).abs().max(dim=1).values / float(want.abs().max())
    assert float(err.median()) < (1e-2 if moe else 2e-3) and int((err > (5e-2 if moe else 1e-2)).sum()) <= (2 if moe else 0), err


@pytest.mark.parametrize("qk_norm", [False, True])
def test_glm4_moe_matches_transformers(tmp_path, qk_norm):
    """GLM-4.5: partial rotary attention with biases (and optional per-head QK-norm), a dense first layer, then routed experts with
    the sigmoid / selection-bias / group router and a shared expert."""
    import transformers as tf
    from fllm_b200.formats.loader import load_hf_checkpoint
    torch.manual_seed(0)
    m = tf.Glm4MoeForCausalLM(tf.Glm4MoeConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4,
                                               num_key_value_heads=2, head_dim=16, attention_bias=True, moe_intermediate_size=32,
                                               num_experts_per_tok=2, n_shared_experts=1, n_routed_experts=8, routed_scaling_factor=1.5,
                                               n_group=2, topk_group=1, first_k_dense_replace=1, use_qk_norm=qk_norm,
                                               max_position_embeddings=256, pad_token_id=0)).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith(("q_proj.weight", "k_proj.weight")):
                p.mul_(12.0)
            if n.endswith("gate.weight"):
                p.mul_(20.0)
            if n.endswith(".bias") and "norm" not in n:
                p.add_(0.05 * torch.randn_like(p))
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.copy_(0.2 * torch.randn_like(b))
    d = str(tmp_path / "glm45")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.ffn_kinds == ["glu", "moe", "moe"] and cfg.rot_dim == 8 and cfg.router_kind == "deepseek_v3" and cfg.qk_norm == qk_norm
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    err = (got - want).abs().max(dim=1).values / float(want.abs().max())
    assert float(err.median()) < 1e-2 and int((err > 5e-2).sum()) <= 2, err


def test_ernie4_5_moe_matches_transformers(tmp_path):
    """ERNIE 4.5 MoE: pair-style rotation, a dense first layer, softmax router whose selection adds a bias, weights renormalised,
    shared experts."""
    import transformers as tf
    from fllm_b200.formats.loader import load_hf_checkpoint
    torch.manual_seed(0)
    m = tf.Ernie4_5_MoeForCausalLM(tf.Ernie4_5_MoeConfig(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                                                         num_attention_heads=4, num_key_value_heads=2, moe_intermediate_size=32, moe_k=2,
                                                         moe_num_experts=8, moe_num_shared_experts=2, moe_layer_start_index=1,
                                                         max_position_embeddings=256)).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith(("q_proj.weight", "k_proj.weight")):
                p.mul_(12.0)
            if n.endswith("gate.weight"):
                p.mul_(20.0)
            if n.endswith("e_score_correction_bias"):
                p.copy_(0.05 * torch.randn_like(p))
    d = str(tmp_path / "ernie")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.ffn_kinds == ["glu", "moe", "moe"] and cfg.rope_style == "pair" and w.layers[1].router_select_b is not None
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    err = (got - want).abs().max(dim=1).values / float(want.abs().max())
    assert float(err.median()) < 1e-2 and int((err > 5e-2).sum()) <= 2, err


def _nemotron_h(latent, hidden=64, vocab=300):
    import transformers as tf
    torch.manual_seed(0)
    m = tf.NemotronHForCausalLM(tf.NemotronHConfig(
        vocab_size=vocab, hidden_size=hidden, layers_block_type=["mamba", "moe", "attention", "moe", "mamba"], num_attention_heads=4,
        num_key_value_heads=2, head_dim=hidden // 4, intermediate_size=2 * hidden, ssm_state_size=16, mamba_num_heads=8,
        mamba_head_dim=hidden // 4, n_groups=2, n_routed_experts=8, moe_intermediate_size=hidden // 2,
        moe_shared_expert_intermediate_size=hidden, num_experts_per_tok=2, moe_latent_size=latent, routed_scaling_factor=1.5)).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith(("q_proj.weight", "k_proj.weight")):
                p.mul_(12.0)
            if "experts." in n and p.dim() == 3:
                p.normal_(0, 0.2)
            if n.endswith("gate.weight"):
                p.normal_(0, 1.0)
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.normal_(0, 0.2)
    return m


@pytest.mark.parametrize("latent", [None, 32])
def test_nemotron_h_matches_transformers(tmp_path, latent):
    """Nemotron-H: one mixer per block (Mamba-2 with a grouped gated norm, attention without rotary embedding, a mixture of
    two-matrix relu^2 experts behind a sigmoid router with a selection bias, with and without the latent projection
    around the routed experts, a shared MLP on the hidden state)."""
    from fllm_b200.formats.loader import load_hf_checkpoint
    m = _nemotron_h(latent)
    d = str(tmp_path / "nemotron_h")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.layer_kinds == ["mamba2", "none", "attention", "none", "mamba2"] and cfg.ffn_kinds == ["none", "moe", "none", "moe", "none"]
    assert not cfg.use_rope and cfg.mlp_kind == "plain" and cfg.act == "relu2" and cfg.moe_latent_size == (latent or 0)
    assert (w.layers[1].moe_latent_in is not None) == bool(latent) and w.layers[1].exp_gate_up.shape[1] == 32
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    assert float((got - want).abs().max() / want.abs().max()) < 2e-3


def test_nemotron_h_pattern_string():
    """Older configs spell the blocks as a pattern string: M Mamba-2, * attention, - MLP, E experts."""
    from fllm_b200.config import ModelConfig
    cfg = ModelConfig.from_hf_config(dict(model_type="nemotron_h", vocab_size=300, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                                   hybrid_override_pattern="M-M*-", intermediate_size=128, mamba_num_heads=8, mamba_head_dim=16,
                                   ssm_state_size=16, n_groups=2))
    assert cfg.layer_kinds == ["mamba2", "none", "mamba2", "attention", "none"] and cfg.ffn_kinds == ["none", "glu", "none", "none", "glu"]
    assert cfg.num_experts == 0 and cfg.num_layers == 5 and cfg.has_recurrent


@pytest.mark.parametrize("norm,before,bias", [(False, True, False), (True, True, True), (True, False, False)])
def test_falcon_h1_matches_transformers(tmp_path, norm, before, bias):
    """Falcon-H1: Mamba-2 and attention read the same normed input and their outputs add; every mu-P multiplier (embeddings,
    head, the five sections of the mixer's input projection, its input and output, attention input / keys / output, the
    MLP's gate and output) is folded into the weights; the mixer's gate with no norm, norm then gate, gate then norm."""
    import transformers as tf
    from fllm_b200.formats.loader import load_hf_checkpoint
    torch.manual_seed(0)
    m = tf.FalconH1ForCausalLM(tf.FalconH1Config(
        vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
        mamba_d_ssm=96, mamba_n_heads=6, mamba_n_groups=2, mamba_d_state=16, mamba_rms_norm=norm, mamba_norm_before_gate=before,
        mamba_proj_bias=bias, attention_bias=bias, lm_head_multiplier=0.7, embedding_multiplier=2.5, mlp_multipliers=[0.8, 1.3],
        key_multiplier=1.7, attention_out_multiplier=0.9, attention_in_multiplier=1.2, ssm_multipliers=[0.9, 1.1, 1.2, 0.8, 1.3],
        ssm_in_multiplier=1.4, ssm_out_multiplier=0.6, max_position_embeddings=256)).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith(("q_proj.weight", "k_proj.weight")):
                p.mul_(12.0)
            if n.endswith("bias") and "conv" not in n and "dt_" not in n:
                p.normal_(0, 0.1)
    d = str(tmp_path / "falcon_h1")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    assert cfg.layer_kinds == ["attention+mamba2"] * 2 and cfg.has_recurrent and cfg.has_kv(1)
    assert cfg.ssm["gate_mode"] == ("gate_only" if not norm else "norm_before_gate" if before else "norm_after_gate")
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    assert float((got - want).abs().max() / want.abs().max()) < 2e-3
