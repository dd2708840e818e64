"""The attention families against Hugging Face `transformers` itself: a random tiny model of each type is saved, read by
the loader and run through the engine (fp32 weights, chunked prefill); teacher-forced logits must agree with the
`transformers` forward pass (the KV pool is fp32 here too; the projections that feed the attention scores are scaled up so
that a wrong rotation, mask or window moves the logits)."""
import pytest
import torch

transformers = pytest.importorskip("transformers")

from fllm_b200.config import EngineConfig
from fllm_b200.runtime.engine import LLMEngine

BASE = dict(vocab_size=300, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
            max_position_embeddings=256)


def _model(kind):
    import transformers as tf
    torch.manual_seed(0)
    if kind == "llama":
        return tf.LlamaForCausalLM(tf.LlamaConfig(**BASE))
    if kind == "llama3_rope":
        return tf.LlamaForCausalLM(tf.LlamaConfig(**BASE, rope_parameters=dict(rope_type="llama3", rope_theta=10000.0, factor=8.0,
                                                  low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=32)))
    if kind == "mistral":
        return tf.MistralForCausalLM(tf.MistralConfig(**BASE, sliding_window=24))
    if kind == "qwen2":
        return tf.Qwen2ForCausalLM(tf.Qwen2Config(**BASE))
    if kind == "qwen3":
        return tf.Qwen3ForCausalLM(tf.Qwen3Config(**BASE, head_dim=32))
    if kind == "gemma":
        return tf.GemmaForCausalLM(tf.GemmaConfig(**BASE, head_dim=16))
    if kind == "gemma2":
        return tf.Gemma2ForCausalLM(tf.Gemma2Config(**BASE, head_dim=16, sliding_window=24, query_pre_attn_scalar=20,
                                                    final_logit_softcapping=20.0, attn_logit_softcapping=30.0,
                                                    attn_implementation="eager"))      # the fused attention path of the library drops the soft-cap
    if kind == "gemma3":
        return tf.Gemma3ForCausalLM(tf.Gemma3TextConfig(**BASE, head_dim=16, sliding_window=24, query_pre_attn_scalar=20,
                                                        layer_types=["sliding_attention", "full_attention"],
                                                        rope_parameters=dict(full_attention=dict(rope_type="linear", factor=4.0, rope_theta=100000.0),
                                                                             sliding_attention=dict(rope_type="default", rope_theta=5000.0))))
    if kind == "granite":
        return tf.GraniteForCausalLM(tf.GraniteConfig(**BASE, embedding_multiplier=3.0, logits_scaling=2.0, residual_multiplier=0.5,
                                                      attention_multiplier=0.2, tie_word_embeddings=True))
    if kind == "seed_oss":
        return tf.SeedOssForCausalLM(tf.SeedOssConfig(**BASE, head_dim=16, pad_token_id=0))
    if kind == "ernie4_5":
        return tf.Ernie4_5ForCausalLM(tf.Ernie4_5Config(**BASE, pad_token_id=0))
    if kind == "glm":
        return tf.GlmForCausalLM(tf.GlmConfig(**BASE, head_dim=16, pad_token_id=0))
    if kind == "glm4":
        return tf.Glm4ForCausalLM(tf.Glm4Config(**BASE, head_dim=16, pad_token_id=0))
    if kind == "helium":
        return tf.HeliumForCausalLM(tf.HeliumConfig(**BASE, head_dim=16, pad_token_id=0))
    if kind == "ministral":
        return tf.MinistralForCausalLM(tf.MinistralConfig(**BASE, head_dim=16, pad_token_id=0, sliding_window=24))
    if kind == "smollm3":
        return tf.SmolLM3ForCausalLM(tf.SmolLM3Config(**BASE, pad_token_id=0, no_rope_layers=[1, 0]))
    if kind == "starcoder2":
        return tf.Starcoder2ForCausalLM(tf.Starcoder2Config(**BASE, sliding_window=24))
    if kind == "stablelm":
        return tf.StableLmForCausalLM(tf.StableLmConfig(**BASE, use_qkv_bias=True))
    if kind == "nemotron":
        return tf.NemotronForCausalLM(tf.NemotronConfig(**BASE, head_dim=16))
    if kind == "arcee":
        return tf.ArceeForCausalLM(tf.ArceeConfig(**BASE, head_dim=16))
    if kind == "phi":
        return tf.PhiForCausalLM(tf.PhiConfig(**BASE))
    if kind == "gpt_neox":
        neox = {k: v for k, v in BASE.items() if k != "num_key_value_heads"}
        return tf.GPTNeoXForCausalLM(tf.GPTNeoXConfig(**neox))
    if kind == "cohere":
        return tf.CohereForCausalLM(tf.CohereConfig(**BASE, pad_token_id=0, logit_scale=0.25))
    if kind == "gpt2":
        return tf.GPT2LMHeadModel(tf.GPT2Config(vocab_size=300, n_positions=256, n_embd=64, n_layer=2, n_head=4))
    if kind == "opt":
        return tf.OPTForCausalLM(tf.OPTConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, ffn_dim=128, num_attention_heads=4,
                                               max_position_embeddings=256, word_embed_proj_dim=64))
    if kind == "olmo2":
        return tf.Olmo2ForCausalLM(tf.Olmo2Config(**BASE, pad_token_id=0))
    if kind == "olmo3":
        return tf.Olmo3ForCausalLM(tf.Olmo3Config(**BASE, pad_token_id=0, sliding_window=24, layer_types=["sliding_attention", "full_attention"]))
    if kind == "phi3":
        return tf.Phi3ForCausalLM(tf.Phi3Config(**BASE, pad_token_id=0))
    if kind == "mixtral":
        return tf.MixtralForCausalLM(tf.MixtralConfig(**BASE, num_local_experts=4, num_experts_per_tok=2))
    if kind == "qwen3_moe":
        return tf.Qwen3MoeForCausalLM(tf.Qwen3MoeConfig(**BASE, head_dim=32, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
                                                         norm_topk_prob=True))
    if kind == "qwen3_moe_raw_weights":         # the selected probabilities are not renormalised (the config's default)
        return tf.Qwen3MoeForCausalLM(tf.Qwen3MoeConfig(**BASE, head_dim=32, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=48,
                                                         norm_topk_prob=False))
    if kind == "gpt_oss":                       # YaRN with fractional correction dimensions, sinks, windowed layers, clamped GLU
        return tf.GptOssForCausalLM(tf.GptOssConfig(**BASE, head_dim=16, num_local_experts=4, num_experts_per_tok=2, sliding_window=24))
    if kind == "olmo":                          # LayerNorm without weights, clamped q / k / v
        return tf.OlmoForCausalLM(tf.OlmoConfig(**BASE, pad_token_id=0, clip_qkv=1.5))
    if kind == "olmoe":                         # full-width QK-norm then the clamp, raw softmax weights for the selected experts
        return tf.OlmoeForCausalLM(tf.OlmoeConfig(**BASE, pad_token_id=0, num_experts=8, num_experts_per_tok=2, clip_qkv=4.0))
    if kind == "cohere2":                       # windowed layers rotate, global layers carry no position signal
        return tf.Cohere2ForCausalLM(tf.Cohere2Config(**BASE, pad_token_id=0, logit_scale=0.25, sliding_window=24,
                                                      layer_types=["sliding_attention", "full_attention"]))
    if kind == "exaone4":
        return tf.Exaone4ForCausalLM(tf.Exaone4Config(**BASE, pad_token_id=0, sliding_window=24, sliding_window_pattern=2,
                                                      layer_types=["sliding_attention", "full_attention"]))
    if kind == "vaultgemma":
        return tf.VaultGemmaForCausalLM(tf.VaultGemmaConfig(**BASE, head_dim=16, sliding_window=24, query_pre_attn_scalar=20,
                                                            final_logit_softcapping=20.0, attn_logit_softcapping=30.0,
                                                            attn_implementation="eager"))
    if kind == "gpt_bigcode":                   # GPT-2 blocks with one key / value head
        return tf.GPTBigCodeForCausalLM(tf.GPTBigCodeConfig(vocab_size=300, n_positions=256, n_embd=64, n_layer=2, n_head=4))
    if kind.startswith("falcon"):               # the three layouts of the fused q|k|v rows, one or two norms, parallel or sequential blocks
        kw = {"falcon_new": dict(new_decoder_architecture=True, num_kv_heads=2),
              "falcon_new_one_norm": dict(new_decoder_architecture=True, num_kv_heads=2, num_ln_in_parallel_attn=1),
              "falcon_mq": dict(multi_query=True, parallel_attn=True),
              "falcon_mha_sequential": dict(multi_query=False, parallel_attn=False, bias=True)}[kind]
        return tf.FalconForCausalLM(tf.FalconConfig(vocab_size=300, hidden_size=64, num_hidden_layers=2, num_attention_heads=4, alibi=False,
                                                    max_position_embeddings=256, **kw))
    if kind == "minimax_m2":                    # full-width QK-norm, half of each head rotated, sigmoid router with a selection bias
        return tf.MiniMaxM2ForCausalLM(tf.MiniMaxM2Config(**dict(BASE, intermediate_size=32), head_dim=16, num_local_experts=8, num_experts_per_tok=2,
                                                          rope_parameters=dict(rope_type="default", rope_theta=10000.0, partial_rotary_factor=0.5)))
    if kind == "glm4_moe_lite":                 # DeepSeek-V3's tensors under another model type (as Kimi-K2 is)
        return tf.Glm4MoeLiteForCausalLM(tf.Glm4MoeLiteConfig(**dict(BASE, num_key_value_heads=4), moe_intermediate_size=32, n_routed_experts=8,
                                                              num_experts_per_tok=2, q_lora_rank=24, kv_lora_rank=32, qk_nope_head_dim=16,
                                                              qk_rope_head_dim=8, v_head_dim=16, first_k_dense_replace=1, n_group=2, topk_group=1))
    if kind == "cwm":                           # Llama with windowed and global layers
        return tf.CwmForCausalLM(tf.CwmConfig(**BASE, pad_token_id=0, sliding_window=24, layer_types=["sliding_attention", "full_attention"]))
    if kind == "jais2":                         # Llama blocks with LayerNorm and a squared-ReLU two-matrix MLP, biases everywhere
        return tf.Jais2ForCausalLM(tf.Jais2Config(**BASE, pad_token_id=0))
    if kind == "youtu":                         # latent attention in front of a dense FFN
        return tf.YoutuForCausalLM(tf.YoutuConfig(**dict(BASE, num_key_value_heads=4), pad_token_id=0, q_lora_rank=24, kv_lora_rank=32,
                                                  qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16))
    if kind == "qwen2_moe":
        return tf.Qwen2MoeForCausalLM(tf.Qwen2MoeConfig(**BASE, num_experts=4, num_experts_per_tok=2, moe_intermediate_size=48,
                                                         shared_expert_intermediate_size=64, norm_topk_prob=False))
    raise ValueError(kind)


@pytest.mark.parametrize("kind", ["llama", "llama3_rope", "mistral", "qwen2", "qwen3", "gemma", "gemma2", "gemma3", "granite", "seed_oss", "ernie4_5", "glm", "glm4", "helium",
                                  "ministral", "smollm3", "starcoder2", "stablelm", "nemotron", "arcee", "phi", "gpt_neox", "cohere", "gpt2", "opt", "olmo2", "olmo3", "phi3", "mixtral", "qwen3_moe",
                                  "qwen2_moe", "qwen3_moe_raw_weights", "gpt_oss", "olmo", "olmoe", "cohere2", "exaone4", "vaultgemma", "gpt_bigcode",
                                  "falcon_new", "falcon_new_one_norm", "falcon_mq", "falcon_mha_sequential", "minimax_m2", "glm4_moe_lite", "cwm", "jais2", "youtu"])
def test_attention_families_match_transformers(tmp_path, kind):
    from fllm_b200.formats.loader import load_hf_checkpoint
    m = _model(kind).eval().float()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "norm" in n:
                p.add_(0.3 * torch.randn_like(p))
            if n.endswith(".bias") and "norm" not in n:
                p.add_(0.05 * torch.randn_like(p))            # biases start at zero: make them count
            if n.endswith(("mlp.gate.weight", "block_sparse_moe.gate.weight")):
                p.mul_(20.0)                                  # clear routing decisions
            if n.endswith("q_b_proj.weight"):
                p.mul_(12.0)
            if n.endswith("sinks"):
                p.normal_(0, 1.0)
            if "experts" in n and p.dim() == 3:
                p.mul_(5.0)                                   # the routed share of the output is large enough to show its weights
            if n.endswith(("q_proj.weight", "k_proj.weight", "qkv_proj.weight", "query_key_value.weight", "c_attn.weight")):
                p.mul_(6.0 if kind.startswith("falcon") else 12.0)                                  # peaked attention: a wrong rotation or mask moves the logits
    d = str(tmp_path / kind)
    with torch.no_grad():
        for n, b in m.named_buffers():
            if n.endswith("e_score_correction_bias"):
                b.normal_(0, 0.2)
    m.save_pretrained(d, safe_serialization=True)
    cfg, w, _ = load_hf_checkpoint(d, device="cpu", dtype=torch.float32)
    eng = LLMEngine(cfg, EngineConfig(max_num_seqs=2, max_num_batched_tokens=16, max_model_len=128, num_kv_blocks=32, block_size=16,
                                      kv_cache_dtype="fp32"), device="cpu", weights=w)
    toks = torch.randint(0, 300, (45,), generator=torch.Generator().manual_seed(1)).tolist()
    got = eng.token_logits(toks)
    with torch.no_grad():
        want = m(torch.tensor([toks])).logits[0].float()
    err = (got - want).abs().max(dim=1).values / float(want.abs().max())
    assert float(err.max()) < 2e-3, err                # fp32 end to end (KV pool and routed experts included)


def test_unknown_families_are_refused():
    """A model type without a mapping must not run as if it were a Llama."""
    from fllm_b200.config import ModelConfig
    with pytest.raises(ValueError, match="not among the families"):
        ModelConfig.from_hf_config(dict(model_type="bloom", vocab_size=10, hidden_size=8, num_hidden_layers=1, num_attention_heads=1))
