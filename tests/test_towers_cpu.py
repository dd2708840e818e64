"""Vision and audio towers against Hugging Face `transformers` on random tiny checkpoints: the SigLIP vision transformer
(last hidden state) and the Whisper encoder."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def test_siglip_vision_tower_matches_transformers(tmp_path):
    from transformers import SiglipVisionConfig, SiglipVisionModel
    from fllm_b200.models.towers import Tower, load_hf_tower
    from fllm_b200.ops.reference import RefOps
    torch.manual_seed(0)
    hc = SiglipVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=32, patch_size=8)
    m = SiglipVisionModel(hc).eval().float()
    d = str(tmp_path / "siglip")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w = load_hf_tower(d, "cpu", torch.float32)
    assert cfg.kind == "siglip" and w.pos.shape[0] == 16 and cfg.act == "gelu_tanh"
    tower = Tower(cfg, w, RefOps(), "cpu")
    assert not tower.kernel_attention                              # head width 16: PyTorch attention
    px = torch.randn(3, 3, 32, 32)
    with torch.no_grad():
        want = m(pixel_values=px).last_hidden_state
    got = tower.forward(px)
    assert got.shape == want.shape and float((got - want).abs().max()) < 1e-4
    with pytest.raises(ValueError):
        tower.forward(torch.randn(1, 3, 40, 40))


def test_whisper_encoder_matches_transformers(tmp_path):
    from transformers import WhisperConfig, WhisperModel
    from fllm_b200.models.towers import Tower, load_hf_tower
    from fllm_b200.ops.reference import RefOps
    torch.manual_seed(0)
    hc = WhisperConfig(vocab_size=100, num_mel_bins=16, d_model=128, encoder_layers=2, encoder_attention_heads=2, encoder_ffn_dim=256,
                       decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=64, max_source_positions=40, max_target_positions=16, pad_token_id=0, bos_token_id=1,
                       eos_token_id=2, decoder_start_token_id=1)
    m = WhisperModel(hc).eval().float()
    d = str(tmp_path / "whisper")
    m.save_pretrained(d, safe_serialization=True)
    cfg, w = load_hf_tower(d, "cpu", torch.float32)
    assert cfg.kind == "whisper" and cfg.head_dim == 64
    tower = Tower(cfg, w, RefOps(), "cpu")
    assert tower.kernel_attention                                  # head width 64: the paged bidirectional attention path
    mel = torch.randn(2, 16, 80)
    with torch.no_grad():
        want = m.encoder(mel).last_hidden_state
    got = tower.forward(mel)
    # the scratch KV pool keeps the activation type (fp32 here), so nothing is rounded on this path
    assert got.shape == want.shape and float((got - want).abs().max()) < 1e-4
