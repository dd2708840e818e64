"""The audio tower on the GPU: sm_100a operators (tcgen05 GEMMs, bidirectional paged attention) against the PyTorch
operators on the same bf16 weights."""
import pytest
import torch

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def test_whisper_encoder_native_operators(tmp_path):
    from transformers import WhisperConfig, WhisperModel
    from fllm_b200.models.towers import Tower, load_hf_tower
    from fllm_b200.ops.native import NativeOps
    from fllm_b200.ops.reference import RefOps
    torch.manual_seed(0)
    hc = WhisperConfig(vocab_size=100, num_mel_bins=16, d_model=256, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=512,
                       decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=64, max_source_positions=100, max_target_positions=16,
                       pad_token_id=0, bos_token_id=1, eos_token_id=2, decoder_start_token_id=1)
    d = str(tmp_path / "whisper")
    WhisperModel(hc).eval().save_pretrained(d, safe_serialization=True)
    cfg, w = load_hf_tower(d, "cuda:0", torch.bfloat16)
    mel = torch.randn(3, 16, 200, device="cuda:0")
    nat = Tower(cfg, w, NativeOps(torch.device("cuda:0")), "cuda:0").forward(mel)
    ref = Tower(cfg, w, RefOps(), "cuda:0").forward(mel)
    assert nat.shape == (3, 100, 256)
    assert float((nat.float() - ref.float()).norm() / ref.float().norm()) < 2e-2
