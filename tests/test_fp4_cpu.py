"""FP4 codecs (NVFP4 / MXFP4) and the packed-weight object on the CPU oracle path."""
import torch

from fllm_b200.ops.fp4 import (MXFP4, NVFP4, Fp4Weight, _e2m1_codes, dequantize_fp4, quantize_decoder_weights,
                               quantize_mxfp4, quantize_nvfp4)


def test_e2m1_rounding_ties_to_even_code():
    x = torch.tensor([0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 7.0, -0.25, -2.5, -6.0, 0.3, 2.4, 2.6])
    got = _e2m1_codes(x).tolist()
    #        0  .25->0  .75->1.0  1.25->1.0  1.75->2.0  2.5->2.0  3.5->4.0  5->4.0  7->6  -.25->-0  -2.5->-2  -6  .3->.5  2.4->2  2.6->3
    assert got == [0, 0, 2, 2, 4, 4, 6, 6, 7, 8, 12, 15, 1, 4, 5]


def test_nvfp4_round_trip_error():
    torch.manual_seed(0)
    w = torch.randn(64, 256) * 0.1
    c, s, a = quantize_nvfp4(w)
    assert c.shape == (64, 128) and s.shape == (64, 16) and c.dtype == torch.uint8
    d = dequantize_fp4(c, s, NVFP4, a)
    rel = ((d - w).norm() / w.norm()).item()
    assert rel < 0.12, rel
    # block maxima survive within the e4m3 scale's precision
    bm_w = w.view(64, 16, 16).abs().amax(-1)
    bm_d = d.view(64, 16, 16).abs().amax(-1)
    assert torch.allclose(bm_w, bm_d, rtol=0.07, atol=1e-6)


def test_mxfp4_round_trip_error_and_power_of_two_scales():
    torch.manual_seed(1)
    w = torch.randn(32, 128) * 3.0
    c, s, a = quantize_mxfp4(w)
    assert a == 1.0 and s.shape == (32, 4)
    d = dequantize_fp4(c, s, MXFP4)
    assert ((d - w).norm() / w.norm()).item() < 0.16
    assert d.abs().max() <= 6.0 * torch.exp2(s.float().max() - 127)


def test_fp4_weight_apply_and_model_quantisation_on_cpu():
    from fllm_b200.config import preset
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.ops.reference import RefOps
    torch.manual_seed(2)
    w = (torch.randn(96, 128) * 0.05).to(torch.bfloat16)
    x = torch.randn(5, 128).to(torch.bfloat16)
    q = Fp4Weight.from_dense(w, "mxfp4")
    y = RefOps().linear(x, q)
    assert y.shape == (5, 96)
    ref = x.float() @ w.float().t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 0.2
    cfg = preset("qwen3-tiny")
    weights = init_random_weights(cfg, device="cpu")
    dense_bytes = sum(getattr(lw, n).numel() * 2 for lw in weights.layers for n in ("wqkv", "wo", "w_gate_up", "w_down"))
    packed = quantize_decoder_weights(weights, "nvfp4")
    assert 0 < packed < dense_bytes * 0.3
