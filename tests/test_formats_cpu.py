"""GGUF round trip, packed codecs and the CPU engine on the synthetic tiny-Llama Q4_K file."""
import os

import numpy as np
import pytest
import torch

from fllm_b200.formats import quant
from fllm_b200.formats.gguf import GgufError, GgufReader, GgufWriter, TYPE_ID


@pytest.mark.parametrize("qt,tol", [(quant.Q4_K, 0.09), (quant.Q5_K, 0.05), (quant.Q6_K, 0.025), (quant.Q8_0, 0.006),
                                    (quant.Q4_0, 0.12), (quant.MXFP4, 0.2), (quant.NVFP4, 0.15),
                                    (quant.BF16, 0.005), (quant.F16, 0.001), (quant.FP8_E4M3, 0.04)])
def test_codec_round_trip_error(qt, tol):
    rng = np.random.default_rng(0)
    x = rng.standard_normal((7, 512), dtype=np.float32) * 0.02
    y = quant.dequantize(quant.quantize(x, qt), qt, 7, 512)
    rel = np.linalg.norm(x - y) / np.linalg.norm(x)
    assert rel < tol, rel


def test_q4k_layout_matches_spec():
    """One hand-built block: d=1, dmin=0, scales all 1 -> values equal the 4-bit codes."""
    blk = bytearray(144)
    blk[0:2] = np.float16(1.0).tobytes()
    blk[2:4] = np.float16(0.0).tobytes()
    sc = [1] * 8
    mn = [0] * 8
    packed = bytearray(12)
    for j in range(4):
        packed[j] = sc[j]
        packed[j + 4] = mn[j]
    for j in range(4, 8):
        packed[j + 4] = (sc[j] & 0xF) | ((mn[j] & 0xF) << 4)
    blk[4:16] = packed
    codes = np.arange(256) % 16
    for j in range(4):
        for l in range(32):
            blk[16 + 32 * j + l] = int(codes[64 * j + l]) | (int(codes[64 * j + 32 + l]) << 4)
    y = quant.dequantize(np.frombuffer(bytes(blk), dtype=np.uint8), quant.Q4_K, 1, 256)
    assert np.array_equal(y[0], codes.astype(np.float32))


def test_e4m3_and_e2m1_are_exact_on_representable_values():
    vals = np.array([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -6.0, 448.0, -448.0, 0.015625, 2.0 ** -9, 240.0, 1.75]],
                    dtype=np.float32)
    y = quant.dequantize(quant.quantize(vals, quant.FP8_E4M3), quant.FP8_E4M3, 1, 16)
    assert np.array_equal(y, vals)


def test_gguf_round_trip(tmp_path):
    p = str(tmp_path / "t.gguf")
    w = GgufWriter(p)
    w.add("general.architecture", "llama")
    w.add("llama.block_count", 2)
    w.add("x.f", 1.5)
    w.add("x.s", ["a", "bc"])
    w.add("x.arr", np.arange(5, dtype=np.int32))
    a = np.random.default_rng(1).standard_normal((4, 256), dtype=np.float32)
    w.add_tensor("a.weight", (4, 256), TYPE_ID["Q4_K"], quant.quantize(a, quant.Q4_K))
    w.add_tensor("b", (3,), TYPE_ID["F32"], np.array([1, 2, 3], dtype=np.float32))
    w.write()
    r = GgufReader(p)
    assert r.metadata["llama.block_count"] == 2 and r.metadata["x.s"] == ["a", "bc"]
    assert list(r.metadata["x.arr"]) == [0, 1, 2, 3, 4]
    assert r.tensors["a.weight"].shape == (4, 256) and r.tensors["a.weight"].type_name == "Q4_K"
    assert np.array_equal(r.tensor_bytes("a.weight"), quant.quantize(a, quant.Q4_K).reshape(-1))
    assert np.allclose(r.tensor_f32("b"), [1, 2, 3])
    for t in r.tensors.values():
        assert t.offset % 32 == 0


def test_gguf_rejects_garbage(tmp_path):
    p = tmp_path / "bad.gguf"
    p.write_bytes(b"GGUF" + b"\x03\0\0\0" + b"\xff" * 40)
    with pytest.raises(GgufError):
        GgufReader(str(p))
    p.write_bytes(b"NOPE")
    with pytest.raises(GgufError):
        GgufReader(str(p))


def test_cpu_engine_tiny_llama(tmp_path):
    """The Q4_K CPU engine is bit-stable and agrees with a float decoder on dequantised weights."""
    from fllm_b200.config import preset
    from fllm_b200.cpu_engine import CpuEngine, write_tiny_llama_gguf
    cfg = preset("tiny-llama")
    cfg.vocab_size = 2048
    path = str(tmp_path / "tiny.gguf")
    write_tiny_llama_gguf(path, cfg, seed=0)
    eng = CpuEngine(path)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, cfg.vocab_size, 40).tolist()
    a = eng.generate(prompt, 16)
    b = eng.generate(prompt, 16)
    assert a == b and len(a) == 16
    # logits vs a dense float forward over the dequantised tensors
    from fllm_b200.models.weights import DecoderWeights, LayerWeights
    from oracle import dense_forward
    r = eng.reader
    f = lambda n: torch.from_numpy(r.tensor_f32(n).copy())
    layers = []
    for l in range(cfg.num_layers):
        pre = f"blk.{l}."
        layers.append(LayerWeights(
            attn_norm=f(pre + "attn_norm.weight"),
            wqkv=torch.cat([f(pre + "attn_q.weight"), f(pre + "attn_k.weight"), f(pre + "attn_v.weight")], 0),
            wo=f(pre + "attn_output.weight"), ffn_norm=f(pre + "ffn_norm.weight"),
            w_gate_up=torch.cat([f(pre + "ffn_gate.weight"), f(pre + "ffn_up.weight")], 0),
            w_down=f(pre + "ffn_down.weight")))
    emb = f("token_embd.weight")
    w = DecoderWeights(embed=emb, layers=layers, final_norm=f("output_norm.weight"), lm_head=emb)
    want = dense_forward(cfg, w, prompt, round_bf16=False)[-1].numpy()
    got = eng.logits(prompt)
    err = np.abs(got - want).max()
    assert err < 0.05 * np.abs(want).max() + 1e-3, err
    eng.close()
