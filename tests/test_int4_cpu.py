"""INT4 group-affine device form: nibble order, GGUF block decoders against the native codecs, CPU path."""
import numpy as np
import torch

from fllm_b200.formats import quant as Q
from fllm_b200.ops.int4 import Int4Weight, pack_codes, unpack_codes


def test_pack_order_and_round_trip():
    q = torch.arange(16, dtype=torch.uint8).view(1, 16) % 16
    codes = pack_codes(q)
    # word 0 holds values 0..7 as nibbles [v0 v2 v4 v6 v1 v3 v5 v7] (low nibble first)
    w = int.from_bytes(bytes(codes[0, :4].tolist()), "little")
    assert [(w >> (4 * j)) & 0xF for j in range(8)] == [0, 2, 4, 6, 1, 3, 5, 7]
    for j in range(4):          # what the kernel extracts: pair (2j, 2j+1)
        pair = (w >> (4 * j)) & 0x000F000F
        assert (pair & 0xF, pair >> 16) == (2 * j, 2 * j + 1)
    r = torch.randint(0, 16, (5, 64), dtype=torch.uint8)
    assert torch.equal(unpack_codes(pack_codes(r)), r)


def _check_gguf(name, qtype, tol):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((6, 512)) * 0.1).astype(np.float32)
    raw = Q.quantize(w, qtype)
    want = Q.dequantize(raw, qtype, 6, 512)
    got = Int4Weight.from_gguf(name, raw, 6, 512).dense().numpy()
    # scale and min are held as bf16 on the device: 2^-8 relative on each term
    scale = np.abs(want).max()
    assert np.abs(got - want).max() <= tol * scale, np.abs(got - want).max() / scale


def test_q4_k_blocks_decode_like_the_native_codec():
    _check_gguf("Q4_K", Q.Q4_K, 1.5e-2)


def test_q4_0_blocks_decode_like_the_native_codec():
    _check_gguf("Q4_0", Q.Q4_0, 1.5e-2)


def test_from_dense_and_cpu_apply():
    from fllm_b200.ops.reference import RefOps
    torch.manual_seed(0)
    w = torch.randn(48, 128) * 0.05
    q = Int4Weight.from_dense(w)
    assert q.codes.shape == (48, 64) and q.sm.shape == (48, 4, 2)
    assert ((q.dense() - w).norm() / w.norm()).item() < 0.08
    q128 = Int4Weight.from_dense(w, group=128)       # AWQ / GPTQ group size: replicated per 32 on the device
    assert q128.sm.shape == (48, 4, 2) and ((q128.dense() - w).norm() / w.norm()).item() < 0.12
    x = torch.randn(3, 128).to(torch.bfloat16)
    y = RefOps().linear(x, q)
    ref = x.float() @ w.t()
    assert ((y.float() - ref).norm() / ref.norm()).item() < 0.1
