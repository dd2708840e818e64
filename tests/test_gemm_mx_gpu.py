"""Block-scaled MX GEMM (tcgen05 kind::mxf8f6f4.block_scale) against fp32 PyTorch math on the same quantised
operands: MXFP8 and packed MXFP4 weights, every token tile, ragged edges, split K, bias."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from fllm_b200.ops import get_ops
    return get_ops("cuda")


def test_activation_quantiser_matches_its_host_statement(ops):
    from fllm_b200.ops.mx import e8m0_to_float, quantize_mxfp8
    g = torch.Generator().manual_seed(0)
    T, K = 70, 512
    x = (torch.randn(T, K, generator=g) * torch.logspace(-3, 2, T).unsqueeze(1)).to(torch.bfloat16)
    x[3] = 0
    x[5, :32] = 448.0                                            # lands exactly on a power-of-two boundary
    xq = torch.empty(T, K, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(ops.k.mx_act_scale_bytes(T, K), dtype=torch.uint8, device="cuda")
    ops.k.quant_mx(x.cuda(), xq, sf)
    q_ref, s_ref = quantize_mxfp8(x)
    bn = 128
    atoms = sf.cpu().view(-1, K // 128, 512)
    got_s = torch.empty(T, K // 32, dtype=torch.uint8)
    for t in range(T):
        r = t % bn
        for kb in range(K // 128):
            for j in range(4):
                got_s[t, kb * 4 + j] = atoms[t // bn, kb, (r % 32) * 16 + (r // 32) * 4 + j]
    assert torch.equal(got_s, s_ref)
    got = xq.cpu().view(torch.float8_e4m3fn).float()
    want = q_ref.view(torch.float8_e4m3fn).float()
    assert torch.equal(got, want)
    assert torch.isfinite(got * e8m0_to_float(got_s).repeat_interleave(32, 1)).all()


@pytest.mark.parametrize("fmt", ["mxfp8", "mxfp4"])
@pytest.mark.parametrize("T", [1, 16, 17, 64, 100, 128, 300])
@pytest.mark.parametrize("N,K", [(256, 512), (4096, 4096), (392, 1024), (1024, 12288)])
def test_linear_mx_matches_fp32_math(ops, fmt, T, N, K):
    from fllm_b200.ops.mx import MxWeight, quantize_act_reference
    g = torch.Generator().manual_seed(T * 7 + N)
    w = torch.randn(N, K, generator=g) * 0.05
    w[:, : K // 2] *= 8.0                                        # scales differ along K
    x = (torch.randn(T, K, generator=g) * (1.0 + torch.arange(T).float().unsqueeze(1) % 5)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g).to(torch.bfloat16) if T % 2 == 0 else None
    mw = MxWeight.from_dense(w, fmt)
    want = quantize_act_reference(x) @ mw.dense().t()
    if bias is not None:
        want = want + bias.float()
    got = mw.to("cuda").apply(ops, x.cuda(), bias.cuda() if bias is not None else None).float().cpu()
    assert ops.check_status() == 0
    err = (got - want).abs().max().item() / (want.abs().max().item() + 1e-9)
    assert err < 1e-2, err
