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
    sf = torch.zeros(ops.k.mx_act_scale_bytes(T, K, 0), dtype=torch.uint8, device="cuda")
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


def test_nvfp4_activation_quantiser_matches_its_host_statement(ops):
    from fllm_b200.ops.mx import dequantize_act_nvfp4, quantize_act_nvfp4
    g = torch.Generator().manual_seed(3)
    T, K = 37, 768
    x = (torch.randn(T, K, generator=g) * torch.logspace(-2, 1.5, T).unsqueeze(1)).to(torch.bfloat16)
    x[4] = 0
    x[:, 256:272] = 0                                           # a block of zeros inside live tokens
    xq = torch.empty(T, K // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(ops.k.mx_act_scale_bytes(T, K, 2), dtype=torch.uint8, device="cuda")
    ts = torch.empty(T, dtype=torch.float32, device="cuda")
    ops.k.quant_nvfp4(x.cuda(), xq, sf, ts)
    c_ref, s_ref, t_ref = quantize_act_nvfp4(x)
    assert torch.allclose(ts.cpu(), t_ref, rtol=1e-6)
    bn = 64
    atoms = sf.cpu().view(-1, K // 64, 512)
    got_s = torch.empty(T, K // 16, dtype=torch.uint8)
    for t in range(T):
        r = t % bn
        for kb in range(K // 64):
            for j in range(4):
                got_s[t, kb * 4 + j] = atoms[t // bn, kb, (r % 32) * 16 + (r // 32) * 4 + j]
    assert (got_s != s_ref).float().mean().item() < 0.01       # a scale on a rounding boundary may differ by one ulp
    got = dequantize_act_nvfp4(xq.cpu(), got_s, ts.cpu())
    want = dequantize_act_nvfp4(c_ref, s_ref, t_ref)
    assert (got - want).abs().max().item() <= 0.26 * x.float().abs().max().item()
    assert ((got - want).abs() > 1e-6 * x.float().abs().max()).float().mean().item() < 0.01
    rel = (got - x.float()).norm() / x.float().norm()
    assert rel < 0.12, rel                                      # 4-bit values with a scale per 16


@pytest.mark.parametrize("T", [1, 16, 17, 64, 100, 128, 300])
@pytest.mark.parametrize("N,K", [(256, 512), (4096, 4096), (392, 1024), (1024, 12288)])
def test_linear_nvfp4_block_scaled_matches_fp32_math(ops, T, N, K):
    """NVFP4 x NVFP4 on kind::mxf4nvf4: the kernel's own activation codes, dequantised on the host, times the
    dequantised weights in fp32."""
    from fllm_b200.ops.mx import Nvfp4TcWeight, dequantize_act_nvfp4
    g = torch.Generator().manual_seed(T * 11 + N)
    w = torch.randn(N, K, generator=g) * 0.05
    w[:, : K // 2] *= 4.0
    x = (torch.randn(T, K, generator=g) * (1.0 + torch.arange(T).float().unsqueeze(1) % 5)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g).to(torch.bfloat16) if T % 2 == 0 else None
    q = Nvfp4TcWeight.from_dense(w).to("cuda")
    xq = torch.empty(T, K // 2, dtype=torch.uint8, device="cuda")
    sf = torch.zeros(ops.k.mx_act_scale_bytes(T, K, 2), dtype=torch.uint8, device="cuda")
    ts = torch.empty(T, dtype=torch.float32, device="cuda")
    ops.k.quant_nvfp4(x.cuda(), xq, sf, ts)
    bn = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
    atoms = sf.cpu().view(-1, K // 64, 512)
    tt = torch.arange(T)
    r = tt % bn
    off = ((r % 32) * 16 + (r // 32) * 4)
    s_rows = torch.stack([atoms[tt // bn, :, :].gather(2, (off.view(T, 1, 1) + j).expand(T, K // 64, 1)).squeeze(-1) for j in range(4)], -1)
    xd = dequantize_act_nvfp4(xq.cpu(), s_rows.reshape(T, K // 16), ts.cpu())
    want = xd @ q.dense().cpu().t()
    if bias is not None:
        want = want + bias.float()
    got = q.apply(ops, x.cuda(), bias.cuda() if bias is not None else None).float().cpu()
    assert ops.check_status() == 0
    err = (got - want).abs().max().item() / (want.abs().max().item() + 1e-9)
    assert err < 1e-2, err
    full = x.float() @ w.t()
    assert (got - (full + (bias.float() if bias is not None else 0))).norm() / full.norm() < 0.25


@pytest.mark.parametrize("fmt", ["int8", "fp8"])
@pytest.mark.parametrize("T", [1, 16, 33, 64, 128, 300])
@pytest.mark.parametrize("N,K", [(256, 512), (4096, 4096), (392, 1024), (1024, 12288)])
def test_linear_w8a8_row_scaled(ops, fmt, T, N, K):
    """int8 x int8 (kind::i8, int32 accumulators) and e4m3 x e4m3 with one scale per feature and per token against
    fp32 math on the same codes; the int8 product is exact up to the final rounding."""
    from fllm_b200.ops.mx import W8A8Weight, dequantize_rows_8bit, quantize_rows_8bit
    g = torch.Generator().manual_seed(T * 13 + N)
    w = torch.randn(N, K, generator=g) * 0.05 * (1.0 + torch.arange(N).float().unsqueeze(1) % 7)
    x = (torch.randn(T, K, generator=g) * (1.0 + torch.arange(T).float().unsqueeze(1) % 5)).to(torch.bfloat16)
    bias = torch.randn(N, generator=g).to(torch.bfloat16) if T % 2 == 0 else None
    q = W8A8Weight.from_dense(w, fmt)
    xq_ref, ts_ref = quantize_rows_8bit(x, fmt == "int8")
    want = dequantize_rows_8bit(xq_ref, ts_ref, fmt == "int8") @ q.dense().t()
    if bias is not None:
        want = want + bias.float()
    got = q.to("cuda").apply(ops, x.cuda(), bias.cuda() if bias is not None else None).float().cpu()
    assert ops.check_status() == 0
    err = (got - want).abs().max().item() / (want.abs().max().item() + 1e-9)
    assert err < 1e-2, err


@pytest.mark.parametrize("fmt", ["mxfp8", "mxfp4_a8", "nvfp4_a4", "int8_w8a8", "fp8_w8a8"])
def test_engine_runs_block_scaled_weight_formats(fmt):
    """qwen3-tiny with every projection in a block-scaled format: the GPU logits of a prompt against the PyTorch
    statement of the same arithmetic (same packed weights, same activation quantisation rule)."""
    from fllm_b200.config import EngineConfig, preset
    from fllm_b200.models.weights import init_random_weights
    from fllm_b200.ops.mx import MxWeight, Nvfp4TcWeight, W8A8Weight
    from fllm_b200.runtime import LLMEngine, SamplingParams
    from fllm_b200.ops.reference import RefOps
    cfg = preset("qwen3-tiny")
    w = init_random_weights(cfg, "cuda:0", seed=2, weight_format=fmt)
    kinds = (MxWeight, Nvfp4TcWeight, W8A8Weight)
    assert isinstance(w.layers[0].wqkv, kinds) and isinstance(w.layers[0].w_down, kinds)
    ec = EngineConfig(max_num_seqs=4, max_num_batched_tokens=64, max_model_len=256, num_kv_blocks=64, use_cuda_graphs=False)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (40,), generator=g).tolist()
    lg = []
    for ref in (True, False):
        eng = LLMEngine(cfg, ec, device="cuda:0", weights=w, **({"ops": RefOps()} if ref else {}))
        lg.append(eng.token_logits(prompt).float().cpu())
        if not ref:
            assert eng.ops.check_status() == 0
            out = eng.generate([prompt], SamplingParams(max_tokens=6))[0]     # decode steps (1 token) run the same kernels
            assert len(out) == 6
    # a value on a rounding boundary of the activation format moves a whole step (large for 4-bit activations), and
    # the step travels through the remaining layers: compare the logit rows as vectors
    err = ((lg[0] - lg[1]).norm() / lg[0].norm()).item()
    assert err < (0.06 if fmt != "nvfp4_a4" else 0.25), err
