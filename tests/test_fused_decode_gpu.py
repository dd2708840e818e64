"""The decode-step fusions against the unfused kernels and the PyTorch fp32 reference:
split-K partials consumed by the norm / rope / activation kernels, the gated activation inside
the GEMM epilogue (both orientations, both row layouts), the multi-CTA argmax."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from fllm_b200.ops.native import NativeOps
    return NativeOps(torch.device("cuda:0"))


@pytest.fixture(scope="module")
def ref():
    from fllm_b200.ops.reference import RefOps
    return RefOps()


def _rand(shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda") * scale).to(dtype)


def _close(y, r, tol=2e-2):
    err = (y.float() - r.float()).abs().max().item()
    scale = r.float().abs().max().item() + 1e-6
    assert err <= tol * scale, f"max abs err {err} vs scale {scale}"


def _block16(w):
    """gate half | up half -> blocks of 16 gate rows followed by the 16 up rows of the same features."""
    I = w.shape[0] // 2
    rest = w.shape[1:]
    return torch.stack([w[:I].reshape(I // 16, 16, *rest), w[I:].reshape(I // 16, 16, *rest)], 1).reshape(2 * I, *rest).contiguous()


@pytest.mark.parametrize("T,splits,bias", [(1, 4, False), (64, 9, True), (37, 3, True), (128, 2, False)])
def test_rmsnorm_consumes_partials(ops, T, splits, bias):
    from fllm_b200.ops.native import Deferred
    H, K = 4096, 2048
    x = _rand((T, K), 1)
    w = _rand((H, K), 2, 0.05)
    b = _rand((H,), 3) if bias else None
    nw = _rand((H,), 4)
    res = _rand((T, H), 5)
    # unfused: GEMM (+ reduction kernel) then add + norm
    y = ops.linear(x, w, b, force_splits=splits)
    r0 = res.clone()
    h0 = ops.rmsnorm(r0, y, nw, 1e-6)
    # fused: the norm adds the partials
    d = ops.linear(x, w, b, force_splits=splits, defer=True)
    assert isinstance(d, Deferred) and 2 <= d.splits <= splits
    r1 = res.clone()
    h1 = ops.rmsnorm(r1, d, nw, 1e-6)
    assert torch.equal(r0, r1), "updated residual must be bit-identical to the two-kernel path"
    # the row's sum of squares is added in another order (32 warps instead of 8): at most one bf16 step apart
    _close(h1, h0, 1e-2)
    assert ops.check_status() == 0


def test_deferred_linear_without_split_returns_tensor(ops):
    x = _rand((64, 256), 1)
    w = _rand((24576, 256), 2, 0.05)       # enough tiles: no split-K
    y = ops.linear(x, w, defer=True)
    assert isinstance(y, torch.Tensor)
    _close(y, x.float() @ w.float().t())


@pytest.mark.parametrize("D,style,qknorm,bias,kv_dtype", [(128, 0, True, False, torch.bfloat16), (128, 0, False, True, torch.bfloat16),
                                                          (64, 1, True, True, torch.bfloat16), (128, 1, False, False, torch.bfloat16),
                                                          (128, 0, True, False, torch.float8_e4m3fn)])
def test_rope_consumes_partials(ops, D, style, qknorm, bias, kv_dtype):
    from fllm_b200.ops.native import Deferred
    T, hq, hkv, bs, nb, K = 29, 8, 2, 16, 12, 2048
    N = (hq + 2 * hkv) * D
    x = _rand((T, K), 1)
    w = _rand((N, K), 2, 0.05)
    b = _rand((N,), 3) if bias else None
    qn = _rand((D,), 4) if qknorm else None
    kn = _rand((D,), 5) if qknorm else None
    pos = torch.arange(T, dtype=torch.int32, device="cuda") * 3
    slots = torch.randperm(nb * bs, device="cuda")[:T].int()
    slots[5] = -1
    inv = (1.0 / (10000 ** (torch.arange(0, D, 2, device="cuda").float() / D))).contiguous()
    mk = lambda: torch.zeros(nb, hkv, bs, D, device="cuda", dtype=torch.bfloat16).to(kv_dtype)
    kc0, vc0, kc1, vc1 = mk(), mk(), mk(), mk()
    qkv = ops.linear(x, w, b, force_splits=4)
    q0 = ops.rope_kv_write(qkv, pos, slots, inv, qn, kn, kc0, vc0, hq, hkv, D, D, style, 1e-6, 1.0).clone()
    d = ops.linear(x, w, b, force_splits=4, defer=True)
    assert isinstance(d, Deferred)
    q1 = ops.rope_kv_write(d, pos, slots, inv, qn, kn, kc1, vc1, hq, hkv, D, D, style, 1e-6, 1.0)
    assert q1.shape == (T, hq * D)
    assert torch.equal(q0, q1)
    assert torch.equal(kc0.view(torch.uint8), kc1.view(torch.uint8)) and torch.equal(vc0.view(torch.uint8), vc1.view(torch.uint8))


@pytest.mark.parametrize("T", [1, 16, 50, 64, 128, 200, 2048])
@pytest.mark.parametrize("kind", [0, 1])
def test_gemm_gated_epilogue_blocked(ops, ref, T, kind):
    I, K = 1536, 1024
    x = _rand((T, K), 1)
    w = _rand((2 * I, K), 2, 0.05)
    want = ref.glu(ref.linear(x, w), kind)
    got = ops.linear_glu(x, _block16(w), None, kind, layout=16)
    assert got.shape == (T, I)
    _close(got, want)
    assert ops.check_status() == 0


@pytest.mark.parametrize("T", [8, 64, 300])
def test_gemm_gated_epilogue_bias_and_pairs(ops, ref, T):
    I, K = 512, 512
    x = _rand((T, K), 1)
    w = _rand((2 * I, K), 2, 0.05)
    b = _rand((2 * I,), 3)
    # blocked layout with a bias
    want = ref.glu(ref.linear(x, w, b), 0)
    got = ops.linear_glu(x, _block16(w), _block16(b), 0, layout=16)
    _close(got, want)
    # pair layout of the clamped SwiGLU-OAI kind (natural order of that kind)
    want2 = ref.glu(ref.linear(x, w, b), 2, 1.702, 7.0)
    got2 = ops.linear_glu(x, w, b, 2, 1.702, 7.0, layout=0)
    _close(got2, want2)


@pytest.mark.parametrize("T,splits", [(64, 4), (5, 2)])
def test_gated_activation_consumes_partials(ops, ref, T, splits):
    I, K = 768, 4096
    x = _rand((T, K), 1)
    w = _rand((2 * I, K), 2, 0.05)
    want = ref.glu(ref.linear(x, w), 0)
    l0 = ops.launches
    got = ops.linear_glu(x, _block16(w), None, 0, layout=16, force_splits=splits)
    assert ops.launches - l0 == 2          # GEMM with split-K + the activation kernel that adds the partials
    _close(got, want)


def test_glu_blocked_layout_kernel(ops, ref):
    gu = _rand((33, 2 * 1024), 1)
    _close(ops.glu(_block16(gu.t().contiguous()).t().contiguous(), 0, layout=16), ref.glu(gu, 0), 1e-2)


@pytest.mark.parametrize("rows,vocab,dtype", [(64, 151936, torch.bfloat16), (1, 32000, torch.bfloat16), (7, 1000, torch.float32),
                                              (130, 50257, torch.bfloat16)])
def test_argmax_split(ops, rows, vocab, dtype):
    lg = _rand((rows, vocab), 1, dtype=dtype)
    lg[0, vocab - 1] = 100.0
    if rows > 2:
        lg[2, 5] = 50.0
        lg[2, 4000 % vocab] = 50.0            # equal maxima: the lowest index wins
    ids, pairs = ops.argmax(lg, id_offset=3, want_pairs=True)
    want = lg.float().argmax(-1)
    assert torch.equal(ids.long(), want + 3)
    assert torch.equal(pairs[:, 1].long(), want + 3)
    assert torch.equal(pairs[:, 0], lg.float().max(-1).values)
    again, _ = ops.argmax(lg, id_offset=3, want_pairs=True)      # counters were re-zeroed
    assert torch.equal(ids, again)
    sel = ops.argmax_pairs_select(torch.stack([pairs, pairs + 1.0, pairs]))
    assert torch.equal(sel.long(), want + 4)


def test_decoder_step_matches_unfused_chain(ops):
    """A tiny dense model: the decode chain with the split-K reductions left to the consumers against
    the same decoder with stand-alone reduction kernels (equal up to the summation order of the norms)."""
    from fllm_b200.config import ModelConfig
    from fllm_b200.models.decoder import Decoder, KVCache, StepBatch
    from fllm_b200.models.weights import init_random_weights
    cfg = ModelConfig(name="t", vocab_size=1024, hidden_size=1024, intermediate_size=1536, num_layers=2, num_heads=8,
                      num_kv_heads=2, head_dim=128, qk_norm=True)
    outs = []
    for fused in (True, False):
        w = init_random_weights(cfg, "cuda", seed=3)
        kv = KVCache(cfg.num_layers, 32, 2, 16, 128, "cuda")
        dec = Decoder(cfg, w, kv, ops)
        if not fused:
            dec._defer = False
        T = 24
        dev = "cuda"
        b = StepBatch(token_ids=torch.arange(T, dtype=torch.int32, device=dev), positions=torch.zeros(T, dtype=torch.int32, device=dev),
                      slots=torch.arange(T, dtype=torch.int32, device=dev) * 16, row_seq=torch.arange(T, dtype=torch.int32, device=dev),
                      block_tables=torch.arange(T, dtype=torch.int32, device=dev).view(T, 1),
                      logit_rows=torch.arange(T, dtype=torch.int32, device=dev), num_seqs=T, num_tokens=T, max_kv_len=1,
                      all_decode=True, q_starts=torch.arange(T + 1, dtype=torch.int32, device=dev),
                      seq_lens=torch.ones(T, dtype=torch.int32, device=dev))
        outs.append(dec.forward(b).float())
    _close(outs[0], outs[1], 2e-2)
