"""The allocation-free C entry point (``fllm_linear_bf16_splitk_noalloc``) gives the same
result as the regular split-K linear op, call after call, although every call reuses one
fixed scratch array that still holds the previous call's partial sums.

The entry point is meant for C hosts that cannot call cudaMalloc while serving (all device
memory already belongs to the KV pool; an allocation would fail or stall every stream), so the
test drives it the way such a host would: through the exported C symbol, with raw device
pointers and a raw stream handle. This file is named to be collected last.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(y, r, tol=2e-2):
    err = (y.float() - r.float()).abs().max().item()
    scale = r.float().abs().max().item() + 1e-6
    assert err <= tol * scale, f"max abs err {err} vs scale {scale}"


@pytest.fixture(scope="module")
def lib():
    from fllm_b200.ops import _lib
    _lib.load_cuda()
    so = ctypes.CDLL(str(_lib._LIB_CUDA))
    fn = so.fllm_linear_bf16_splitk_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                   ctypes.c_void_p, ctypes.c_void_p]
    so.fllm_noalloc_last_error.restype = ctypes.c_char_p
    so.fllm_noalloc_init.restype = ctypes.c_int
    so.fllm_noalloc_scratch_bytes.restype = ctypes.c_size_t
    return so


def _call(lib, x, w, bias, y, splits, status=None):
    stream = torch.cuda.current_stream().cuda_stream
    return lib.fllm_linear_bf16_splitk_noalloc(
        x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), bias.data_ptr() if bias is not None else None,
        y.data_ptr(), y.stride(0), x.shape[0], w.shape[0], x.shape[1], splits,
        status.data_ptr() if status is not None else None, ctypes.c_void_p(stream))


def test_matches_regular_entry_point_on_two_calls_in_a_row(lib):
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(11)
    ws = torch.zeros(32 << 20, dtype=torch.uint8, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert lib.fllm_noalloc_init() == 0, lib.fllm_noalloc_last_error()
    assert lib.fllm_noalloc_init() == 0                 # idempotent
    # later calls: other shape, other data, fewer splits (down to none) - stale partials must not leak in
    for T, N, K, splits, with_bias in [(64, 2048, 4096, 4, True), (24, 1024, 2048, 2, False), (64, 2048, 4096, 1, True)]:
        x = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device="cuda") * 0.05).to(torch.bfloat16)
        b = torch.randn(N, generator=g, device="cuda").to(torch.bfloat16) if with_bias else None
        want = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
        torch.ops.fllm_b200.linear(x, w, b, want, ws, status, splits)
        got = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device="cuda")
        rc = _call(lib, x, w, b, got, splits, status)
        assert rc == 0, lib.fllm_noalloc_last_error()
        torch.cuda.synchronize()
        _close(got, want)
        _close(got, x.float() @ w.float().t() + (b.float() if b is not None else 0))
        assert int(status.item()) == 0


def test_rejects_what_does_not_fit_the_scratch_array(lib):
    torch.cuda.set_device(0)
    cap = lib.fllm_noalloc_scratch_bytes()
    assert cap == 8 << 20
    T, N, K, splits = 128, 8192, 512, 4                # 16 MiB of partials
    assert 4 * splits * T * N > cap
    x = torch.zeros(T, K, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(N, K, dtype=torch.bfloat16, device="cuda")
    y = torch.ones(T, N, dtype=torch.bfloat16, device="cuda")
    assert _call(lib, x, w, None, y, splits) == -2
    msg = lib.fllm_noalloc_last_error().decode()
    assert "exceeds" in msg and str(cap) in msg
    torch.cuda.synchronize()
    assert bool((y == 1).all())                         # nothing was launched
    assert _call(lib, x[:, :K - 4], w, None, y, 1) == -1   # k not a multiple of 8
    assert _call(lib, x.view(-1)[8:8 + 64 * K].view(64, K)[:, :K], w, None, y, 1) == 0      # 16-byte aligned offset: fine
    odd = x.view(-1)[4:4 + 64 * K].view(64, K)           # 8-byte offset: rejected before anything is launched
    assert _call(lib, odd, w, None, y, 1) == -1 and "aligned" in lib.fllm_noalloc_last_error().decode()
