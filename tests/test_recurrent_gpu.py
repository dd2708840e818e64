"""Recurrent mixer kernels against the fp32 PyTorch statement of the same ops (fllm_b200/ops/recurrent.py), on ragged
batches that mix fresh prompts, continued chunks and single decode rows (the reference checks its recurrent ops the
same way in rust/engine/src/backend/selftest/rwkv.rs and selftest.rs: device op vs host reference on random data)."""
import pytest
import torch

from fllm_b200.ops.recurrent import GATED_DELTA, KDA, RWKV6, RWKV7

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from fllm_b200.ops.native import NativeOps
    from fllm_b200.ops.reference import RefOps
    return NativeOps(torch.device("cuda")), RefOps()


def ragged(lens, fresh, slots, device="cuda"):
    """q_starts, seq_state, positions for sequences of the given step lengths; a non-fresh one continues at 37."""
    qs, pos, t = [0], [], 0
    for n, f in zip(lens, fresh):
        t += n
        qs.append(t)
        pos += list(range(0 if f else 37, (0 if f else 37) + n))
    mk = lambda v: torch.tensor(v, dtype=torch.int32, device=device)
    return mk(qs), mk(slots), mk(pos), t


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9))


CASES = [([5, 1, 17, 1], [True, False, False, True], [3, 0, 2, 5]), ([1, 1, 1], [False, False, False], [1, 2, 0]),
         ([300], [True], [4])]


@pytest.mark.parametrize("W", [2, 3, 4])
@pytest.mark.parametrize("case", CASES)
def test_causal_conv1d(ops, W, case):
    nat, ref = ops
    qs, ss, pos, T = ragged(*case)
    C = 328
    g = torch.Generator(device="cuda").manual_seed(W)
    x = torch.randn(T, C + 8, device="cuda", generator=g).bfloat16()[:, 8:]             # a strided view
    w = torch.randn(C, W, device="cuda", generator=g) * 0.5
    bias = torch.randn(C, device="cuda", generator=g)
    st = torch.randn(6, W - 1, C, device="cuda", generator=g).bfloat16()
    st_ref = st.clone()
    y = nat.causal_conv1d(x, w, bias, st, qs, ss, pos, act=True)
    y_ref = ref.causal_conv1d(x, w, bias, st_ref, qs, ss, pos, act=True)
    torch.cuda.synchronize()
    assert rel(y, y_ref) < 1e-2
    assert torch.equal(st, st_ref)                                # windows are copies of inputs: exact


@pytest.mark.parametrize("max_q", [0, 100, 700])
def test_causal_conv1d_token_runs(ops, max_q):
    """Long sequences are cut into runs of tokens over the grid; a bound below the longest sequence stays correct (the
    last run goes on to the end), and continued sequences still read and move their windows."""
    nat, ref = ops
    qs, ss, pos, T = ragged([700, 130, 2, 1], [False, True, False, False], [3, 0, 2, 5])
    C, W = 328, 4
    g = torch.Generator(device="cuda").manual_seed(max_q)
    x = torch.randn(T, C, device="cuda", generator=g).bfloat16()
    w, bias = torch.randn(C, W, device="cuda", generator=g) * 0.5, torch.randn(C, device="cuda", generator=g)
    st = torch.randn(6, W - 1, C, device="cuda", generator=g).bfloat16()
    st_ref = st.clone()
    y = nat.causal_conv1d(x, w, bias, st, qs, ss, pos, act=True, max_q_len=max_q)
    y_ref = ref.causal_conv1d(x, w, bias, st_ref, qs, ss, pos, act=True)
    torch.cuda.synchronize()
    assert rel(y, y_ref) < 1e-2 and torch.equal(st, st_ref)


@pytest.mark.parametrize("N,P,H,G", [(128, 64, 8, 2), (64, 64, 4, 1), (16, 32, 6, 3), (256, 80, 2, 1), (32, 64, 4, 4)])
@pytest.mark.parametrize("case", CASES)
def test_mamba2_scan(ops, N, P, H, G, case):
    nat, ref = ops
    qs, ss, pos, T = ragged(*case)
    g = torch.Generator(device="cuda").manual_seed(N + P)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    proj = rn(T, (H * P + 2 * G * N + H + 7) // 8 * 8).bfloat16()   # x | B | C | dt as views of one projection
    x, Bm, Cm, dt = proj[:, :H * P], proj[:, H * P:H * P + G * N], proj[:, H * P + G * N:H * P + 2 * G * N], proj[:, H * P + 2 * G * N:H * P + 2 * G * N + H]
    A = -torch.exp(rn(H) * 0.5)
    D, dtb = rn(H), rn(H) * 0.5
    st = rn(6, H, P, N) * 0.5
    st_ref = st.clone()
    y = nat.mamba2_scan(x, dt, Bm, Cm, A, D, dtb, st, qs, ss, pos, H, P, G, N, 0.001, 100.0)
    y_ref = ref.mamba2_scan(x, dt, Bm, Cm, A, D, dtb, st_ref, qs, ss, pos, H, P, G, N, 0.001, 100.0)
    torch.cuda.synchronize()
    assert rel(y, y_ref) < 1e-2
    assert rel(st, st_ref) < 1e-4


@pytest.mark.parametrize("seg_len", [64, 128])
def test_mamba2_scan_sequence_parallel(ops, seg_len):
    """Segments side by side + combine + second pass give the plain walk's outputs and states: a fresh long prompt, a
    continued one, a short one (most of its segments empty) and a decode row in one step; also when `segs` is sized
    for fewer tokens than the longest sequence has."""
    nat, ref = ops
    lens, fresh, slots = [700, 300, 40, 1], [True, False, True, False], [3, 0, 2, 5]
    qs, ss, pos, T = ragged(lens, fresh, slots)
    H, P, G, N = 8, 64, 2, 128
    g = torch.Generator(device="cuda").manual_seed(seg_len)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x, dt = rn(T, H * P).bfloat16(), rn(T, H).bfloat16()
    Bm, Cm = rn(T, G * N).bfloat16(), rn(T, G * N).bfloat16()
    A, D, dtb = -torch.exp(rn(H) * 0.5), rn(H), rn(H) * 0.5 - 1.0
    st0 = rn(6, H, P, N) * 0.5
    st_ref = st0.clone()
    y_ref = ref.mamba2_scan(x, dt, Bm, Cm, A, D, dtb, st_ref, qs, ss, pos, H, P, G, N, 0.001, 100.0)
    for max_q in (700, 500):
        st = st0.clone()
        y = nat.mamba2_scan(x, dt, Bm, Cm, A, D, dtb, st, qs, ss, pos, H, P, G, N, 0.001, 100.0, max_q_len=max_q, seg_len=seg_len)
        torch.cuda.synchronize()
        assert rel(y, y_ref) < 1e-2 and rel(st, st_ref) < 1e-3, max_q
    assert nat.launches >= 6                                     # three launches per segmented call


@pytest.mark.parametrize("N", [16, 8])
@pytest.mark.parametrize("case", CASES)
def test_mamba1_scan(ops, N, case):
    nat, ref = ops
    qs, ss, pos, T = ragged(*case)
    Dm = 200
    g = torch.Generator(device="cuda").manual_seed(N)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x, dt, z = rn(T, Dm).bfloat16(), rn(T, Dm).bfloat16(), rn(T, Dm).bfloat16()
    bc = rn(T, 2 * N).bfloat16()
    Bm, Cm = bc[:, :N], bc[:, N:]
    A = -torch.exp(rn(Dm, N) * 0.5)
    D, dtb = rn(Dm), rn(Dm) * 0.5
    st = rn(6, Dm, N) * 0.5
    st_ref = st.clone()
    if N == 8:                                                     # 8 bf16 = one 16-byte word: views stay aligned
        Bm, Cm = Bm.contiguous(), Cm.contiguous()
    y = nat.mamba1_scan(x, dt, Bm, Cm, z, A, D, dtb, st, qs, ss, pos)
    y_ref = ref.mamba1_scan(x, dt, Bm, Cm, z, A, D, dtb, st_ref, qs, ss, pos)
    torch.cuda.synchronize()
    assert rel(y, y_ref) < 1e-2
    assert rel(st, st_ref) < 1e-4


@pytest.mark.parametrize("kind", [RWKV6, RWKV7, GATED_DELTA, KDA])
@pytest.mark.parametrize("DK,DV,H,ratio", [(64, 64, 4, 1), (128, 128, 4, 2), (32, 48, 2, 1), (256, 64, 2, 1)])
@pytest.mark.parametrize("case", CASES)
def test_matrix_state_scan(ops, kind, DK, DV, H, ratio, case):
    nat, ref = ops
    if kind in (RWKV6, RWKV7, KDA) and ratio != 1:
        ratio = 1
    qs, ss, pos, T = ragged(*case)
    g = torch.Generator(device="cuda").manual_seed(kind * 7 + DK)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    Hk = H // ratio
    r, k = rn(T, Hk * DK).bfloat16(), (rn(T, Hk * DK) * (0.3 if kind != RWKV7 else 1.0)).bfloat16()
    v = rn(T, H * DV).bfloat16()
    a = b = u = beta = None
    if kind == RWKV7:                                              # a = -kk, b = kk * gate with kk a unit vector per head
        kk = torch.nn.functional.normalize(rn(T, Hk, DK), dim=-1)
        a = (-kk).reshape(T, -1).bfloat16()
        b = (kk * torch.sigmoid(rn(T, Hk, DK))).reshape(T, -1).bfloat16()
        k = (k.float() * 0.3).bfloat16()
    if kind == RWKV6:
        u = rn(Hk * DK) * 0.5
    if kind in (GATED_DELTA, KDA):
        beta = torch.sigmoid(rn(T, H)).bfloat16()
    w = -torch.exp(rn(T, H if kind == GATED_DELTA else Hk * DK) - 1.0)
    st = rn(6, H, DV, DK) * 0.3
    st_ref = st.clone()
    l2 = kind in (GATED_DELTA, KDA)
    y = nat.matrix_state_scan(kind, r, k, v, a, b, w, u, beta, st, qs, ss, pos, H, DK, DV, ratio, l2, DK ** -0.5)
    y_ref = ref.matrix_state_scan(kind, r, k, v, a, b, w, u, beta, st_ref, qs, ss, pos, H, DK, DV, ratio, l2, DK ** -0.5)
    torch.cuda.synchronize()
    assert rel(y, y_ref) < 1e-2
    assert rel(st, st_ref) < 1e-4


@pytest.mark.parametrize("gs,before,D", [(0, False, 640), (64, False, 640), (128, True, 640), (40, True, 640),
                                          (0, False, 5120), (2048, False, 4096), (0, True, 10240), (0, False, 1026)])
def test_gated_rmsnorm(ops, gs, before, D):
    nat, ref = ops
    T = 37
    g = torch.Generator(device="cuda").manual_seed(3)
    x, z = torch.randn(T, D, device="cuda", generator=g).bfloat16(), torch.randn(T, D, device="cuda", generator=g).bfloat16()
    w = torch.randn((gs or D) if before else D, device="cuda", generator=g).bfloat16()
    y = nat.gated_rmsnorm(x, z, w, 1e-5, gs, before)
    y_ref = ref.gated_rmsnorm(x, z, w, 1e-5, gs, before)
    assert rel(y, y_ref) < 1e-2
    y2 = nat.gated_rmsnorm(x, None, w, 1e-5, gs, before)
    assert rel(y2, ref.gated_rmsnorm(x, None, w, 1e-5, gs, before)) < 1e-2


@pytest.mark.parametrize("H", [4, 16, 6, 40])
def test_latent_attention_kernel(ops, H):
    """Ragged rows (two prefill chunks and decode rows) over a paged latent pool with shuffled blocks."""
    nat, ref = ops
    g = torch.Generator(device="cuda").manual_seed(H)
    bs, nblocks = 16, 40
    cache = (torch.randn(nblocks + 1, bs, 576, device="cuda", generator=g) * 0.5).bfloat16()
    lens = [(0, 33), (100, 1), (17, 20), (299, 1)]                 # (tokens before the step, rows in the step)
    perm = torch.randperm(nblocks, device="cuda", generator=g).int()
    tables = torch.zeros(len(lens), 20, dtype=torch.int32, device="cuda")
    row_seq, pos, used = [], [], 0
    for s, (past, n) in enumerate(lens):
        need = (past + n + bs - 1) // bs
        tables[s, :need] = perm[used:used + need]
        used += need
        row_seq += [s] * n
        pos += list(range(past, past + n))
    row_seq = torch.tensor(row_seq, dtype=torch.int32, device="cuda")
    pos = torch.tensor(pos, dtype=torch.int32, device="cuda")
    T = len(pos)
    q_abs = torch.randn(H, T, 512, device="cuda", generator=g).bfloat16()
    q_pe = torch.randn(T, H, 64, device="cuda", generator=g).bfloat16()
    want = ref.attention_mla(q_abs, q_pe, cache, tables, row_seq, pos, 576 ** -0.5)
    out = nat.attention_mla(q_abs, q_pe, cache, tables, row_seq, pos, 576 ** -0.5, tensor_cores=False)
    torch.cuda.synchronize()
    assert rel(out, want) < 1e-2
    for splits in (1, 2, 4):                                      # tensor-core kernel; slices beyond a short row's keys are empty
        out = nat.attention_mla(q_abs, q_pe, cache, tables, row_seq, pos, 576 ** -0.5, splits=splits)
        torch.cuda.synchronize()
        assert rel(out, want) < 1e-2, splits
    assert int(nat.k.attention_mla_splits(4, 16, 4096)) > 1 and int(nat.k.attention_mla_splits(2048, 16, 4096)) == 1


def test_latent_prepare_kernel(ops):
    """RMSNorm + rotation into cache rows (padding rows write nothing) and the rotated query parts."""
    nat, ref = ops
    g = torch.Generator(device="cuda").manual_seed(9)
    T, H = 23, 6
    ckv = torch.randn(T, 576, device="cuda", generator=g).bfloat16()
    q = torch.randn(T, H, 192, device="cuda", generator=g).bfloat16()
    pos = torch.randint(0, 5000, (T,), device="cuda", generator=g).int()
    slots = torch.randperm(16 * 8, device="cuda", generator=g)[:T].int()
    slots[5] = -1
    inv_freq = (10000.0 ** (-torch.arange(32, device="cuda").float() / 32)).contiguous()
    w = (1 + 0.3 * torch.randn(512, device="cuda", generator=g)).bfloat16()
    c1 = torch.zeros(8, 16, 576, device="cuda", dtype=torch.bfloat16)
    c2 = c1.clone()
    a = nat.mla_prepare(ckv, q, 128, pos, slots, inv_freq, 1.3, w, 1e-6, c1)
    b = ref.mla_prepare(ckv, q, 128, pos, slots, inv_freq, 1.3, w, 1e-6, c2)
    torch.cuda.synchronize()
    assert rel(a, b) < 1e-2 and rel(c1, c2) < 1e-2
    assert int((c1.view(-1, 576).abs().sum(-1) > 0).sum()) == T - 1


def test_gated_delta_raw_gates(ops):
    """The scan computes the step size and the decay from their logits (views of one projection output)."""
    nat, ref = ops
    qs, ss, pos, T = ragged([5, 1, 17, 1], [True, False, False, True], [3, 0, 2, 5])
    Hv, Hk, D = 4, 2, 128
    g = torch.Generator(device="cuda").manual_seed(11)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    r, k, v = rn(T, Hk * D).bfloat16(), (rn(T, Hk * D) * 0.3).bfloat16(), rn(T, Hv * D).bfloat16()
    ba = rn(T, 2 * Hv + 8).bfloat16()
    A, dtb = -torch.exp(rn(Hv) * 0.5), rn(Hv) * 0.5
    st = rn(6, Hv, D, D) * 0.3
    st_ref = st.clone()
    args = (GATED_DELTA, r, k, v, None, None, None, None, ba[:, :Hv])
    kw = dict(gate_raw=ba[:, Hv:2 * Hv], gate_A=A, gate_dt_bias=dtb)
    y = nat.matrix_state_scan(*args, st, qs, ss, pos, Hv, D, D, 2, True, D ** -0.5, **kw)
    y_ref = ref.matrix_state_scan(*args, st_ref, qs, ss, pos, Hv, D, D, 2, True, D ** -0.5, **kw)
    torch.cuda.synchronize()
    assert rel(y, y_ref) < 1e-2 and rel(st, st_ref) < 1e-4


@pytest.mark.parametrize("seg_len", [64, 128])
def test_mamba1_scan_sequence_parallel(ops, seg_len):
    nat, ref = ops
    lens, fresh, slots = [700, 300, 40, 1], [True, False, True, False], [3, 0, 2, 5]
    qs, ss, pos, T = ragged(lens, fresh, slots)
    Dm, N = 200, 16
    g = torch.Generator(device="cuda").manual_seed(seg_len + 1)
    rn = lambda *s: torch.randn(*s, device="cuda", generator=g)
    x, dt, z = rn(T, Dm).bfloat16(), (rn(T, Dm) - 1.0).bfloat16(), rn(T, Dm).bfloat16()
    bc = rn(T, 2 * N).bfloat16()
    A, D, dtb = -torch.exp(rn(Dm, N) * 0.5), rn(Dm), rn(Dm) * 0.5
    st0 = rn(6, Dm, N) * 0.5
    st_ref = st0.clone()
    y_ref = ref.mamba1_scan(x, dt, bc[:, :N], bc[:, N:], z, A, D, dtb, st_ref, qs, ss, pos)
    for max_q in (700, 500):
        st = st0.clone()
        y = nat.mamba1_scan(x, dt, bc[:, :N], bc[:, N:], z, A, D, dtb, st, qs, ss, pos, max_q_len=max_q, seg_len=seg_len)
        torch.cuda.synchronize()
        assert rel(y, y_ref) < 1e-2 and rel(st, st_ref) < 1e-3, max_q
