"""Numerics of the sm_100a kernels against plain PyTorch fp32 references of the same ops.
Shapes include odd row counts, partial tiles and forced split-K."""
import math

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
    if y.numel() == 0:
        return
    err = (y.float() - r.float()).abs().max().item()
    scale = r.float().abs().max().item() + 1e-6
    assert err <= tol * scale, f"max abs err {err} vs scale {scale}"


@pytest.mark.parametrize("T", [1, 7, 16, 33, 64, 100, 128, 129, 300, 2048])
@pytest.mark.parametrize("N,K", [(256, 128), (1024, 4096), (1000, 320), (6144, 4096)])
def test_linear(ops, T, N, K):
    x = _rand((T, K), 1)
    w = _rand((N, K), 2, 0.05)
    y = ops.linear(x, w)
    _close(y, x.float() @ w.float().t())
    assert ops.check_status() == 0


@pytest.mark.parametrize("T,splits", [(5, 2), (64, 4), (128, 7), (16, 16)])
def test_linear_split_k_and_bias(ops, T, splits):
    x = _rand((T, 4096), 3)
    w = _rand((512, 4096), 4, 0.05)
    b = _rand((512,), 5)
    y = ops.linear(x, w, b, force_splits=splits)
    _close(y, x.float() @ w.float().t() + b.float())
    y1 = ops.linear(x, w, b, force_splits=1)
    _close(y1, x.float() @ w.float().t() + b.float())


def test_linear_strided_operands(ops):
    big = _rand((70, 3 * 512), 6)
    x = big[:, 512:1024]                       # row pitch 1536, offset 512 elements
    w = _rand((768, 512), 7, 0.05)
    out_big = torch.zeros(70, 2048, dtype=torch.bfloat16, device="cuda")
    y = out_big[:, 256:1024]
    ops.linear(x, w, out=y)
    _close(y, x.float() @ w.float().t())
    assert out_big[:, :256].abs().max() == 0 and out_big[:, 1024:].abs().max() == 0


def test_linear_deterministic(ops):
    x = _rand((64, 4096), 8)
    w = _rand((4096, 4096), 9, 0.05)
    assert torch.equal(ops.linear(x, w), ops.linear(x, w))


@pytest.mark.parametrize("rows,hidden", [(1, 256), (13, 4096), (64, 2880), (5, 8192)])
def test_rmsnorm(ops, ref, rows, hidden):
    x = _rand((rows, hidden), 1)
    d = _rand((rows, hidden), 2)
    w = _rand((hidden,), 3)
    xr, xn = x.clone(), x.clone()
    y = ops.rmsnorm(xn, d, w, 1e-6)
    yr = ref.rmsnorm(xr, d, w, 1e-6)
    _close(y, yr, 1e-2)
    assert torch.equal(xn, xr)
    _close(ops.rmsnorm(x.clone(), None, w, 1e-5), ref.rmsnorm(x.clone(), None, w, 1e-5), 1e-2)


@pytest.mark.parametrize("D,style,qknorm,rot", [(128, 0, True, 128), (64, 0, False, 64), (128, 1, False, 128),
                                                 (64, 1, True, 64), (128, 0, False, 64), (256, 0, True, 256)])
def test_rope_kv_write(ops, ref, D, style, qknorm, rot):
    T, hq, hkv, bs, nb = 37, 8, 2, 16, 12
    qkv = _rand((T, (hq + 2 * hkv) * D), 1)
    pos = torch.randint(0, 5000, (T,), device="cuda", dtype=torch.int32)
    slots = torch.randperm(nb * bs, device="cuda")[:T].int()
    slots[3] = -1
    inv = (10000.0 ** (-torch.arange(0, rot, 2, device="cuda").float() / rot))
    qn = _rand((D,), 2) if qknorm else None
    kn = _rand((D,), 3) if qknorm else None
    kc = torch.zeros(nb, hkv, bs, D, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    kc_r, vc_r, qkv_r = kc.clone(), vc.clone(), qkv.clone()
    ops.rope_kv_write(qkv, pos, slots, inv, qn, kn, kc, vc, hq, hkv, D, rot, style, 1e-6, 1.0)
    ref.rope_kv_write(qkv_r, pos, slots, inv, qn, kn, kc_r, vc_r, hq, hkv, D, rot, style, 1e-6, 1.0)
    _close(qkv[:, : hq * D], qkv_r[:, : hq * D], 2e-2)
    _close(kc, kc_r, 2e-2)
    assert torch.equal(vc, vc_r)


@pytest.mark.parametrize("kind", [0, 1, 2])
def test_glu(ops, ref, kind):
    x = _rand((19, 2 * 1376), 1, 2.0)
    _close(ops.glu(x, kind, 1.702, 7.0), ref.glu(x, kind, 1.702, 7.0), 1e-2)


def _paged_setup(B, lens, hkv, D, bs=16, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    max_blocks = max((l + bs - 1) // bs for l in lens)
    nb = sum((l + bs - 1) // bs for l in lens) + 3
    perm = torch.randperm(nb, generator=g, device="cuda").int()
    tables = torch.zeros(B, max_blocks, dtype=torch.int32, device="cuda")
    o = 0
    for i, l in enumerate(lens):
        n = (l + bs - 1) // bs
        tables[i, :n] = perm[o:o + n]
        o += n
    kc = (torch.randn(nb, hkv, bs, D, generator=g, device="cuda")).to(torch.bfloat16)
    vc = (torch.randn(nb, hkv, bs, D, generator=g, device="cuda")).to(torch.bfloat16)
    return tables, kc, vc


@pytest.mark.parametrize("D,hq,hkv", [(128, 8, 2), (64, 8, 8), (128, 4, 1)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (20, True, 0.0), (0, False, 30.0)])
def test_attention_generic(ops, ref, D, hq, hkv, window, sinks, softcap):
    lens = [1, 17, 64, 130]
    tables, kc, vc = _paged_setup(len(lens), lens, hkv, D)
    # mixed rows: last token of every sequence plus a few prefill rows of the longest one
    row_seq = torch.tensor([0, 1, 2, 3, 3, 3], dtype=torch.int32, device="cuda")
    pos = torch.tensor([0, 16, 63, 129, 50, 7], dtype=torch.int32, device="cuda")
    q = _rand((6, hq * D), 5)
    sk = torch.randn(hq, device="cuda") if sinks else None
    y = ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap)
    yr = ref.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap)
    _close(y, yr, 2e-2)


def test_argmax_and_sampler(ops):
    from fllm_b200.ops.native import pack_sample_rows
    from fllm_b200.ops.reference import sample_reference
    R, V = 9, 5003
    lg = _rand((R, V), 1, 3.0, torch.float32)
    ids = ops.argmax(lg)
    assert torch.equal(ids.long(), lg.argmax(-1))
    ids_b = ops.argmax(lg.to(torch.bfloat16), id_offset=100)
    assert torch.equal(ids_b.long() - 100, lg.to(torch.bfloat16).float().argmax(-1))
    rows = []
    for r in range(R):
        rows.append((0.8 + 0.1 * r, [1.0, 0.9, 0.5][r % 3], [0.0, 0.05][r % 2], 1.0, 0.0, 0.0, [0, 5, 50][r % 3], r, 1234 + r))
    prm = torch.frombuffer(bytearray(pack_sample_rows(rows)), dtype=torch.uint8).cuda()
    got = ops.sample(lg.clone(), prm).tolist()
    want = [sample_reference(lg[r], *[rows[r][i] for i in (0, 6, 1, 2, 8, 7)]) for r in range(R)]
    assert sum(g == w for g, w in zip(got, want)) >= R - 1, (got, want)
    # greedy rows through the full sampler, with a penalty that flips the winner
    rows = [(0.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0, 0, 1)] * R
    prm = torch.frombuffer(bytearray(pack_sample_rows(rows)), dtype=torch.uint8).cuda()
    top = lg.argmax(-1)
    pen_ids = top.int().view(R, 1).contiguous()
    pen_cnt = torch.ones_like(pen_ids)
    rows_pen = [(0.0, 1.0, 0.0, 1.0, 100.0, 0.0, 0, 0, 1)] * R
    prm_pen = torch.frombuffer(bytearray(pack_sample_rows(rows_pen)), dtype=torch.uint8).cuda()
    assert torch.equal(ops.sample(lg.clone(), prm).long(), top)
    second = lg.clone().scatter_(1, top.view(-1, 1), -1e30).argmax(-1)
    assert torch.equal(ops.sample(lg.clone(), prm_pen, pen_ids, pen_cnt).long(), second)


def test_sampler_distribution(ops):
    """Gumbel-max draws follow softmax(logits / T) (chi-square style bound on 4 tokens)."""
    from fllm_b200.ops.native import pack_sample_rows
    R = 4000
    base = torch.tensor([2.0, 1.0, 0.0, -1.0], device="cuda")
    lg = base.repeat(R, 1).contiguous()
    rows = [(1.0, 1.0, 0.0, 1.0, 0.0, 0.0, 0, r, 99) for r in range(R)]
    prm = torch.frombuffer(bytearray(pack_sample_rows(rows)), dtype=torch.uint8).cuda()
    ids = ops.sample(lg, prm)
    freq = torch.bincount(ids.long(), minlength=4).float() / R
    want = torch.softmax(base, 0)
    assert (freq - want).abs().max().item() < 0.03, (freq, want)


def test_spec_verify_greedy(ops):
    k = 4
    draft = torch.tensor([[5, 6, 7, 8], [1, 2, 3, 4], [9, 9, 9, 9]], dtype=torch.int32, device="cuda")
    target = torch.tensor([[5, 6, 0, 8, 1], [1, 2, 3, 4, 77], [3, 9, 9, 9, 9]], dtype=torch.int32, device="cuda")
    n_acc = torch.zeros(3, dtype=torch.int32, device="cuda")
    out = torch.full((3, k + 1), -1, dtype=torch.int32, device="cuda")
    ops.k.spec_verify_greedy(draft, target, None, n_acc, out)
    assert n_acc.tolist() == [2, 4, 0]
    assert out[0, :3].tolist() == [5, 6, 0] and out[1].tolist() == [1, 2, 3, 4, 77] and out[2, 0].item() == 3


def test_spec_verify_device_rule_equals_host_rule(ops):
    """Ragged verify rows, sampled and greedy rows, with and without draft logits: the device decision equals the
    host statement of the rule on the same counter-based random numbers."""
    from fllm_b200.ops.reference import RefOps
    ref = RefOps()
    g = torch.Generator().manual_seed(5)
    V, k = 1000, 3
    nd = [3, 1, 2, 3, 0, 3]
    B = len(nd)
    starts, r = [], 2                                         # two unrelated rows first
    for n in nd:
        starts.append(r)
        r += n + 1
    tl = (torch.randn(r, V, generator=g) * 2.0).cuda()
    dl = (tl[torch.tensor([min(s + i, r - 1) for s in starts for i in range(k)])].cpu()
          + torch.randn(B * k, V, generator=g) * 0.7).cuda()  # drafts resemble the target: both outcomes occur
    draft = torch.full((B, k), -1, dtype=torch.int32)
    for b in range(B):
        for i in range(nd[b]):
            draft[b, i] = int(torch.multinomial(torch.softmax(dl[b * k + i].cpu(), -1), 1, generator=g))
    draft = draft.clamp_min(0).cuda()
    n_d = torch.tensor(nd, dtype=torch.int32, device="cuda")
    rs = torch.tensor(starts, dtype=torch.int32, device="cuda")
    accepted = 0
    for trial in range(4):
        params = [(0.0 if b == 4 else 0.9, 1.0, 0.0, 1.0, 0.0, 0.0, 0, 2 * trial, 1234 + 17 * b + trial) for b in range(B)]
        for q in (dl, None):
            a_dev, o_dev = ops.spec_verify_sampled(tl, q, draft, params, n_d, rs)
            a_ref, o_ref = ref.spec_verify_sampled(tl.cpu(), None if q is None else q.cpu(), draft.cpu(), params, n_d.cpu(), rs.cpu())
            assert a_dev.cpu().tolist() == a_ref.tolist(), (trial, a_dev, a_ref)
            for b in range(B):
                n = int(a_ref[b]) + 1
                assert o_dev[b, :n].cpu().tolist() == o_ref[b, :n].tolist(), (trial, b)
            accepted += int(a_ref.sum())
    assert 0 < accepted < 8 * sum(nd)
    # greedy ids, ragged
    ids = tl.argmax(-1).int()
    gd = draft.clone()
    gd[0, 0] = ids[starts[0]]
    a_dev, o_dev = ops.spec_verify_greedy(gd, ids, n_d, rs)
    a_ref, o_ref = ref.spec_verify_greedy(gd.cpu(), ids.cpu(), n_d.cpu(), rs.cpu())
    assert a_dev.cpu().tolist() == a_ref.tolist() and int(a_ref[0]) >= 1
    for b in range(B):
        n = int(a_ref[b]) + 1
        assert o_dev[b, :n].cpu().tolist() == o_ref[b, :n].tolist()


class _Meta:
    pass


def _tc_meta(q_lens, kv_lens):
    m = _Meta()
    qs = [0]
    for n in q_lens:
        qs.append(qs[-1] + n)
    m.q_starts = torch.tensor(qs, dtype=torch.int32, device="cuda")
    m.seq_lens = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    m.num_seqs, m.max_q_len, m.min_q_len, m.max_kv_len = len(q_lens), max(q_lens), min(q_lens), max(kv_lens)
    return m


@pytest.mark.parametrize("D,hq,hkv", [(128, 8, 2), (64, 8, 8), (128, 4, 1), (64, 16, 2), (128, 32, 8)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (40, True, 0.0), (0, False, 30.0)])
@pytest.mark.parametrize("case", ["decode", "decode_few", "prefill", "mixed", "verify"])
def test_attention_tc(ops, ref, D, hq, hkv, window, sinks, softcap, case):
    if case == "decode":
        kv_lens, q_lens = [1, 17, 64, 130, 700, 33, 16, 257], [1] * 8
    elif case == "decode_few":            # few sequences: exercises the split-KV path + merge
        kv_lens, q_lens = [900, 35], [1, 1]
    elif case == "prefill":
        kv_lens, q_lens = [200, 64, 130, 17], [200, 64, 100, 17]
    elif case == "mixed":
        kv_lens, q_lens = [300, 90, 45, 128], [1, 90, 1, 64]
    else:                                  # speculative verify rows: up to 16 / group queries
        n = max(1, min(4, 16 // (hq // hkv)))
        kv_lens, q_lens = [100, 37, 260], [n, n, n]
    tables, kc, vc = _paged_setup(len(kv_lens), kv_lens, hkv, D, seed=3)
    T = sum(q_lens)
    row_seq = torch.tensor([i for i, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device="cuda")
    pos = torch.tensor([kv - n + j for kv, n in zip(kv_lens, q_lens) for j in range(n)], dtype=torch.int32, device="cuda")
    q = _rand((T, hq * D), 5)
    sk = torch.randn(hq, device="cuda") if sinks else None
    meta = _tc_meta(q_lens, kv_lens)
    y = ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap, meta=meta)
    yr = ref.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap)
    _close(y, yr, 2e-2)
    # the always-correct generic kernel agrees too
    yg = ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap)
    _close(yg, yr, 2e-2)


@pytest.mark.parametrize("D,hq,hkv", [(128, 8, 8), (128, 8, 2), (128, 16, 2), (128, 32, 8), (128, 16, 1),
                                      (64, 8, 8), (64, 16, 2), (64, 64, 8)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (150, True, 0.0), (0, False, 30.0)])
def test_attention_prefill_on_tensor_memory(ops, ref, D, hq, hkv, window, sinks, softcap):
    """Prompts long enough for several 128-token KV tiles and several 128-row query tiles per sequence go
    through the tcgen05 prefill kernel (head_dim 128 and 64): chunk continuation (kv > q), a ragged tail, causal
    diagonal tiles, sliding window, sinks and soft capping against the fp32 reference; status stays 0."""
    kv_lens, q_lens = [1000, 520, 300, 131], [1000, 200, 300, 40]
    tables, kc, vc = _paged_setup(len(kv_lens), kv_lens, hkv, D, seed=11)
    T = sum(q_lens)
    row_seq = torch.tensor([i for i, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device="cuda")
    pos = torch.tensor([kv - n + j for kv, n in zip(kv_lens, q_lens) for j in range(n)], dtype=torch.int32, device="cuda")
    q = _rand((T, hq * D), 7)
    sk = torch.randn(hq, device="cuda") if sinks else None
    meta = _tc_meta(q_lens, kv_lens)
    y = ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap, meta=meta)
    yr = torch.empty_like(y)
    o = 0
    for i, (n, kv) in enumerate(zip(q_lens, kv_lens)):          # fp32 reference, one dense sequence at a time
        blocks = tables[i, :(kv + 15) // 16].long()
        k = kc[blocks].float().permute(1, 0, 2, 3).reshape(hkv, -1, D)[:, :kv].repeat_interleave(hq // hkv, 0)
        v = vc[blocks].float().permute(1, 0, 2, 3).reshape(hkv, -1, D)[:, :kv].repeat_interleave(hq // hkv, 0)
        qs = q[o:o + n].float().view(n, hq, D).permute(1, 0, 2)
        sc = torch.einsum("hqd,hkd->hqk", qs, k) * D ** -0.5
        if softcap > 0:
            sc = softcap * torch.tanh(sc / softcap)
        qpos = torch.arange(kv - n, kv, device="cuda")[:, None]
        kpos = torch.arange(kv, device="cuda")[None, :]
        hide = kpos > qpos
        if window > 0:
            hide = hide | (kpos <= qpos - window)
        sc = sc.masked_fill(hide[None], float("-inf"))
        if sk is not None:
            pr = torch.softmax(torch.cat([sc, sk.float()[:, None, None].expand(hq, n, 1)], -1), -1)[..., :-1]
        else:
            pr = torch.softmax(sc, -1)
        yr[o:o + n] = torch.einsum("hqk,hkd->qhd", pr, v).reshape(n, hq * D).to(y.dtype)
        o += n
    _close(y, yr, 2e-2)
    assert ops.check_status() == 0


@pytest.mark.parametrize("tp,T", [(2, 64), (4, 13), (8, 64), (8, 5), (4, 300), (2, 2048)])
def test_fused_tp_chain_single_device_emulation(tp, T):
    """GEMM->reduce-scatter, reduce+norm+all-gather and all-gather->GEMM for `tp` virtual ranks on
    one GPU, launched phase by phase (a kernel never waits for a kernel that has not been
    launched yet). Run twice: the counters are monotonic, so the second pass checks replay."""
    from fllm_b200.comm.symm import FusedTP
    H, K, N2 = 512, 256, 384
    ranks = FusedTP.local_group(tp, H, 2048)
    g = torch.Generator(device="cuda").manual_seed(tp * 1000 + T)
    rnd = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device="cuda") * sc).to(torch.bfloat16)
    for it in range(2):
        xs = [rnd(T, K, sc=0.5) for _ in range(tp)]
        ws = [rnd(H, K, sc=0.05) for _ in range(tp)]
        w2 = rnd(N2, H, sc=0.05)
        res_full = rnd(T, H)
        normw = rnd(H)
        shards = []
        for r in ranks:
            lo, hi = r.my_rows(T)
            sh = torch.zeros(max(hi - lo, 1), H, dtype=torch.bfloat16, device="cuda")
            sh[: hi - lo] = res_full[lo:hi]
            shards.append(sh)
        for r, x, w in zip(ranks, xs, ws):
            r.linear_rs(x, w)
        for r, sh in zip(ranks, shards):
            r.norm(sh, T, True, normw, 1e-6)
        outs = [r.linear_ag(T, w2) for r in ranks]
        torch.cuda.synchronize()
        if T <= 128:
            # one-shot layout: partial sums broadcast to every rank, every rank reduces all rows
            fulls = [res_full.clone() for _ in ranks]
            for r, x, w in zip(ranks, xs, ws):
                r.linear_rs(x, w, None, True)
            for r, f in zip(ranks, fulls):
                r.norm(f, T, True, normw, 1e-6, 0.0, True)
            torch.cuda.synchronize()
            gathered = [r.ag_local[:T].clone() for r in ranks]
        part = sum(x.float() @ w.float().t() for x, w in zip(xs, ws))
        new_res = (res_full.float() + part.to(torch.bfloat16).float()).to(torch.bfloat16)
        hn = new_res.float() * torch.rsqrt(new_res.float().pow(2).mean(-1, keepdim=True) + 1e-6) * normw.float()
        want = hn.to(torch.bfloat16).float() @ w2.float().t()
        for r, sh, o in zip(ranks, shards, outs):
            lo, hi = r.my_rows(T)
            _close(sh[: hi - lo], new_res[lo:hi], 3e-2)
            _close(o, want, 3e-2)
            assert r.check_status() == 0
        # every rank computed bit-identical gathered activations
        for o in outs[1:]:
            assert torch.equal(o, outs[0])
        if T <= 128:
            for f, gth in zip(fulls, gathered):
                _close(f, new_res, 3e-2)
                _close(gth, hn, 3e-2)
                assert torch.equal(gth, gathered[0])


def test_fused_tp_allreduce_single_device_emulation():
    """All virtual ranks push first (phase 1 is part of the same kernel), so on one device the
    kernel of rank r can only complete once every rank has pushed: launch order would deadlock a
    real wait, hence this test only exercises the time-out path of the first rank and checks
    that the status word reports it and the context stays usable."""
    from fllm_b200.comm.symm import FusedTP
    ranks = FusedTP.local_group(2, 256, 64)
    x = torch.ones(64, dtype=torch.float32, device="cuda")
    out = ranks[0].all_reduce(x)          # rank 1 never arrives: bounded wait, then error status
    torch.cuda.synchronize()
    assert ranks[0].check_status() == 2
    y = torch.ones(8, device="cuda") * 2  # the CUDA context still works
    assert float(y.sum()) == 16.0


@pytest.mark.parametrize("T,E,k,H,I,act", [(5, 8, 4, 256, 256, "swiglu_oai"), (64, 32, 4, 512, 384, "swiglu"),
                                            (300, 16, 2, 256, 128, "swiglu"), (33, 128, 4, 384, 192, "swiglu_oai")])
@pytest.mark.parametrize("lo_frac", [0.0, 0.5])
def test_moe_native_matches_reference(ops, T, E, k, H, I, act, lo_frac):
    """Device MoE (route, align, gather, grouped tcgen05 GEMMs, combine) against the fp32 oracle,
    for all experts local and for the upper half of the experts only (expert parallel shard)."""
    from types import SimpleNamespace
    from fllm_b200.config import ModelConfig
    from fllm_b200.models.moe import moe_ffn, moe_reference
    from fllm_b200.models.weights import LayerWeights
    cfg = ModelConfig(hidden_size=H, num_experts=E, experts_per_token=k, moe_intermediate_size=I, act=act,
                      expert_bias=True)
    lo = int(E * lo_frac)
    el = E - lo
    lw = LayerWeights(attn_norm=None, wqkv=None, wo=None, ffn_norm=None)
    lw.router_w, lw.router_b = _rand((E, H), 1, 0.2), _rand((E,), 2, 0.1)
    lw.exp_gate_up, lw.exp_gate_up_b = _rand((el, 2 * I, H), 3, 0.05), _rand((el, 2 * I), 4, 0.1)
    lw.exp_down, lw.exp_down_b = _rand((el, H, I), 5, 0.05), _rand((el, H), 6, 0.1)
    h = _rand((T, H), 7)
    dec = SimpleNamespace(cfg=cfg, ops=ops, act_kind={"swiglu": 0, "swiglu_oai": 2}[act],
                          spec=SimpleNamespace(expert_parallel=lo > 0, expert_start=lo))
    got = moe_ffn(dec, lw, h)
    want = moe_reference(cfg, lw, h, lo)
    _close(got, want, 3e-2)
    assert ops.check_status() == 0


@pytest.mark.parametrize("T", [1, 16, 33, 64, 100, 300, 2048])
@pytest.mark.parametrize("N,K", [(256, 256), (1024, 4096), (3584, 8192), (1280, 12288)])
def test_linear_fp8_block(ops, T, N, K):
    """Block-scaled e4m3 GEMM against fp32 math on the de-quantised operands (so only the
    accumulation order and the bf16 output rounding differ), and against the unquantised product
    with the tolerance FP8 allows."""
    from fllm_b200.ops.native import Fp8BlockLinear, quantize_weight_fp8_block
    x = _rand((T, K), 1)
    w = _rand((N, K), 2, 0.05)
    wq, sw = quantize_weight_fp8_block(w)
    bias = _rand((N,), 3) if T % 2 == 0 else None          # split-K adds it in the reduction, the single pass in the epilogue
    lin = Fp8BlockLinear(ops, wq, sw, bias)
    y = lin(x)
    # oracle on the same quantised values
    xq = torch.empty(T, K, dtype=torch.uint8, device="cuda")
    sx = torch.empty(T, K // 128, dtype=torch.float32, device="cuda")
    ops.k.quant_fp8_1x128(x, xq, sx)
    xd = xq.view(torch.float8_e4m3fn).float().view(T, K // 128, 128) * sx[:, :, None]
    wd = wq.view(torch.float8_e4m3fn).float().view(N // 128, 128, K // 128, 128) * sw[:, None, :, None]
    badd = bias.float() if bias is not None else 0
    ref = xd.view(T, K) @ wd.view(N, K).t() + badd
    _close(y, ref, 1e-2)
    _close(y, x.float() @ w.float().t() + badd, 8e-2)
    # the activation quantiser itself: amax / 448 scales, values within one e4m3 step
    amax = x.float().view(T, K // 128, 128).abs().amax(-1).clamp_min(1e-10)
    assert torch.allclose(sx, amax / 448.0, rtol=1e-6)
    assert ops.check_status() == 0


@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp4"])
@pytest.mark.parametrize("T", [1, 16, 33, 64, 100, 128, 300])
@pytest.mark.parametrize("N,K", [(256, 256), (1000, 320), (1024, 4096), (6144, 4096), (512, 12288)])
def test_linear_w4a16(ops, fmt, T, N, K):
    """Packed FP4 weights x bf16 activations against fp32 math on the de-quantised matrix (the
    expansion inside the kernel is exact, so only accumulation order and output rounding differ).
    Covers partial feature tiles, every token-tile width, the split-K path (few feature tiles,
    long K) and the expand-then-dense route of long steps."""
    from fllm_b200.ops.fp4 import Fp4Weight
    if fmt == "mxfp4" and K % 32:
        pytest.skip("block of 32")
    x = _rand((T, K), 1)
    w = _rand((N, K), 2, 0.05)
    bias = _rand((N,), 3, 0.1) if N == 1024 else None
    q = Fp4Weight.from_dense(w, fmt)
    y = ops.linear(x, q, bias)
    ref = x.float() @ q.dense().t()
    if bias is not None:
        ref = ref + bias.float()
    _close(y, ref, 1e-2)
    # FP4 itself: block-scaled e2m1 keeps the product within ~10 % of the unquantised one
    _close(y, x.float() @ w.float().t() + (bias.float() if bias is not None else 0), 0.2)
    assert ops.check_status() == 0


def test_w4_dequant_matches_reference(ops):
    from fllm_b200.ops.fp4 import Fp4Weight
    for fmt in ("nvfp4", "mxfp4"):
        w = _rand((384, 512), 5, 0.3)
        q = Fp4Weight.from_dense(w, fmt)
        out = torch.empty(384, 512, dtype=torch.bfloat16, device="cuda")
        ops.k.w4_dequant(q.codes, q.scales, q.fmt, q.alpha, out)
        assert torch.equal(out.float(), q.dense().to(torch.bfloat16).float())


@pytest.mark.parametrize("T", [1, 16, 33, 64, 128, 300])
@pytest.mark.parametrize("N,K", [(256, 256), (1000, 320), (6144, 4096), (512, 12288)])
def test_linear_int4_group_affine(ops, T, N, K):
    """INT4 codes with a (scale, min) pair per 32 values (the device form of Q4_K / Q4_0 / AWQ): the
    packed GEMM against fp32 math on the matrix the kernel expands to (bf16 of q * s - m)."""
    from fllm_b200.ops.int4 import Int4Weight
    x = _rand((T, K), 1)
    w = _rand((N, K), 2, 0.05)
    q = Int4Weight.from_dense(w)
    y = ops.linear(x, q)
    ref = x.float() @ q.dense().to(torch.bfloat16).float().t()
    _close(y, ref, 1e-2)
    _close(y, x.float() @ w.float().t(), 0.15)
    assert ops.check_status() == 0


def test_int4_from_q4_k_file_blocks(ops):
    """Q4_K super-blocks as a GGUF file stores them -> device form -> packed GEMM, against the
    native codec's de-quantisation."""
    import numpy as np
    from fllm_b200.formats import quant as Q
    from fllm_b200.ops.int4 import Int4Weight
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((384, 1024)) * 0.05).astype(np.float32)
    raw = Q.quantize(w, Q.Q4_K)
    want = torch.from_numpy(Q.dequantize(raw, Q.Q4_K, 384, 1024)).cuda()
    q = Int4Weight.from_gguf("Q4_K", raw, 384, 1024, device="cuda")
    x = _rand((20, 1024), 3)
    _close(ops.linear(x, q), x.float() @ want.t(), 2e-2)


@pytest.mark.parametrize("ranks,T,E,k", [(2, 24, 8, 2), (4, 40, 16, 4), (4, 7, 8, 4)])
def test_expert_parallel_all_to_all_emulated(ops, ranks, T, E, k):
    """Dispatch / return over peer buffers with `ranks` virtual ranks on one GPU (their kernels run
    phase by phase, never waiting on each other): every rank's rows, routed to experts held by other
    ranks and back, must equal the fp32 oracle computed with all experts local. Run twice to cover
    the counter reset and the monotonic flags."""
    from types import SimpleNamespace
    from fllm_b200.comm.ep_a2a import EpAllToAll, moe_ffn_a2a_phases
    from fllm_b200.config import ModelConfig
    from fllm_b200.models.moe import moe_reference
    from fllm_b200.models.weights import LayerWeights
    H, I = 256, 128
    cfg = ModelConfig(hidden_size=H, num_experts=E, experts_per_token=k, moe_intermediate_size=I, act="swiglu_oai",
                      expert_bias=True)
    full = LayerWeights(attn_norm=None, wqkv=None, wo=None, ffn_norm=None)
    full.router_w, full.router_b = _rand((E, H), 1, 0.2), _rand((E,), 2, 0.1)
    full.exp_gate_up, full.exp_gate_up_b = _rand((E, 2 * I, H), 3, 0.05), _rand((E, 2 * I), 4, 0.1)
    full.exp_down, full.exp_down_b = _rand((E, H, I), 5, 0.05), _rand((E, H), 6, 0.1)
    per = E // ranks
    shards = []
    for r in range(ranks):
        lw = LayerWeights(attn_norm=None, wqkv=None, wo=None, ffn_norm=None)
        lw.router_w, lw.router_b = full.router_w, full.router_b
        sl = slice(r * per, (r + 1) * per)
        lw.exp_gate_up, lw.exp_gate_up_b = full.exp_gate_up[sl].contiguous(), full.exp_gate_up_b[sl].contiguous()
        lw.exp_down, lw.exp_down_b = full.exp_down[sl].contiguous(), full.exp_down_b[sl].contiguous()
        shards.append(lw)
    eps = EpAllToAll.local_group(ranks, H, per, max_tokens=64, k=k)
    dec = SimpleNamespace(cfg=cfg, ops=ops, act_kind=2)
    for round_ in range(2):
        hs = [_rand((T, H), 10 + 7 * round_ + r) for r in range(ranks)]
        gens = [moe_ffn_a2a_phases(dec, shards[r], eps[r], hs[r]) for r in range(ranks)]
        assert [next(g) for g in gens] == ["dispatched"] * ranks
        assert [next(g) for g in gens] == ["returned"] * ranks
        outs = [next(g) for g in gens]
        torch.cuda.synchronize()
        for r in range(ranks):
            _close(outs[r], moe_reference(cfg, full, hs[r], 0), 3e-2)
            assert eps[r].check_status() == 0
    assert ops.check_status() == 0


def test_cluster_splitk_reduction_opt_in():
    """The on-chip split-K reduction (thread-block cluster + distributed shared memory) is opt-in through
    the environment, which the library reads once: run it in a child process against fp32 math."""
    import os
    import subprocess
    import sys
    code = (
        "import torch\n"
        "from fllm_b200.ops.native import NativeOps\n"
        "ops = NativeOps(torch.device('cuda:0'))\n"
        "g = torch.Generator(device='cuda').manual_seed(0)\n"
        "worst = 0.0\n"
        "for T, N, K in ((1, 4096, 4096), (33, 4096, 12288), (64, 6144, 4096), (128, 1000, 2048)):\n"
        "    x = torch.randn(T, K, generator=g, device='cuda').to(torch.bfloat16)\n"
        "    w = (torch.randn(N, K, generator=g, device='cuda') * 0.05).to(torch.bfloat16)\n"
        "    b = torch.randn(N, generator=g, device='cuda').to(torch.bfloat16)\n"
        "    y = ops.linear(x, w, b)\n"
        "    r = x.float() @ w.float().t() + b.float()\n"
        "    worst = max(worst, ((y.float() - r).abs().max() / r.abs().max()).item())\n"
        "    assert ops.launches >= 1\n"
        "print('WORST', worst, 'STATUS', ops.check_status(), 'LAUNCHES', ops.launches)\n")
    env = dict(os.environ, FLLM_CLUSTER_SPLITK="1", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [l for l in out.stdout.splitlines() if l.startswith("WORST")][-1].split()
    assert float(line[1]) < 1e-2 and int(line[3]) == 0
    assert int(line[5]) == 4          # one launch per product: no separate reduction kernel ran


@pytest.mark.parametrize("style", [0, 1])
def test_fp8_kv_write_and_generic_attention_read(ops, ref, style):
    """e4m3 KV cache: the rope kernel's stores equal PyTorch's float8 rounding of the same values, and
    the generic attention kernel on that cache equals the fp32 oracle reading the same bytes."""
    T, hq, hkv, D, bs, nb = 40, 8, 2, 128, 16, 8
    qkv = _rand((T, (hq + 2 * hkv) * D), 1)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    slots = torch.arange(T, device="cuda", dtype=torch.int32)
    inv = (10000.0 ** (-torch.arange(0, D, 2, device="cuda").float() / D))
    kc = torch.zeros(nb, hkv, bs, D, dtype=torch.float8_e4m3fn, device="cuda")
    vc = torch.zeros_like(kc)
    kc_r, vc_r, qkv_r = kc.clone(), vc.clone(), qkv.clone()
    ops.rope_kv_write(qkv, pos, slots, inv, None, None, kc, vc, hq, hkv, D, D, style, 1e-6, 1.0)
    ref.rope_kv_write(qkv_r, pos, slots, inv, None, None, kc_r, vc_r, hq, hkv, D, D, style, 1e-6, 1.0)
    assert torch.equal(vc.view(torch.uint8), vc_r.view(torch.uint8))
    # keys pass through sin/cos in fp32 on both sides: allow one e4m3 step on a few elements
    dk = (kc.float() - kc_r.float()).abs()
    assert (dk > 0).float().mean().item() < 0.02 and dk.max().item() <= 0.13 * kc_r.float().abs().max().item()
    tables = torch.arange(nb, device="cuda", dtype=torch.int32).view(1, nb)
    row_seq = torch.zeros(T, device="cuda", dtype=torch.int32)
    q = qkv[:, : hq * D].contiguous()
    got = ops.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5)
    want = ref.attention(q, kc, vc, tables, row_seq, pos, hq, hkv, D, D ** -0.5)
    _close(got, want, 2e-2)


@pytest.mark.parametrize("T,E,k,H,I", [(5, 8, 4, 256, 256), (64, 32, 4, 512, 384), (300, 16, 2, 256, 128)])
def test_moe_with_packed_mxfp4_experts(ops, T, E, k, H, I):
    """Expert stacks held as MXFP4 (the way gpt-oss checkpoints store them) through the grouped packed GEMM,
    against the fp32 oracle on the de-quantised experts."""
    from types import SimpleNamespace
    from fllm_b200.config import ModelConfig
    from fllm_b200.models.moe import _dense_experts, moe_ffn, moe_reference
    from fllm_b200.models.weights import LayerWeights
    from fllm_b200.ops.fp4 import Fp4ExpertStack
    cfg = ModelConfig(hidden_size=H, num_experts=E, experts_per_token=k, moe_intermediate_size=I, act="swiglu_oai",
                      expert_bias=True)
    lw = LayerWeights(attn_norm=None, wqkv=None, wo=None, ffn_norm=None)
    lw.router_w, lw.router_b = _rand((E, H), 1, 0.2), _rand((E,), 2, 0.1)
    lw.exp_gate_up = Fp4ExpertStack.from_dense(_rand((E, 2 * I, H), 3, 0.05))
    lw.exp_gate_up_b = _rand((E, 2 * I), 4, 0.1)
    lw.exp_down = Fp4ExpertStack.from_dense(_rand((E, H, I), 5, 0.05))
    lw.exp_down_b = _rand((E, H), 6, 0.1)
    h = _rand((T, H), 7)
    dec = SimpleNamespace(cfg=cfg, ops=ops, act_kind=2, spec=SimpleNamespace(expert_parallel=False, expert_start=0))
    got = moe_ffn(dec, lw, h)
    want = moe_reference(cfg, _dense_experts(lw), h, 0)
    _close(got, want, 3e-2)
    assert ops.check_status() == 0


class _Canary:
    """Tensors carved out of a larger buffer whose margins hold a sentinel: any kernel that stores outside
    its output shows up as a changed margin (the role a memory checker would play)."""
    PAD = 4096

    def __init__(self):
        self.bufs = []

    def empty(self, shape, dtype=torch.bfloat16):
        n = 1
        for d in shape:
            n *= d
        esz = torch.empty(0, dtype=dtype).element_size()
        raw = torch.full((n * esz + 2 * self.PAD,), 0xA5, dtype=torch.uint8, device="cuda")
        self.bufs.append((raw, n * esz))
        return raw[self.PAD: self.PAD + n * esz].view(dtype).view(*shape)

    def check(self):
        for raw, nbytes in self.bufs:
            assert bool((raw[: self.PAD] == 0xA5).all()) and bool((raw[self.PAD + nbytes:] == 0xA5).all()), "out-of-bounds store"


@pytest.mark.parametrize("T", [1, 7, 33, 64, 100, 129, 300])
def test_kernels_never_store_outside_their_outputs(ops, T):
    """Odd row counts and widths that leave partial tiles, outputs placed between sentinel margins."""
    from fllm_b200.ops.fp4 import Fp4Weight
    from fllm_b200.ops.int4 import Int4Weight
    c = _Canary()
    N, K = 1000, 320
    x, w = _rand((T, K), 1), _rand((N, K), 2, 0.05)
    for splits in (0, 3):
        ops.linear(x, w, out=c.empty((T, N)), force_splits=splits)
    ops.linear(x[:, :256].contiguous(), Fp4Weight.from_dense(w[:, :256].contiguous(), "mxfp4"), out=c.empty((T, N)))
    ops.linear(x[:, :256].contiguous(), Int4Weight.from_dense(w[:, :256].contiguous()), out=c.empty((T, N)))
    H = 1376
    y = c.empty((T, H))
    ops.k.rmsnorm(_rand((T, H), 3), _rand((T, H), 4), _rand((H,), 5), y, 1e-6, 0.0)
    g = c.empty((T, H // 2))
    ops.k.glu(_rand((T, H), 6), g, 0, 1.702, 7.0)
    ids, vals = c.empty((T,), torch.int32), c.empty((T,), torch.float32)
    ops.k.argmax(_rand((T, 1003), 7), ids, vals, 0)
    # paged attention + KV write on odd lengths
    hq, hkv, D, bs, nb = 8, 2, 128, 16, (T + 15) // 16 + 1
    kc, vc = c.empty((nb, hkv, bs, D)), c.empty((nb, hkv, bs, D))
    kc.zero_(); vc.zero_()
    qkv = _rand((T, (hq + 2 * hkv) * D), 8)
    pos = torch.arange(T, device="cuda", dtype=torch.int32)
    inv = (10000.0 ** (-torch.arange(0, D, 2, device="cuda").float() / D))
    ops.rope_kv_write(qkv, pos, pos.clone(), inv, None, None, kc, vc, hq, hkv, D, D, 0, 1e-6, 1.0)
    out = c.empty((T, hq * D))
    tables = torch.arange(nb, device="cuda", dtype=torch.int32).view(1, nb)
    ops.k.attention_generic(qkv[:, : hq * D].contiguous(), kc, vc, tables, torch.zeros(T, device="cuda", dtype=torch.int32),
                            pos, out, hq, hkv, D, D ** -0.5, 0, None, 0.0)
    torch.cuda.synchronize()
    c.check()
    assert ops.check_status() == 0


@pytest.mark.parametrize("fmt", ["int4g", "mxfp4", "nvfp4"])
@pytest.mark.parametrize("T", [1, 2, 3, 4])
@pytest.mark.parametrize("N,K", [(256, 256), (1000, 320), (6144, 4096), (520, 12288)])
def test_gemv_w4_dp4a(ops, fmt, T, N, K):
    """The few-token path of the packed 4-bit weights (dp4a on int8 activations quantised per 32 values inside the
    kernel) against fp32 math on the same quantised activations and the dequantised weights."""
    from fllm_b200.ops.fp4 import Fp4Weight
    from fllm_b200.ops.int4 import Int4Weight
    x = _rand((T, K), 11 + T)
    w = _rand((N, K), 12, 0.05)
    bias = _rand((N,), 13) if T % 2 == 0 else None
    if fmt == "int4g":
        q = Int4Weight.from_dense(w)
        dense = q.dense().float()
        y = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
        ops.k.gemv_w4(x, q.codes, q.sm.view(torch.uint8).view(N, -1), 2, 1.0, bias, y)
    else:
        q = Fp4Weight.from_dense(w, fmt)
        dense = q.dense().float()
        y = torch.empty(T, N, dtype=torch.bfloat16, device="cuda")
        ops.k.gemv_w4(x, q.codes, q.scales, q.fmt, q.alpha, bias, y)
    xb = x.float().view(T, K // 32, 32)
    d = xb.abs().amax(-1, keepdim=True) / 127.0
    xq = torch.where(d > 0, torch.round(xb / d.clamp_min(1e-30)), torch.zeros_like(xb)) * d
    ref = xq.view(T, K) @ dense.t() + (bias.float() if bias is not None else 0)
    _close(y, ref, 1e-2)
    _close(y, x.float() @ dense.t() + (bias.float() if bias is not None else 0), 3e-2)
    # the weight classes take this path by themselves for up to 4 tokens
    y2 = ops.linear(x, q, bias)
    assert torch.equal(y2, y)
    assert ops.check_status() == 0


@pytest.mark.parametrize("D,hq,hkv", [(128, 8, 2), (64, 8, 8), (128, 32, 8), (64, 16, 2)])
@pytest.mark.parametrize("window,sinks,softcap", [(0, False, 0.0), (40, True, 0.0), (0, False, 30.0)])
@pytest.mark.parametrize("case", ["decode", "decode_few", "verify"])
def test_attention_tc_decode_reads_e4m3_cache(ops, ref, D, hq, hkv, window, sinks, softcap, case):
    """An e4m3 KV pool through the tensor-core decode kernel (pages widened to f16 in shared memory) against the
    fp32 reference on the same e4m3 values, and against the generic kernel."""
    if case == "decode":
        kv_lens, q_lens = [1, 17, 64, 130, 700, 33, 16, 257], [1] * 8
    elif case == "decode_few":
        kv_lens, q_lens = [900, 35], [1, 1]
    else:
        n = max(1, min(4, 16 // (hq // hkv)))
        kv_lens, q_lens = [100, 37, 260], [n, n, n]
    tables, kc, vc = _paged_setup(len(kv_lens), kv_lens, hkv, D, seed=3)
    kc8, vc8 = kc.to(torch.float8_e4m3fn), vc.to(torch.float8_e4m3fn)
    T = sum(q_lens)
    row_seq = torch.tensor([i for i, n in enumerate(q_lens) for _ in range(n)], dtype=torch.int32, device="cuda")
    pos = torch.tensor([kv - n + j for kv, n in zip(kv_lens, q_lens) for j in range(n)], dtype=torch.int32, device="cuda")
    q = _rand((T, hq * D), 5)
    sk = torch.randn(hq, device="cuda") if sinks else None
    meta = _tc_meta(q_lens, kv_lens)
    l0 = ops.launches
    y = ops.attention(q, kc8, vc8, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap, meta=meta)
    assert ops.launches - l0 in (1, 2)                       # decode kernel (+ merge), not the generic one's count of 1 only
    yr = ref.attention(q, kc8.to(torch.bfloat16), vc8.to(torch.bfloat16), tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap)
    _close(y, yr, 2e-2)
    yg = ops.attention(q, kc8, vc8, tables, row_seq, pos, hq, hkv, D, D ** -0.5, window, sk, softcap)
    _close(yg, y, 2e-2)
    assert ops.check_status() == 0


@pytest.mark.parametrize("T", [256, 300, 1024, 2048])
@pytest.mark.parametrize("N,K", [(512, 512), (4096, 4096), (1000, 320), (6144, 4096), (256, 12288)])
def test_linear_on_cta_pairs(ops, T, N, K):
    """tcgen05 cta_group::2 GEMM (256 x 256 tiles over two SMs) against fp32 math: ragged token and feature edges,
    a K that is not a multiple of the stage depth, bias, several tiles per cluster."""
    x = _rand((T, K), 21)
    w = _rand((N, K), 22, 0.05)
    bias = _rand((N,), 23) if T % 512 == 0 else None
    y = torch.full((T + 2, N), 7.0, dtype=torch.bfloat16, device="cuda")     # two sentinel rows after the output
    ops.k.linear_pair(x, w, bias, y[:T], ops.status)
    ref = x.float() @ w.float().t() + (bias.float() if bias is not None else 0)
    _close(y[:T], ref, 1e-2)
    assert bool((y[T:] == 7.0).all())
    assert ops.check_status() == 0


@pytest.mark.parametrize("kind,layout", [(0, 16), (1, 16), (2, 16), (2, 0)])
def test_large_batch_linear_glu_goes_through_the_pair_kernel(ops, ref, kind, layout):
    """2048 tokens x a gate|up matrix: the planner picks the CTA-pair kernel and its epilogue applies the gated
    activation (blocked-16 and pairwise layouts)."""
    T, N, K = 2048, 4096, 1024
    x = _rand((T, K), 31)
    w = _rand((N, K), 32, 0.05)
    bias = _rand((N,), 33)
    y = ops.linear_glu(x, w, bias, kind, 1.702, 7.0, layout)
    yr = ref.linear_glu(x, w, bias, kind, 1.702, 7.0, layout)
    _close(y, yr, 2e-2)
    assert ops.check_status() == 0


@pytest.mark.parametrize("qname", ["Q5_K", "Q6_K", "Q8_0"])
@pytest.mark.parametrize("T", [1, 2, 4, 9])
@pytest.mark.parametrize("N,K", [(256, 256), (1000, 512), (4096, 4096), (520, 12288)])
def test_packed_5_6_8_bit_weights(ops, qname, T, N, K):
    """Q5_K / Q6_K / Q8_0 in their planar device form: the dp4a product (up to 4 tokens) against fp32 math on the
    int8-quantised activations, the bf16 expansion bit for bit against the codec, longer steps through the GEMM."""
    import numpy as np
    from fllm_b200.formats import quant as Q
    from fllm_b200.ops.intk import IntKWeight
    rng = np.random.default_rng(N + K + T)
    w = (rng.standard_normal((N, K)) * 0.05).astype(np.float32)
    tid = {"Q5_K": Q.Q5_K, "Q6_K": Q.Q6_K, "Q8_0": Q.Q8_0}[qname]
    raw = Q.quantize(w, tid)
    dense = torch.from_numpy(Q.dequantize(raw, tid, N, K)).cuda()
    q = IntKWeight.from_gguf(qname, raw, N, K, device="cuda")
    assert abs(q.nbytes() * 8 / (N * K) - {"Q5_K": 5.625, "Q6_K": 6.5625, "Q8_0": 8.5}[qname]) < 0.01
    out = torch.empty(N, K, dtype=torch.bfloat16, device="cuda")
    ops.k.wk_dequant(q.codes, q.high, q.sub, q.sup, q.fmt, out)
    assert torch.equal(out.float(), dense.to(torch.bfloat16).float())
    x = _rand((T, K), 41 + T)
    bias = _rand((N,), 42) if T % 2 == 0 else None
    y = ops.linear(x, q, bias)
    if T <= 4:
        xb = x.float().view(T, K // 32, 32)
        d = xb.abs().amax(-1, keepdim=True) / 127.0
        xq = torch.where(d > 0, torch.round(xb / d.clamp_min(1e-30)), torch.zeros_like(xb)) * d
        _close(y, xq.view(T, K) @ dense.t() + (bias.float() if bias is not None else 0), 1e-2)
    _close(y, x.float() @ dense.t() + (bias.float() if bias is not None else 0), 3e-2)
    assert ops.check_status() == 0


@pytest.mark.parametrize("D,heads", [(64, 12), (128, 8), (64, 4)])
@pytest.mark.parametrize("lens", [[5, 12, 33], [200, 64, 130, 17], [700, 300]])
def test_bidirectional_attention_for_encoders(ops, ref, D, heads, lens):
    """No causal mask: every query row of a packed sequence sees the whole sequence. The tensor-core prefill kernels
    (tcgen05 for long rows, mma.sync for short ones) with the flag, and the generic kernel through the visibility
    limit alone, against the fp32 reference."""
    tables, kc, vc = _paged_setup(len(lens), lens, heads, D, seed=9)
    T = sum(lens)
    row_seq = torch.tensor([i for i, n in enumerate(lens) for _ in range(n)], dtype=torch.int32, device="cuda")
    vis = torch.tensor([n - 1 for n in lens for _ in range(n)], dtype=torch.int32, device="cuda")
    q = _rand((T, heads * D), 6)
    meta = _tc_meta(lens, lens)
    y = ops.attention(q, kc, vc, tables, row_seq, vis, heads, heads, D, D ** -0.5, meta=meta, bidirectional=True)
    yr = ref.attention(q, kc, vc, tables, row_seq, vis, heads, heads, D, D ** -0.5)
    _close(y, yr, 2e-2)
    yg = ops.attention(q, kc, vc, tables, row_seq, vis, heads, heads, D, D ** -0.5)       # generic kernel
    _close(yg, yr, 2e-2)
    # the causal result differs (the flag really changes the mask)
    pos = torch.tensor([j for n in lens for j in range(n)], dtype=torch.int32, device="cuda")
    yc = ops.attention(q, kc, vc, tables, row_seq, pos, heads, heads, D, D ** -0.5, meta=meta)
    assert (yc.float() - y.float()).abs().max().item() > 1e-2
    assert ops.check_status() == 0


@pytest.mark.parametrize("D,hq,hkv", [(128, 8, 2), (64, 8, 8)])
def test_tree_attention_kernel(ops, ref, D, hq, hkv):
    """Draft-tree rows (context + ancestors through a 64-bit mask per row) on the generic kernel against the
    reference; two sequences with different trees and contexts, a 64-node tree among them."""
    from fllm_b200.runtime.speculative import DraftTree
    trees = [DraftTree.from_chains([[5, 6, 7], [5, 9], [4, 4, 4]]),
             DraftTree(list(range(64)), [-1] + [i // 2 for i in range(63)])]
    ctxs = [37, 130]
    kv_lens = [c + len(t) for c, t in zip(ctxs, trees)]
    tables, kc, vc = _paged_setup(2, kv_lens, hkv, D, seed=4)
    rows = sum(len(t) for t in trees)
    row_seq = torch.tensor([i for i, t in enumerate(trees) for _ in range(len(t))], dtype=torch.int32, device="cuda")
    pos = torch.tensor([kv_lens[i] - 1 for i, t in enumerate(trees) for _ in range(len(t))], dtype=torch.int32, device="cuda")
    base = torch.tensor([ctxs[i] for i, t in enumerate(trees) for _ in range(len(t))], dtype=torch.int32, device="cuda")
    mask = torch.tensor([m for t in trees for m in t.masks_i64()], dtype=torch.int64, device="cuda")
    q = _rand((rows, hq * D), 8)
    y = ops.attention_tree(q, kc, vc, tables, row_seq, pos, mask, base, hq, hkv, D, D ** -0.5)
    yr = ref.attention_tree(q, kc, vc, tables, row_seq, pos, mask, base, hq, hkv, D, D ** -0.5)
    _close(y, yr, 2e-2)


def test_logit_softcap_kernel():
    from fllm_b200.ops.native import NativeOps
    ops = NativeOps(torch.device("cuda"))
    x = (torch.randn(7, 1001, device="cuda") * 40).bfloat16()
    view = torch.empty(7, 1010, device="cuda", dtype=torch.bfloat16)[:, :1001]
    view.copy_(x)
    want = (30.0 * torch.tanh(x.float() / 30.0))
    ops.softcap_(view, 30.0)
    assert (view.float() - want).abs().max().item() <= 0.13          # bf16 steps near +-30


@pytest.mark.parametrize("cols,bias,delta", [(256, True, True), (5120, False, True), (770, True, False)])
def test_add_layernorm_and_activations(cols, bias, delta):
    from fllm_b200.ops.native import NativeOps
    from fllm_b200.ops.reference import RefOps
    nat, ref = NativeOps(torch.device("cuda")), RefOps()
    g = torch.Generator(device="cuda").manual_seed(cols)
    x = torch.randn(37, cols, device="cuda", generator=g).bfloat16()
    d = torch.randn(37, cols, device="cuda", generator=g).bfloat16() if delta else None
    w = (1 + 0.3 * torch.randn(cols, device="cuda", generator=g)).bfloat16()
    b = torch.randn(cols, device="cuda", generator=g).bfloat16() if bias else None
    x1, x2 = x.clone(), x.clone()
    y1 = nat.layernorm(x1, d, w, b, 1e-5, 1.0)
    y2 = ref.layernorm(x2, d, w, b, 1e-5, 1.0)
    assert torch.equal(x1, x2)                                          # the residual update is the same bf16 sum
    assert (y1.float() - y2.float()).abs().max().item() <= 0.05
    for kind in ("gelu", "gelu_tanh", "relu2", "silu", "relu"):
        a = (torch.randn(9, cols, device="cuda", generator=g) * 2).bfloat16()
        want = ref.act_(a.clone(), kind)
        got = nat.act_(a.clone(), kind)
        assert (got.float() - want.float()).abs().max().item() <= 0.04 * max(1.0, want.float().abs().max().item())


@pytest.mark.parametrize("kind,E,k,bias,norm", [("deepseek_v2", 64, 6, False, False), ("deepseek_v3", 128, 8, True, True),
                                                 ("deepseek_v2", 60, 4, True, True), ("deepseek_v3", 8, 2, False, False)])
def test_score_weighted_router_kernel(kind, E, k, bias, norm):
    """The router kernel of the DeepSeek / GLM-4.5 / ERNIE 4.5 families against the same rule in tensor operations."""
    from fllm_b200.config import ModelConfig
    from fllm_b200.models.moe import route_deepseek
    from fllm_b200.ops.native import NativeOps
    ops = NativeOps(torch.device("cuda"))
    cfg = ModelConfig(num_experts=E, experts_per_token=k, router_kind=kind, router_scale=2.5, router_norm_topk=norm)
    g = torch.Generator(device="cuda").manual_seed(E + k)
    Ep = (E + 7) // 8 * 8
    logits = (torch.randn(77, Ep, device="cuda", generator=g) * 3).bfloat16()[:, :E]       # a view with a wider pitch
    sb = (torch.randn(E, device="cuda", generator=g) * 0.2) if bias else None
    want_ids, want_w = route_deepseek(cfg, logits, sb)
    ids = torch.empty(77, k, dtype=torch.int32, device="cuda")
    w = torch.empty(77, k, dtype=torch.float32, device="cuda")
    ops.k.moe_route_scored(logits, sb, k, 2 if kind == "deepseek_v3" else 1, norm, 2.5, ids, w)
    so, sw = ids.long().sort(1), want_ids.long().sort(1)
    same = (so.values == sw.values).all(1)
    assert int((~same).sum()) <= 1                                   # a tie between two experts may resolve differently
    a = torch.gather(w, 1, so.indices)[same]
    b = torch.gather(want_w, 1, sw.indices)[same]
    assert float((a - b).abs().max()) < 2e-3 * float(b.abs().max())
