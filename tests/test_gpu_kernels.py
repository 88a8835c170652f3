"""Each CUDA kernel alone against a plain torch float32 statement of the same operation, at sizes other
than the engine's tiny configurations (odd widths, tails, empty groups, window edges)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def K():
    from cpi_b200.csrc import lib
    return lib


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# ------------------------------------------------------------------------------------------------ rows
@pytest.mark.parametrize("H,tdt", [(70, torch.bfloat16), (1000, torch.float32)])
def test_embedding(H, tdt):
    V, T = 37, 9
    table = rnd(V, H, dtype=tdt)
    toks = torch.tensor([0, 36, 5, 5, 17, 1, 2, 3, 36], dtype=torch.int32, device=DEV)
    out = torch.empty(T, H, device=DEV)
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().embedding(toks, table, out, err)
    assert torch.equal(out, table[toks.long()].float()) and int(err) == 0
    toks[4] = 37
    K().embedding(toks, table, out, err)
    assert int(err) == 5 and float(out[4].abs().sum()) == 0


@pytest.mark.parametrize("n,xdt,odt,wdt", [(5120, torch.float32, torch.bfloat16, torch.bfloat16),
                                           (100, torch.float32, torch.float32, torch.float32),
                                           (48, torch.bfloat16, torch.bfloat16, None)])
def test_rmsnorm(n, xdt, odt, wdt):
    x = rnd(7, n, dtype=xdt, scale=3.0)
    w = None if wdt is None else rnd(n, dtype=wdt, seed=1)
    out = torch.empty(7, n, dtype=odt, device=DEV)
    K().rmsnorm(x, w, 1e-6, out)
    xf = x.float()
    ref = xf / torch.sqrt((xf * xf).mean(-1, keepdim=True) + 1e-6)
    if w is not None:
        ref = ref * w.float()
    tol = 1e-5 if odt == torch.float32 else 1e-2
    assert torch.allclose(out.float(), ref, atol=tol * float(ref.abs().max()))
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, n, dtype=odt, device=DEV)
    K().rmsnorm(x, w, 1e-6, out2, rows)
    assert torch.equal(out2, out[rows.long()])


# ------------------------------------------------------------------------------------------------ GEMM
def ref_gemm(a, w, mode, out0=None, row_scale=None):
    acc = a.float() @ w.float().T
    if row_scale is not None:
        acc = acc * row_scale[:, None]
    if mode == 2:
        n = w.shape[0] // 2
        g, u = acc[:, :n], acc[:, n:]
        return g / (1 + torch.exp(-g)) * u
    return acc if mode == 0 else out0 + acc


@pytest.mark.parametrize("M,N,Kd", [(1, 7, 5), (13, 70, 33), (64, 64, 16), (100, 200, 300)])
@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.float32, torch.bfloat16),
                                     (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32)])
def test_gemm_fp32_pipe_modes(M, N, Kd, adt, wdt):
    a, scale = rnd(M, Kd, dtype=adt), rnd(M, seed=5).abs()
    for mode in (0, 1, 2):
        w = rnd(2 * N if mode == 2 else N, Kd, dtype=wdt, seed=2)
        out = rnd(M, N, seed=3)
        ref = ref_gemm(a, w, mode, out.clone(), scale)
        K().gemm_simt(a, w, out, mode, row_scale=scale)
        assert torch.allclose(out, ref, atol=2e-5 * max(1.0, float(ref.abs().max()))), (mode, float((out - ref).abs().max()))


def test_gemm_fp32_pipe_grouped_gather_scatter():
    G, N, Kd, M = 5, 40, 24, 37
    w = rnd(G, N, Kd, dtype=torch.bfloat16)
    a = rnd(50, Kd)
    counts = [0, 11, 0, 25, 1]
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    a_rows = torch.randperm(50)[:M].to(torch.int32).to(DEV)
    out_rows = torch.randperm(60)[:M].to(torch.int32).to(DEV)
    out = torch.zeros(60, N, device=DEV)
    K().gemm_simt(a, w, out, 1, m_rows=M, a_rows=a_rows, out_rows=out_rows, group_offsets=offs, n_groups=G,
                  rows_per_group_hint=8)
    ref = torch.zeros(60, N, device=DEV)
    m = 0
    for g, c in enumerate(counts):
        for _ in range(c):
            ref[out_rows[m]] += a[a_rows[m]] @ w[g].float().T
            m += 1
    assert torch.allclose(out, ref, atol=1e-5 * float(ref.abs().max()))


TC_SHAPES = [(1, 128, 64), (8, 256, 512), (8, 7168, 5120), (17, 200, 200), (64, 5120, 8192), (100, 384, 1024),
             (300, 640, 264), (2048, 1024, 512)]


@pytest.mark.parametrize("T,N,Kd", TC_SHAPES)
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_tensor_core_modes(T, N, Kd, mode):
    a = rnd(T, Kd, dtype=torch.bfloat16)
    w = rnd(2 * N if mode == 2 else N, Kd, dtype=torch.bfloat16, seed=2, scale=Kd ** -0.5)
    scale = rnd(T, seed=5).abs()
    for odt in ([torch.float32] if mode == 1 else [torch.bfloat16] if mode == 2 else [torch.bfloat16, torch.float32]):
        out = rnd(T, N, dtype=odt, seed=3)
        ref = ref_gemm(a, w, mode, out.float().clone(), scale)
        assert K().gemm_tc(a, w, out, mode, row_scale=scale)
        torch.cuda.synchronize()
        assert int(K().tc_error_flag(DEV)) == 0
        tol = (2e-5 if odt == torch.float32 else 1e-2) * max(1.0, float(ref.abs().max()))
        err = float((out.float() - ref).abs().max())
        assert err <= tol, (odt, err, tol)


@pytest.mark.parametrize("persistent", [True, False])
@pytest.mark.parametrize("T,N,Kd", [(512, 256, 64), (2048, 1024, 512), (700, 512, 200), (1000, 768, 1032), (4096, 5120, 256),
                                    (5000, 2048, 1024)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_tensor_core_pair_kernel(T, N, Kd, mode, persistent):
    """Two CTAs on one tile: every mode, token tails that are no multiple of 32, k tails; as a pair per SM
    pair that works through the tiles (more tiles than pairs in the last shape) and as a launch slot per tile."""
    K().gemm_pair_persistent(persistent)
    try:
        _pair_kernel_case(T, N, Kd, mode)
    finally:
        K().gemm_pair_persistent(1)


def _pair_kernel_case(T, N, Kd, mode):
    a = rnd(T, Kd, dtype=torch.bfloat16)
    w = rnd(2 * N if mode == 2 else N, Kd, dtype=torch.bfloat16, seed=2, scale=Kd ** -0.5)
    scale = rnd(T, seed=5).abs()
    for odt in ([torch.float32] if mode == 1 else [torch.bfloat16] if mode == 2 else [torch.bfloat16, torch.float32]):
        out = rnd(T, N, dtype=odt, seed=3)
        ref = ref_gemm(a, w, mode, out.float().clone(), scale)
        assert K().gemm_tc_pair(a, w, out, mode, row_scale=scale)
        torch.cuda.synchronize()
        assert int(K().tc_error_flag(DEV)) == 0
        tol = (2e-5 if odt == torch.float32 else 1e-2) * max(1.0, float(ref.abs().max()))
        err = float((out.float() - ref).abs().max())
        assert err <= tol, (odt, err, tol)
    assert not K().gemm_tc_pair(a[:100], w, out[:100], mode)                # too few tokens
    if N % 256 == 0:
        wn = w[: (2 * (N - 128) if mode == 2 else N - 128)].contiguous()
        assert not K().gemm_tc_pair(a, wn, out[:, : N - 128], mode)         # features no multiple of 256


@pytest.mark.parametrize("persistent", [2, 0])
@pytest.mark.parametrize("counts", [[300, 0, 129, 83], [128, 128, 128, 128, 1, 255, 256, 0], [700, 3, 0, 0, 513, 64]])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_tensor_core_pair_kernel_grouped(counts, mode, persistent):
    K().gemm_pair_persistent(persistent)
    try:
        _pair_kernel_grouped_case(counts, mode)
    finally:
        K().gemm_pair_persistent(1)


def _pair_kernel_grouped_case(counts, mode):
    G, N, Kd = len(counts), 512, 320
    M = sum(counts)
    w = rnd(G, 2 * N if mode == 2 else N, Kd, dtype=torch.bfloat16, seed=1, scale=Kd ** -0.5)
    a = rnd(M, Kd, dtype=torch.bfloat16)
    scale = rnd(M, seed=4).abs()
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    grp = torch.repeat_interleave(torch.arange(G), torch.tensor(counts)).to(DEV)
    acc = torch.einsum("mk,mnk->mn", a.float(), w.float()[grp]) * scale[:, None]
    if mode == 1:
        out_rows = torch.randperm(M + 10)[:M].to(torch.int32).to(DEV)
        out = rnd(M + 10, N, seed=7)
        ref = out.clone()
        ref[out_rows.long()] += acc
    elif mode == 2:
        out_rows, out = None, torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        g_, u_ = acc[:, :N], acc[:, N:]
        ref = g_ / (1 + torch.exp(-g_)) * u_
    else:
        out_rows, out, ref = None, torch.zeros(M, N, device=DEV), acc
    assert K().gemm_tc_pair(a, w, out, mode, m_rows=M, out_rows=out_rows, row_scale=scale, group_offsets=offs, n_groups=G)
    torch.cuda.synchronize()
    assert int(K().tc_error_flag(DEV)) == 0
    tol = (1e-2 if mode == 2 else 2e-5) * max(1.0, float(ref.abs().max()))
    assert float((out.float() - ref).abs().max()) <= tol


def test_gemm_tensor_core_refuses_what_it_cannot_take():
    a, w = rnd(4, 36, dtype=torch.bfloat16), rnd(128, 36, dtype=torch.bfloat16)
    out = torch.empty(4, 128, dtype=torch.bfloat16, device=DEV)
    assert not K().gemm_tc(a, w, out, 0)                                        # K is no multiple of 8
    a, w = rnd(4, 64), rnd(128, 64)
    assert not K().gemm_tc(a, w, torch.empty(4, 128, device=DEV), 0)            # float32 operands
    from cpi_b200.parts.linear import project                                   # the dispatcher falls back
    a, w = rnd(4, 36, dtype=torch.bfloat16), rnd(128, 36, dtype=torch.bfloat16)
    project(a, w, out)
    ref = a.float() @ w.float().T
    assert float((out.float() - ref).abs().max()) <= 1e-2 * float(ref.abs().max())


@pytest.mark.parametrize("counts,bn_rows", [([0, 3, 0, 1, 4], 8), ([40, 0, 170, 1, 0, 29], 240), ([1], 1)])
@pytest.mark.parametrize("mode", [1, 2])
def test_gemm_tensor_core_grouped(counts, bn_rows, mode):
    G, N, Kd = len(counts), 320, 256
    M = sum(counts)
    w = rnd(G, 2 * N if mode == 2 else N, Kd, dtype=torch.bfloat16, seed=1, scale=Kd ** -0.5)
    a = rnd(M + 3, Kd, dtype=torch.bfloat16)
    scale = rnd(M, seed=4).abs()
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    if mode == 1:
        out_rows = torch.randperm(M + 10)[:M].to(torch.int32).to(DEV)
        out = rnd(M + 10, N, seed=7)
        ref = out.clone()
    else:
        out_rows = None
        out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
        ref = torch.zeros(M, N, device=DEV)
    m = 0
    for g, c in enumerate(counts):
        for _ in range(c):
            r = ref_gemm(a[m:m + 1], w[g], 2 if mode == 2 else 0, None, scale[m:m + 1])[0]
            if mode == 1:
                ref[out_rows[m]] += r
            else:
                ref[m] = r
            m += 1
    assert K().gemm_tc(a, w, out, mode, m_rows=M, out_rows=out_rows, row_scale=scale, group_offsets=offs, n_groups=G)
    torch.cuda.synchronize()
    assert int(K().tc_error_flag(DEV)) == 0
    tol = (2e-5 if mode == 1 else 1e-2) * max(1.0, float(ref.abs().max()))
    assert float((out.float() - ref).abs().max()) <= tol


@pytest.mark.parametrize("T,N,Kd", [(5, 384, 1024), (16, 200, 2048), (30, 256, 1280), (64, 640, 1536),
                                    (100, 384, 2048), (128, 128, 4096)])
@pytest.mark.parametrize("mode", [0, 1, 2])
def test_gemm_tensor_core_split_k(T, N, Kd, mode):
    """Products with so few tiles that the k range is cut (the splits of a tile are a cluster and meet in its
    shared memory): the right product, and the same bits from one launch to the next."""
    a = rnd(T, Kd, dtype=torch.bfloat16)
    w = rnd(2 * N if mode == 2 else N, Kd, dtype=torch.bfloat16, seed=2, scale=Kd ** -0.5)
    scale = rnd(T, seed=5).abs()
    odt = torch.float32 if mode == 1 else torch.bfloat16
    bn, splits = K().gemm_tc_plan(T, N, Kd, 0, mode == 2)
    assert splits > 1, "the case is meant to split k"
    outs = []
    for _ in range(3):
        out = rnd(T, N, dtype=odt, seed=3)
        ref = ref_gemm(a, w, mode, out.float().clone(), scale)
        assert K().gemm_tc(a, w, out, mode, row_scale=scale)
        torch.cuda.synchronize()
        assert int(K().tc_error_flag(DEV)) == 0
        outs.append(out)
    tol = (2e-5 if odt == torch.float32 else 1e-2) * max(1.0, float(ref.abs().max()))
    assert float((outs[0].float() - ref).abs().max()) <= tol
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_gemm_tensor_core_grouped_split_k():
    """One token per expert (a decode step of batch 3 over 6 experts), the k range cut."""
    counts, N, Kd = [1, 0, 0, 1, 0, 1], 256, 2048
    G, M = len(counts), sum(counts)
    w = rnd(G, 2 * N, Kd, dtype=torch.bfloat16, seed=1, scale=Kd ** -0.5)
    a = rnd(M, Kd, dtype=torch.bfloat16)
    offs = torch.tensor([0] + list(torch.tensor(counts).cumsum(0)), dtype=torch.int32, device=DEV)
    grp = torch.repeat_interleave(torch.arange(G), torch.tensor(counts)).to(DEV)
    acc = torch.einsum("mk,mnk->mn", a.float(), w.float()[grp])
    ref = acc[:, :N] / (1 + torch.exp(-acc[:, :N])) * acc[:, N:]
    out = torch.zeros(M, N, dtype=torch.bfloat16, device=DEV)
    assert K().gemm_tc_plan(M, N, Kd, G, True)[1] > 1
    assert K().gemm_tc(a, w, out, 2, m_rows=M, group_offsets=offs, n_groups=G)
    torch.cuda.synchronize()
    assert int(K().tc_error_flag(DEV)) == 0
    assert float((out.float() - ref).abs().max()) <= 1e-2 * max(1.0, float(ref.abs().max()))


def test_a_wait_that_runs_out_raises_the_flag_and_the_next_launch_is_right():
    """A tensor-core kernel never waits without a limit.  Here one small product is launched with a poll limit
    of a few thousand and a barrier that expects 64 bytes more than its loads bring, so that the wait runs out:
    the kernel must come back by itself with the error word set (nothing faults or hangs: the loads land, the
    tensor memory is freed), `Engine.check_device_errors` must raise and clear it, and the same product launched
    again in the ordinary way must be right."""
    from cpi_b200.engine import Engine
    T, N, Kd = 16, 128, 256
    a = rnd(T, Kd, dtype=torch.bfloat16)
    w = rnd(N, Kd, dtype=torch.bfloat16, seed=2, scale=Kd ** -0.5)
    out = torch.zeros(T, N, dtype=torch.bfloat16, device=DEV)
    assert K().gemm_tc_plan(T, N, Kd)[1] == 1
    torch.cuda.synchronize()
    assert int(K().tc_error_flag(DEV)) == 0
    K().gemm_tc_wait_probe(4096, 64)
    try:
        assert K().gemm_tc(a, w, out, 0)
        torch.cuda.synchronize()
    finally:
        K().gemm_tc_wait_probe(0, 0)
    assert int(K().tc_error_flag(DEV)) == 1
    import tiny
    e = Engine.from_random(tiny.config("A"), seed=0, dtype="bfloat16", max_tokens=64)
    with pytest.raises(RuntimeError, match="gave up waiting"):
        e.check_device_errors()
    e.check_device_errors()                                   # cleared
    assert int(K().tc_error_flag(DEV)) == 0
    out.zero_()
    assert K().gemm_tc(a, w, out, 0)
    torch.cuda.synchronize()
    ref = ref_gemm(a, w, 0, out.float().clone(), None)
    assert float((out.float() - ref).abs().max()) <= 1e-2 * max(1.0, float(ref.abs().max()))
    assert int(K().tc_error_flag(DEV)) == 0


def test_gemm_tensor_core_split_k_is_deterministic():
    a, w = rnd(8, 5120, dtype=torch.bfloat16), rnd(640, 5120, dtype=torch.bfloat16, scale=0.02)
    outs = []
    for _ in range(5):
        out = torch.zeros(8, 640, device=DEV)
        assert K().gemm_tc(a, w, out, 1)
        outs.append(out)
    assert all(torch.equal(outs[0], o) for o in outs[1:])


# ------------------------------------------------------------------------------------------------ attention
def paged_cache(n_seq, lengths, NKV, D, page, dtype, seed=0):
    """Random keys/values for sequences of the given lengths scattered over shuffled pages."""
    blocks = [-(-l // page) for l in lengths]
    n_pages = sum(blocks) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(seed)).tolist()
    table = torch.zeros(n_seq + 2, max(blocks) + 1, dtype=torch.int32)
    k = rnd(n_pages, NKV, page, D, dtype=dtype, seed=seed + 1)
    v = rnd(n_pages, NKV, page, D, dtype=dtype, seed=seed + 2)
    it = iter(perm)
    for s in range(n_seq):
        for b in range(blocks[s]):
            table[s + 1, b] = next(it)          # slot = s + 1
    return k, v, table.to(DEV)


def gather_kv(cache, table, slot, n, page):
    rows = [cache[int(table[slot, t // page]), :, t % page, :] for t in range(n)]
    return torch.stack(rows).float()            # [n, NKV, D]


def ref_attention(q, k, v, pos, lo, scale):
    """q [NH, D] at position pos over keys lo..pos; k, v [n, NKV, D]."""
    NH, G = q.shape[0], q.shape[0] // k.shape[1]
    out = torch.empty_like(q)
    for h in range(NH):
        s = (k[lo:pos + 1, h // G] @ q[h]) * scale
        p = torch.softmax(s, 0)
        out[h] = p @ v[lo:pos + 1, h // G]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("NH,NKV,D,page,window", [(6, 2, 48, 16, ("full", 0)), (5, 5, 16, 64, ("chunk", 40)),
                                                  (8, 1, 256, 32, ("sliding", 33)), (12, 4, 128, 64, ("chunk", 128))])
def test_attention_general_over_pages(dtype, NH, NKV, D, page, window):
    lengths = [1, 130, 77, 300]
    k, v, table = paged_cache(len(lengths), lengths, NKV, D, page, dtype)
    # queries: the last position of each sequence, plus window edges of the longest
    qs = [(s, l - 1) for s, l in enumerate(lengths)]
    wk, wsz = window
    if wk != "full":
        qs += [(3, wsz - 1), (3, wsz), (3, wsz + 1), (3, 2 * wsz - 1), (3, 2 * wsz)]
    T = len(qs)
    q = rnd(T, NH * D, dtype=dtype, seed=9)
    out = torch.empty_like(q)
    token_seq = torch.tensor([s for s, _ in qs], dtype=torch.int32, device=DEV)
    token_pos = torch.tensor([p for _, p in qs], dtype=torch.int32, device=DEV)
    seq_slot = torch.arange(1, len(lengths) + 1, dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(D)
    K().attention_general(q, out, k, v, table, page, token_seq, token_pos, seq_slot, n_heads=NH, n_kv_heads=NKV,
                          head_dim=D, window_kind=K().WINDOW_KINDS[wk], window_size=wsz, scale=scale)
    for i, (s, pos) in enumerate(qs):
        kk, vv = gather_kv(k, table, s + 1, lengths[s], page), gather_kv(v, table, s + 1, lengths[s], page)
        lo = 0 if wk == "full" else ((pos // wsz) * wsz if wk == "chunk" else max(0, pos - wsz + 1))
        ref = ref_attention(q[i].float().view(NH, D), kk, vv, pos, lo, scale).reshape(-1)
        tol = 2e-5 if dtype == torch.float32 else 1.5e-2
        assert float((out[i].float() - ref).abs().max()) <= tol * max(1.0, float(ref.abs().max())), (i, s, pos)


def test_attention_finds_one_far_key_among_hundreds():
    """A key far back whose score stands out must take all the weight, wherever its page lies."""
    NH, NKV, D, page = 4, 2, 64, 64
    lengths = [700]
    k, v, table = paged_cache(1, lengths, NKV, D, page, torch.float32, seed=3)
    q = rnd(1, NH * D, seed=4)
    far = 13
    pg, off = int(table[1, far // page]), far % page
    for kvh in range(NKV):
        k[pg, kvh, off] = q.view(NH, D)[kvh * 2] * 40.0
    out = torch.empty_like(q)
    one = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().attention_general(q, out, k, v, table, page, one, torch.tensor([699], dtype=torch.int32, device=DEV),
                          torch.ones(1, dtype=torch.int32, device=DEV), n_heads=NH, n_kv_heads=NKV, head_dim=D,
                          window_kind=0, window_size=0, scale=1.0)
    for kvh in range(NKV):
        assert torch.allclose(out.view(NH, D)[kvh * 2], v[pg, kvh, off], atol=1e-4)
    # with a chunk window the far key is outside: the result must change
    out2 = torch.empty_like(q)
    K().attention_general(q, out2, k, v, table, page, one, torch.tensor([699], dtype=torch.int32, device=DEV),
                          torch.ones(1, dtype=torch.int32, device=DEV), n_heads=NH, n_kv_heads=NKV, head_dim=D,
                          window_kind=1, window_size=100, scale=1.0)
    assert float((out2 - out).abs().max()) > 0.1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D,interleaved,norm,before,temp,heads", [
    (16, False, True, False, None, (3, 1)), (48, True, True, True, None, (3, 1)),
    (128, False, False, False, (32.0, 0.1), (3, 1)), (256, True, True, False, (8.0, 0.5), (3, 1)),
    # heads of 128 in bfloat16 take the 16-byte kernel: odd and large head counts, both norm orders
    (128, False, True, False, (32.0, 0.1), (6, 2)), (128, False, True, True, None, (40, 8)),
    (128, False, False, False, None, (16, 1))])
def test_qkv_post(dtype, D, interleaved, norm, before, temp, heads):
    (NH, NKV), page, T = heads, 16, 6
    qkv = rnd(T, (NH + 2 * NKV) * D, dtype=dtype, seed=1)
    pos = [0, 1, 31, 32, 1000, 17]
    table = torch.tensor([[0] * 70, list(range(5, 75))], dtype=torch.int32, device=DEV)
    kc = torch.zeros(80, NKV, page, D, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, NH * D, dtype=dtype, device=DEV)
    inv_freq = (10000.0 ** (-torch.arange(D // 2).float() * 2 / D)).to(DEV)
    K().qkv_post(qkv, q_out, kc, vc, table, page, torch.zeros(T, dtype=torch.int32, device=DEV),
                 torch.tensor(pos, dtype=torch.int32, device=DEV), torch.ones(1, dtype=torch.int32, device=DEV),
                 n_heads=NH, n_kv_heads=NKV, head_dim=D, inv_freq=inv_freq, interleaved=interleaved, qk_norm=norm,
                 norm_before_rope=before, norm_eps=1e-5, temperature=temp)
    x = qkv.float().view(T, NH + 2 * NKV, D)

    def l2(t):
        return t / torch.sqrt((t * t).mean(-1, keepdim=True) + 1e-5)

    def rot(t):
        ang = torch.tensor(pos, device=DEV).float()[:, None] * inv_freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        o = torch.empty_like(t)
        if interleaved:
            a, b = t[..., 0::2], t[..., 1::2]
            o[..., 0::2], o[..., 1::2] = a * c - b * s, a * s + b * c
        else:
            a, b = t[..., :D // 2], t[..., D // 2:]
            o[..., :D // 2], o[..., D // 2:] = a * c - b * s, a * s + b * c
        return o

    qk = x[:, :NH + NKV]
    if norm and before:
        qk = l2(qk)
    qk = rot(qk)
    if norm and not before:
        qk = l2(qk)
    qr, kr = qk[:, :NH].clone(), qk[:, NH:]
    if temp is not None:
        p = torch.tensor(pos, device=DEV).float()
        qr = qr * (1 + temp[1] * torch.log(torch.floor((p + 1) / temp[0]) + 1))[:, None, None]
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    # position 1000 at high frequencies: sin/cos of a large float32 angle -- both sides use float32 angles
    assert float((q_out.float().view(T, NH, D) - qr).abs().max()) <= tol * float(qr.abs().max())
    for i, p_ in enumerate(pos):
        pg = 5 + p_ // page
        assert float((kc[pg, :, p_ % page].float() - kr[i]).abs().max()) <= tol * float(kr.abs().max())
        assert torch.equal(vc[pg, :, p_ % page].float(), x[i, NH + NKV:])


# ------------------------------------------------------------------------------------------------ routing
@pytest.mark.parametrize("T,H,E,k", [(1, 40, 3, 1), (50, 96, 8, 2), (300, 128, 16, 4), (7, 64, 128, 1)])
def test_router_and_lists(T, H, E, k):
    h, w = rnd(T, H, dtype=torch.bfloat16), rnd(E, H, dtype=torch.bfloat16, seed=1)
    w[1] = w[0]                                     # an exact tie: the lower index must win
    idx = torch.empty(T, k, dtype=torch.int32, device=DEV)
    gate = torch.empty(T, k, device=DEV)
    logits = torch.empty(T, E, device=DEV)
    K().router_topk(h, w, idx, gate, top_k=k, sigmoid_gate=True, logits_out=logits)
    ref = h.float() @ w.float().T
    assert torch.allclose(logits, ref, atol=1e-4 * float(ref.abs().max()))
    if T >= 128:          # many tokens take another kernel: a logit must have the same bits either way
        part = torch.empty(50, E, device=DEV)
        K().router_topk(h[100:150], w, idx[100:150].clone(), gate[100:150].clone(), top_k=k, sigmoid_gate=True,
                        logits_out=part)
        assert torch.equal(part, logits[100:150])
    for t in range(T):
        row = logits[t].tolist()
        order = sorted(range(E), key=lambda e: (-row[e], e))[:k]
        assert idx[t].tolist() == order
        assert torch.allclose(gate[t], torch.sigmoid(logits[t, idx[t].long()]), atol=1e-6)
    M = T * k
    offs = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    row_token = torch.empty(M, dtype=torch.int32, device=DEV)
    row_scale = torch.empty(M, device=DEV)
    row_of_slot = torch.empty(M, dtype=torch.int32, device=DEV)
    K().moe_lists(idx, gate, offs, row_token, row_scale, row_of_slot, n_tokens=T, top_k=k, n_experts=E)
    flat = idx.flatten().tolist()
    counts = [flat.count(e) for e in range(E)]
    assert offs.tolist() == [0] + list(torch.tensor(counts).cumsum(0).tolist())
    assert sorted(row_of_slot.tolist()) == list(range(M))
    for s in range(M):
        m = int(row_of_slot[s])
        assert offs[flat[s]] <= m < offs[flat[s] + 1]
        assert int(row_token[m]) == s // k and float(row_scale[m]) == float(gate.flatten()[s])
    for e in range(E):                               # stable: rows of an expert in token order
        seg = row_token[int(offs[e]):int(offs[e + 1])].tolist()
        assert seg == sorted(seg)


@pytest.mark.parametrize("T,H,E,k,dt", [(1, 64, 16, 1, torch.bfloat16), (8, 5120, 16, 1, torch.bfloat16),
                                        (64, 256, 16, 1, torch.bfloat16), (32, 128, 128, 1, torch.bfloat16),
                                        (5, 96, 8, 2, torch.float32), (50, 64, 7, 3, torch.bfloat16),
                                        (300, 128, 16, 1, torch.bfloat16), (9, 100, 4, 2, torch.bfloat16)])
def test_moe_route_one_launch_equals_the_separate_kernels(T, H, E, k, dt):
    """The routing of a whole step (choice, lists, rows in expert order) through `moe_route`, which takes
    one kernel for few tokens, against router_topk + moe_lists + gather_rows: same bits everywhere."""
    h, w = rnd(T, H, dtype=dt), rnd(E, H, dtype=dt, seed=1)
    w[1] = w[0]
    M = T * k
    def buffers():
        return dict(idx=torch.full((T, k), -1, dtype=torch.int32, device=DEV), gate=torch.zeros(T, k, device=DEV),
                    logits=torch.zeros(T, E, device=DEV), offs=torch.full((E + 1,), -1, dtype=torch.int32, device=DEV),
                    row_token=torch.full((M,), -1, dtype=torch.int32, device=DEV), row_scale=torch.zeros(M, device=DEV),
                    row_of_slot=torch.full((M,), -1, dtype=torch.int32, device=DEV),
                    sorted_h=torch.zeros(M, H, dtype=dt, device=DEV))
    a, b = buffers(), buffers()
    K().router_topk(h, w, a["idx"], a["gate"], top_k=k, sigmoid_gate=True, logits_out=a["logits"])
    K().moe_lists(a["idx"], a["gate"], a["offs"], a["row_token"], a["row_scale"], a["row_of_slot"], n_tokens=T, top_k=k,
                  n_experts=E)
    sortable = (H * h.element_size()) % 16 == 0
    if sortable:
        K().gather_rows(h, a["row_token"], a["sorted_h"])
    done = K().moe_route(h, w, b["idx"], b["gate"], b["logits"], b["offs"], b["row_token"], b["row_scale"],
                         b["row_of_slot"], top_k=k, sigmoid_gate=True, sorted_h=b["sorted_h"] if sortable else None)
    if sortable and not done:
        K().gather_rows(h, b["row_token"], b["sorted_h"])
    assert done == (sortable and M <= 256 and T * E <= 4096)
    torch.cuda.synchronize()
    for name in a:
        assert torch.equal(a[name], b[name]), name


def test_moe_combine_and_gather_and_swiglu():
    T, k, H = 9, 3, 200
    res = rnd(T, H)
    y = rnd(T * k, H, seed=1)
    ros = torch.randperm(T * k).to(torch.int32).to(DEV)
    ref = res.clone()
    for t in range(T):
        for j in range(k):
            ref[t] += y[ros[t * k + j]]
    K().moe_combine(res, y, ros, top_k=k)
    assert torch.allclose(res, ref, atol=1e-6)
    src = rnd(11, 72, dtype=torch.bfloat16)
    rows = torch.tensor([10, 0, 0, 5], dtype=torch.int32, device=DEV)
    dst = torch.empty(4, 72, dtype=torch.bfloat16, device=DEV)
    K().gather_rows(src, rows, dst)
    assert torch.equal(dst, src[rows.long()])
    gu = rnd(5, 2 * 33)
    out = torch.empty(5, 33, device=DEV)
    K().swiglu(gu, out)
    g, u = gu[:, :33], gu[:, 33:]
    assert torch.allclose(out, g / (1 + torch.exp(-g)) * u, atol=1e-6)


def test_argmax_first_maximum_and_odd_vocabulary():
    V = 202049
    lg = rnd(3, V)
    lg[0, 777] = lg[0, 200000] = 50.0
    lg[2, V - 1] = 60.0
    out = torch.empty(3, dtype=torch.int32, device=DEV)
    K().argmax(lg, out)
    assert out.tolist() == [777, int(lg[1].argmax()), V - 1]


@pytest.mark.parametrize("NH,NKV,D,window,splits", [(40, 8, 128, ("full", 0), 1), (40, 8, 128, ("full", 0), 7),
                                                    (6, 2, 64, ("chunk", 100), 3), (16, 1, 128, ("sliding", 70), 2),
                                                    (5, 5, 64, ("chunk", 64), 4), (40, 8, 128, ("full", 0), 8),
                                                    (40, 8, 128, ("full", 0), 12), (6, 2, 64, ("sliding", 200), 9)])
def test_attention_decode_tensor_core_kernel(NH, NKV, D, window, splits):
    page = 64
    lengths = [1, 64, 65, 700, 333, 128]
    k, v, table = paged_cache(len(lengths), lengths, NKV, D, page, torch.bfloat16, seed=5)
    # stale contents beyond a sequence's length must not leak: poison the tail of every last page
    for s, l in enumerate(lengths):
        if l % page:
            pg = int(table[s + 1, (l - 1) // page])
            k[pg, :, l % page:] = float("nan")
            v[pg, :, l % page:] = float("nan")
    T = len(lengths)
    q = rnd(T, NH * D, dtype=torch.bfloat16, seed=9)
    out = torch.empty_like(q)
    token_seq = torch.arange(T, dtype=torch.int32, device=DEV)
    token_pos = torch.tensor([l - 1 for l in lengths], dtype=torch.int32, device=DEV)
    seq_slot = torch.arange(1, T + 1, dtype=torch.int32, device=DEV)
    wk, wsz = window
    scale = 1.0 / math.sqrt(D)
    assert K().attention_decode_supported(NH, NKV, D, page)
    K().attention_decode(q, out, k, v, table, page, token_seq, token_pos, seq_slot, n_heads=NH, n_kv_heads=NKV,
                         head_dim=D, window_kind=K().WINDOW_KINDS[wk], window_size=wsz, scale=scale, n_splits=splits)
    for i, l in enumerate(lengths):
        pos = l - 1
        kk = gather_kv(torch.nan_to_num(k), table, i + 1, l, page)
        vv = gather_kv(torch.nan_to_num(v), table, i + 1, l, page)
        lo = 0 if wk == "full" else ((pos // wsz) * wsz if wk == "chunk" else max(0, pos - wsz + 1))
        ref = ref_attention(q[i].float().view(NH, D), kk, vv, pos, lo, scale).reshape(-1)
        err = float((out[i].float() - ref).abs().max())
        assert err <= 1.5e-2 * max(1.0, float(ref.abs().max())), (i, l, err)
    assert not K().attention_decode_supported(12, 4, 48, 64) and not K().attention_decode_supported(34, 2, 128, 64)


def test_attention_decode_far_key():
    NH, NKV, D, page = 10, 2, 128, 64
    k, v, table = paged_cache(1, [2000], NKV, D, page, torch.bfloat16, seed=3)
    q = rnd(1, NH * D, dtype=torch.bfloat16, seed=4)
    far = 77
    pg, off = int(table[1, far // page]), far % page
    for kvh in range(NKV):
        k[pg, kvh, off] = (q.view(NH, D)[kvh * 5 + 2].float() * 30.0).bfloat16()
    out = torch.empty_like(q)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    K().attention_decode(q, out, k, v, table, page, z, torch.tensor([1999], dtype=torch.int32, device=DEV),
                         torch.ones(1, dtype=torch.int32, device=DEV), n_heads=NH, n_kv_heads=NKV, head_dim=D,
                         window_kind=0, window_size=0, scale=1.0, n_splits=5)
    for kvh in range(NKV):
        assert torch.allclose(out.view(NH, D)[kvh * 5 + 2].float(), v[pg, kvh, off].float(), atol=2e-2)


def _prefill_case(NH, NKV, D, window, seqs, seed=0, tile=128):
    """seqs: list of (cached positions before the step, new tokens).  Returns everything a launch needs."""
    page = 64
    lengths = [s + n for s, n in seqs]
    k, v, table = paged_cache(len(seqs), lengths, NKV, D, page, torch.bfloat16, seed=seed)
    for i, l in enumerate(lengths):                  # poison what lies beyond each sequence
        if l % page:
            pg = int(table[i + 1, (l - 1) // page])
            k[pg, :, l % page:] = float("nan")
            v[pg, :, l % page:] = float("nan")
    token_seq, token_pos, tiles = [], [], []
    base = 0
    for i, (s, n) in enumerate(seqs):
        token_seq += [i] * n
        token_pos += list(range(s, s + n))
        for off in range(0, n, tile):
            tiles.append((base + off, min(tile, n - off)))
        base += n
    T = base
    q = rnd(T, NH * D, dtype=torch.bfloat16, seed=seed + 7)
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(q=q, k=k, v=v, table=table, token_seq=dev(token_seq), token_pos=dev(token_pos),
                seq_slot=torch.arange(1, len(seqs) + 1, dtype=torch.int32, device=DEV),
                tile_tok0=dev([t[0] for t in tiles]), tile_rows=dev([t[1] for t in tiles]),
                lengths=lengths, pos=token_pos, seq=token_seq)


@pytest.mark.parametrize("tile", [256, 128, 200])
@pytest.mark.parametrize("NH,NKV,D,window", [(4, 2, 128, ("full", 0)), (6, 6, 64, ("chunk", 200)),
                                             (5, 1, 128, ("sliding", 130)), (8, 2, 64, ("chunk", 128))])
def test_attention_prefill_tensor_core_kernel(NH, NKV, D, window, tile):
    """Query tiles of up to 256 rows (two tiles of 128 per block), of exactly 128 (the second tile absent) and of 200
    (a ragged second tile), against sequences that start on a filled cache, in the middle of a page and of a key
    tile, with windows whose low end falls between the two query tiles."""
    page = 64
    assert K().load().cpi_attention_prefill_tile_rows() == K().PREFILL_TILE_ROWS == 256
    c = _prefill_case(NH, NKV, D, window, [(0, 1), (0, 129), (0, 300), (70, 200), (256, 64), (0, 64), (100, 700),
                                           (130, 256)], tile=tile)
    out = torch.full_like(c["q"], float("nan"))
    wk, wsz = window
    scale = 1.0 / math.sqrt(D)
    assert K().attention_prefill_supported(NH, NKV, D, page)
    K().attention_prefill(c["q"], out, c["k"], c["v"], c["table"], page, c["token_seq"], c["token_pos"], c["seq_slot"],
                          c["tile_tok0"], c["tile_rows"], n_heads=NH, n_kv_heads=NKV, head_dim=D,
                          window_kind=K().WINDOW_KINDS[wk], window_size=wsz, scale=scale)
    torch.cuda.synchronize()
    assert int(K().tc_error_flag(DEV)) == 0
    kk = [gather_kv(torch.nan_to_num(c["k"]), c["table"], i + 1, l, page) for i, l in enumerate(c["lengths"])]
    vv = [gather_kv(torch.nan_to_num(c["v"]), c["table"], i + 1, l, page) for i, l in enumerate(c["lengths"])]
    worst = 0.0
    for t, (s, pos) in enumerate(zip(c["seq"], c["pos"])):
        lo = 0 if wk == "full" else ((pos // wsz) * wsz if wk == "chunk" else max(0, pos - wsz + 1))
        ref = ref_attention(c["q"][t].float().view(NH, D), kk[s], vv[s], pos, lo, scale).reshape(-1)
        err = float((out[t].float() - ref).abs().max()) / max(1.0, float(ref.abs().max()))
        worst = max(worst, err)
        assert err <= 1.5e-2, (t, s, pos, err)
    print("prefill attention worst error", worst)


def test_attention_prefill_far_key_and_general_kernel_agree():
    NH, NKV, D, page = 4, 1, 128, 64
    c = _prefill_case(NH, NKV, D, ("full", 0), [(0, 900)], seed=3)
    far = 5
    pg, off = int(c["table"][1, far // page]), far % page
    c["k"][pg, 0, off] = (c["q"][899].view(NH, D)[1].float() * 30.0).bfloat16()
    out = torch.empty_like(c["q"])
    args = (c["k"], c["v"], c["table"], page, c["token_seq"], c["token_pos"], c["seq_slot"])
    K().attention_prefill(c["q"], out, *args, c["tile_tok0"], c["tile_rows"], n_heads=NH, n_kv_heads=NKV, head_dim=D,
                          window_kind=0, window_size=0, scale=1.0)
    assert torch.allclose(out[899].view(NH, D)[1].float(), c["v"][pg, 0, off].float(), atol=2e-2)
    gen = torch.empty_like(c["q"])
    K().attention_general(c["q"], gen, *args, n_heads=NH, n_kv_heads=NKV, head_dim=D, window_kind=0, window_size=0,
                          scale=1.0)
    assert float((out.float() - gen.float()).abs().max()) <= 2e-2 * float(gen.float().abs().max())


# ------------------------------------------------------------------------------------------------ sampling
@pytest.mark.parametrize("V,quantum", [(50021, 0.0), (50021, 0.5), (3000, 2.0), (202048, 0.0)])
def test_sample_kernel_keeps_the_k_most_probable_with_ties_by_index(V, quantum):
    """Temperature / top-k / top-p draws at a large vocabulary against a host walk over the kernel's own
    weights (its scratch holds e = exp(logit / T - max) after the call): the k largest, equal ones by
    index, mass cut at top_p with the crossing token kept, renormalised, drawn with the given uniform.
    Quantised logits make thousands of exact ties around the k-th place."""
    g = torch.Generator().manual_seed(V)
    cases = [(0.7, 1, 1.0), (1.0, 7, 1.0), (0.8, 40, 0.9), (1.3, 256, 0.3), (1.0, 256, 1.0), (0.5, 100, 0.95),
             (1.0, 300, 1.0), (2.0, 13, 0.5)]
    R = len(cases) * 3
    logits = torch.randn(R, V, generator=g) * 3
    if quantum:
        logits = torch.round(logits / quantum) * quantum
    logits[1, 5] = float("nan")
    logits[2, 7] = float("inf")
    T = torch.tensor([c[0] for c in cases] * 3)
    k = torch.tensor([c[1] for c in cases] * 3, dtype=torch.int32)
    p = torch.tensor([c[2] for c in cases] * 3)
    u = torch.rand(R, generator=g)
    dev = lambda t: t.to(DEV)
    work = torch.empty(R * V, device=DEV)
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    K().sample(dev(logits), work, dev(T), dev(k), dev(p), dev(u), out)
    torch.cuda.synchronize()
    e_all = work.view(R, V).cpu()
    near = 0
    for r in range(R):
        e = e_all[r]
        kk = max(1, min(int(k[r]), V, 256))
        order = sorted(range(V), key=lambda i: (-float(e[i]), i))[:kk] if V <= 5000 else None
        if order is None:                                   # the same order without sorting the whole vocabulary
            top = torch.topk(e, min(V, kk + 4096)).values[-1]
            idx = (e >= top).nonzero().flatten().tolist()
            order = sorted(idx, key=lambda i: (-float(e[i]), i))[:kk]
        order = [i for i in order if float(e[i]) > 0]
        total = float(e.double().sum())
        probs, mass = [], 0.0
        margin = 1.0
        for i in order:
            q = float(e[i]) / total
            probs.append(q)
            mass += q
            if 0 < float(p[r]) < 1:
                margin = min(margin, abs(mass - float(p[r])))
                if mass >= float(p[r]):
                    break
        kept = order[:len(probs)]
        s = sum(probs)
        run, pick = 0.0, kept[-1]
        for i, q in zip(kept, probs):
            run += q / s
            margin = min(margin, abs(run - float(u[r])))
            if float(u[r]) <= run:
                pick = i
                break
        if margin < 1e-5:                                   # a float32 rounding could decide: not a fair case
            near += 1
            continue
        assert int(out[r]) == pick, (r, cases[r % len(cases)], int(out[r]), pick)
    assert near <= 2


# ------------------------------------------------------------------------------------------------ load time
def test_load_time_kernels_random_fill_widen_and_transpose():
    """The kernels that run once at load: the counter-based random fill gives the host generator's bits (any start,
    any length, both dtypes); float16 is widened exactly; the experts' matrices are turned for odd sizes too."""
    from cpi_b200.weights.random_init import _normal_table_on, counter_normal
    table = _normal_table_on(torch.device(DEV))
    for n, start, seed, std, dt in [(1, 0, 5, 0.02, torch.bfloat16), (1000003, 0, 0x7FFFFFFFFFFFFFFF, 0.05, torch.bfloat16),
                                    (4099, 123456789012, 42, 1.0, torch.float32), (70000, 7, 1 << 40, 0.02, torch.float32)]:
        out = torch.empty(n, dtype=dt, device=DEV)
        K().random_normal(out, start, seed, std, table)
        ref = counter_normal(seed, start, n, std, "cpu").to(dt)
        assert torch.equal(out.cpu(), ref), (n, start, seed)
    h = (torch.randn(5, 77, generator=torch.Generator().manual_seed(1)) * 100).half().to(DEV)
    h[0, 0], h[0, 1], h[0, 2] = 65504.0, 6e-8, float("-inf")
    w = torch.empty(5, 77, dtype=torch.float32, device=DEV)
    K().widen_f16(h, w)
    assert torch.equal(w, h.float())
    for shape, dt in [((3, 70, 129), torch.bfloat16), ((1, 33, 31), torch.float32), ((4, 128, 256), torch.bfloat16),
                      ((65, 100), torch.float32)]:
        a = rnd(*shape, dtype=dt, seed=9)
        assert torch.equal(K().transpose_last2(a), a.transpose(-1, -2).contiguous())
