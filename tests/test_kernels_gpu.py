"""Each kernel alone against a plain float32 restatement of the same operation,
at sizes other than the tiny models'."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from janas_b200.csrc import ops as o
    return o


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator().manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("dm", [100, 2560])
def test_embed(dtype, dm):
    table = rnd(300, dm, dtype=dtype)
    toks = torch.tensor([5, 299, 0, 5, 123], dtype=torch.int32)
    got = ops().embed(table.to(DEV), toks.to(DEV)).cpu()
    assert torch.equal(got, table[toks.long()].float())


@pytest.mark.parametrize("wdt", DTYPES)
@pytest.mark.parametrize("odt", DTYPES)
@pytest.mark.parametrize("n,dm", [(1, 40), (5, 2560), (33, 1000), (300, 1000), (257, 2560)])
def test_rmsnorm(wdt, odt, n, dm):
    x = rnd(n, dm, scale=3.0)
    w = (1 + 0.1 * rnd(dm)).to(wdt)
    want = plain.rms_norm(x, w.float(), 1e-5)
    got = ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-5, odt).cpu().float()
    tol = 2e-6 if odt == torch.float32 else 2 ** -8
    assert (got - want).abs().max() <= tol * want.abs().max()
    # with a stack of partial sums added first, and x updated in place
    delta = rnd(3, n, dm, seed=1)
    xd = x.to(DEV).clone()
    got = ops().rmsnorm(xd, w.to(DEV), 1e-5, odt, delta=delta.to(DEV)).cpu().float()
    x2 = x + delta[0] + delta[1] + delta[2]
    assert torch.equal(xd.cpu(), x2)
    want = plain.rms_norm(x2, w.float(), 1e-5)
    assert (got - want).abs().max() <= tol * want.abs().max()
    # chosen rows only
    rows = torch.tensor([n - 1, 0], dtype=torch.int32)
    got = ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-5, odt, rows=rows.to(DEV)).cpu().float()
    want = plain.rms_norm(x[rows.long()], w.float(), 1e-5)
    assert (got - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("wdt", DTYPES)
@pytest.mark.parametrize("n,dm,S", [(1, 1024, 1), (8, 2560, 14), (3, 1027, 17), (5, 9000, 2),
                                    (2, 17000, 3), (64, 2560, 14), (40, 100, 9), (33, 4096, 1),
                                    (200, 1000, 20)])
def test_rmsnorm_few_rows(wdt, n, dm, S):
    """Few rows with bfloat16 output (a row shared out among the CTAs of a cluster)
    and a middling number (a block per row, four values per thread).  One value of
    each row is large, so that a missing share would show."""
    x = rnd(n, dm, scale=3.0)
    x[:, dm - 3] = 200.0
    w = (1 + 0.1 * rnd(dm)).to(wdt)
    delta = rnd(S, n, dm, seed=1)
    xd = x.to(DEV).clone()
    got = ops().rmsnorm(xd, w.to(DEV), 1e-5, torch.bfloat16, delta=delta.to(DEV)).cpu().float()
    x2 = x.clone()
    for s in range(S):
        x2 = x2 + delta[s]
    assert torch.equal(xd.cpu(), x2)
    want = plain.rms_norm(x2, w.float(), 1e-5)
    assert (got - want).abs().max() <= 2 ** -8 * want.abs().max()
    rows = torch.tensor([n - 1, 0], dtype=torch.int32)
    got = ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-5, torch.bfloat16, rows=rows.to(DEV)).cpu().float()
    want = plain.rms_norm(x[rows.long()], w.float(), 1e-5)
    assert (got - want).abs().max() <= 2 ** -8 * want.abs().max()


@pytest.mark.parametrize("wdt", DTYPES)
@pytest.mark.parametrize("n,dm,S", [(257, 2560, 1), (1001, 516, 3), (4097, 260, 2), (5003, 1000, 1),
                                    (8193, 132, 1), (9001, 260, 2)])
def test_rmsnorm_many_rows(wdt, n, dm, S):
    """Many rows with bfloat16 output: four, two or one warp per row by the number
    of rows, row counts that leave a block's last rows empty, widths that leave
    lanes without values.  One value of each row is large, so that a warp's share
    missing from the row's sum would show."""
    x = rnd(n, dm, scale=3.0)
    x[:, dm - 3] = 200.0
    x[:, 1] = -150.0
    w = (1 + 0.1 * rnd(dm)).to(wdt)
    delta = rnd(S, n, dm, seed=1)
    xd = x.to(DEV).clone()
    got = ops().rmsnorm(xd, w.to(DEV), 1e-5, torch.bfloat16, delta=delta.to(DEV)).cpu().float()
    x2 = x.clone()
    for s in range(S):
        x2 = x2 + delta[s]
    assert torch.equal(xd.cpu(), x2)
    want = plain.rms_norm(x2, w.float(), 1e-5)
    assert ((got - want).abs().max(dim=1).values <= 2 ** -8 * want.abs().max(dim=1).values).all()
    got = ops().rmsnorm(x.to(DEV), w.to(DEV), 1e-5, torch.bfloat16).cpu().float()
    want = plain.rms_norm(x, w.float(), 1e-5)
    assert ((got - want).abs().max(dim=1).values <= 2 ** -8 * want.abs().max(dim=1).values).all()


@pytest.mark.parametrize("odt", DTYPES)
def test_swiglu(odt):
    n, ff = 7, 300
    gu = rnd(2, n, 2 * ff, scale=4.0)
    s = gu[0] + gu[1]
    g, u = s[:, :ff], s[:, ff:]
    want = g / (1 + torch.exp(-g)) * u
    got = ops().swiglu(gu.to(DEV), odt).cpu().float()
    tol = 2e-6 if odt == torch.float32 else 2 ** -8
    assert (got - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("adt", DTYPES)
@pytest.mark.parametrize("wdt", DTYPES)
@pytest.mark.parametrize("n,m,k", [(1, 1, 1), (3, 70, 50), (65, 129, 33), (130, 64, 256),
                                   (2, 300, 2560)])
def test_gemm_simt(adt, wdt, n, m, k):
    a, w = rnd(n, k, dtype=adt), rnd(m, k, dtype=wdt, seed=3)
    want = (a.double() @ w.double().T).float()
    got = ops().linear(a.to(DEV), w.to(DEV), force_simt=True)
    assert got.shape == (1, n, m)
    assert (got[0].cpu() - want).abs().max() <= 1e-6 * math.sqrt(k) * max(1.0, want.abs().max())


def test_gemm_rows_do_not_depend_on_the_batch():
    a, w = rnd(70, 96), rnd(200, 96, seed=4)
    whole = ops().linear(a.to(DEV), w.to(DEV))[0]
    one = ops().linear(a[37:38].contiguous().to(DEV), w.to(DEV))[0]
    assert torch.equal(whole[37:38], one)


def test_rope_table():
    for theta, hd in ((10000.0, 16), (1e6, 128), (50000.0, 48)):
        half = hd // 2
        expo = np.float32(-2.0) * np.arange(half, dtype=np.float32) / np.float32(hd)
        inv = np.power(np.float64(np.float32(theta)), expo.astype(np.float64)).astype(np.float32)
        cs, sn = ops().rope_table(torch.from_numpy(inv).to(DEV), 9000)
        pos = [0, 1, 63, 64, 1000, 8999]
        c, s = plain.rope_table(pos, hd, theta)
        assert torch.equal(cs.cpu()[pos], c) and torch.equal(sn.cpu()[pos], s)


def paged(k, v, n_pages, perm_seed=0):
    """Lays [n, nkv, hd] keys and values of ONE sequence out in pages in a
    shuffled order; returns caches and the block table."""
    n, nkv, hd = k.shape
    need = (n + 63) // 64
    order = np.random.default_rng(perm_seed).permutation(n_pages)[:need]
    kc = torch.zeros(n_pages, nkv, 64, hd, dtype=k.dtype)
    vc = torch.zeros_like(kc)
    for t in range(n):
        kc[order[t // 64], :, t % 64] = k[t]
        vc[order[t // 64], :, t % 64] = v[t]
    bt = torch.full((1, (need + 7) // 8 * 8), -1, dtype=torch.int32)
    bt[0, :need] = torch.from_numpy(order.astype(np.int32))
    return kc, vc, bt


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, 0), (8, 1, 64, 0), (5, 5, 80, 0),
                                              (6, 2, 32, 50), (4, 4, 16, 130), (16, 2, 256, 0)])
def test_attention_whole_sequence(dtype, nh, nkv, hd, window):
    n = 300
    q, k, v = rnd(n, nh, hd, dtype=dtype), rnd(n, nkv, hd, dtype=dtype, seed=1), \
        rnd(n, nkv, hd, dtype=dtype, seed=2)
    want = plain.attention(q.float(), k.float(), v.float(), window)
    kc, vc, bt = paged(k, v, 9)
    pos = torch.arange(n, dtype=torch.int32)
    seq = torch.zeros(n, dtype=torch.int32)
    chunk = ops().attention_chunk()
    mc = (n - 1) // chunk + 1 if not window else min((n - 1) // chunk + 1, (window - 1) // chunk + 2)
    got = ops().attention(q.to(DEV), kc.to(DEV), vc.to(DEV), pos.to(DEV), seq.to(DEV), bt.to(DEV),
                          window, 1 / math.sqrt(hd), mc).cpu().float()
    tol = 5e-6 if dtype == torch.float32 else 2 ** -8
    assert (got - want).abs().max() <= tol * want.abs().max()


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_a_far_key_and_the_window_s_edge(dtype):
    """One key among 700 has a score that stands out: the output is its value.
    With a window the key is seen by exactly the rows whose window holds it."""
    n, nh, nkv, hd = 700, 4, 2, 64
    q = torch.zeros(n, nh, hd)
    k = torch.zeros(n, nkv, hd)
    v = rnd(n, nkv, hd)
    q[:, :, 3] = 24.0
    k[133, :, 3] = 24.0        # score 576 / 8 = 72 above the others
    if dtype == torch.bfloat16:
        v = v.to(dtype).float()
    kc, vc, bt = paged(k.to(dtype), v.to(dtype), 12, perm_seed=5)
    pos = torch.arange(n, dtype=torch.int32)
    seq = torch.zeros(n, dtype=torch.int32)
    chunk = ops().attention_chunk()
    for window in (0, 200):
        mc = (n - 1) // chunk + 1 if not window else (window - 1) // chunk + 2
        got = ops().attention(q.to(dtype).to(DEV), kc.to(DEV), vc.to(DEV), pos.to(DEV),
                              seq.to(DEV), bt.to(DEV), window, 1 / math.sqrt(hd), mc).cpu().float()
        tol = 1e-5 if dtype == torch.float32 else 2 ** -7
        last_seeing = n - 1 if not window else 133 + window - 1
        for r in (133, 134, 400 if not window else 300, last_seeing):
            assert (got[r, 1] - v[133, 0]).abs().max() <= tol, (window, r)
        if window:
            r = last_seeing + 1          # the key has just left the window
            want = v[r + 1 - window:r + 1, 1].mean(0)
            assert (got[r, 3] - want).abs().max() <= 10 * tol, (window, r)
        want = v[:100, 0].mean(0)        # before the key: uniform over what is visible
        assert (got[99, 0] - want).abs().max() <= 10 * tol


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n0,n1,hd,nh,nkv", [(25, 15, 48, 6, 2), (300, 58, 128, 6, 2), (3, 1, 16, 6, 2),
                                             (40, 9, 32, 5, 1), (17, 30, 64, 9, 3),
                                             (9, 11, 256, 3, 3), (6, 3, 80, 4, 2),
                                             (260, 20, 32, 5, 1), (250, 30, 64, 9, 3),
                                             (270, 10, 256, 3, 3), (310, 64, 128, 32, 8)])
def test_qk_norm_rope_append(dtype, n0, n1, hd, nh, nkv):
    """The kernel for any even head size (48, 16, 80) and the 16-byte ones for head
    sizes 32, 64, 128 and 256 (a block per row from 256 rows on), with head counts
    that leave a warp partly empty."""
    n = n0 + n1
    width = (nh + 2 * nkv) * hd
    qkv = rnd(2, n, width, scale=2.0)
    qw, kw = (1 + 0.1 * rnd(hd)).to(dtype), (1 + 0.1 * rnd(hd, seed=1)).to(dtype)
    # two sequences: the first rows are positions 70.. of sequence 0, the others
    # positions 0.. of sequence 1
    pos = torch.cat([torch.arange(70, 70 + n0), torch.arange(0, n1)]).int()
    seq = torch.cat([torch.zeros(n0), torch.ones(n1)]).int()
    bt = torch.tensor([[4, 2, 0, 3, 5, 7, -1, -1], [1, -1, -1, -1, -1, -1, -1, -1]],
                      dtype=torch.int32)
    kc = torch.zeros(8, nkv, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    half = hd // 2
    expo = np.float32(-2.0) * np.arange(half, dtype=np.float32) / np.float32(hd)
    inv = np.power(np.float64(np.float32(1e6)), expo.astype(np.float64)).astype(np.float32)
    cs, sn = ops().rope_table(torch.from_numpy(inv).to(DEV), 512)
    q = ops().qk_norm_rope_append(qkv.to(DEV), qw.to(DEV), kw.to(DEV), 1e-6, cs, sn,
                                  pos.to(DEV), seq.to(DEV), bt.to(DEV), kc, vc, nh, nkv, hd,
                                  dtype).cpu().float()
    s = qkv[0] + qkv[1]
    qs, ks, vs = s[:, :nh * hd].view(n, nh, hd), s[:, nh * hd:(nh + nkv) * hd].view(n, nkv, hd), \
        s[:, (nh + nkv) * hd:].view(n, nkv, hd)
    c, sgn = plain.rope_table(pos.tolist(), hd, 1e6)
    wq = plain.rope_neox(plain.rms_norm(qs, qw.float(), 1e-6), c, sgn)
    wk = plain.rope_neox(plain.rms_norm(ks, kw.float(), 1e-6), c, sgn)
    tol = 3e-6 if dtype == torch.float32 else 2 ** -8
    assert (q - wq).abs().max() <= tol * wq.abs().max()
    kc, vc = kc.cpu().float(), vc.cpu().float()
    for r in range(n):
        page = bt[seq[r], pos[r] // 64]
        assert (kc[page, :, pos[r] % 64] - wk[r]).abs().max() <= tol * wk.abs().max()
        assert (vc[page, :, pos[r] % 64] - vs[r]).abs().max() <= tol * vs.abs().max()
    # nothing else was written
    written = torch.zeros(8, 64, dtype=torch.bool)
    for r in range(n):
        written[bt[seq[r], pos[r] // 64], pos[r] % 64] = True
    kc, vc = kc.permute(0, 2, 1, 3), vc.permute(0, 2, 1, 3)      # [page, position, head, value]
    assert float(kc[~written].abs().sum()) == 0.0 and float(vc[~written].abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,nh,nkv", [(128, 6, 2), (32, 5, 1), (64, 9, 3), (256, 3, 3)])
def test_qk_norm_rope_append_same_bits_for_few_and_many_rows(dtype, hd, nh, nkv):
    """From 256 rows on another kernel runs; a row's values must be the same bits
    whether it comes among 300 rows or among 100."""
    n = 300
    qkv = rnd(3, n, (nh + 2 * nkv) * hd, scale=2.0).to(DEV)
    qw, kw = (1 + 0.1 * rnd(hd)).to(dtype).to(DEV), (1 + 0.1 * rnd(hd, seed=1)).to(dtype).to(DEV)
    pos = torch.arange(5, 5 + n).int().to(DEV)
    seq = torch.zeros(n).int().to(DEV)
    bt = torch.tensor([[4, 2, 0, 3, 5, 7, -1, -1]], dtype=torch.int32).to(DEV)
    half = hd // 2
    expo = np.float32(-2.0) * np.arange(half, dtype=np.float32) / np.float32(hd)
    inv = np.power(np.float64(np.float32(1e4)), expo.astype(np.float64)).astype(np.float32)
    cs, sn = ops().rope_table(torch.from_numpy(inv).to(DEV), 512)
    res = []
    for cuts in ([(0, n)], [(0, 100), (100, 200), (200, n)]):
        kc = torch.zeros(8, nkv, 64, hd, dtype=dtype, device=DEV)
        vc = torch.zeros_like(kc)
        q = torch.cat([ops().qk_norm_rope_append(qkv[:, a:b].contiguous(), qw, kw, 1e-6, cs, sn,
                                                 pos[a:b].contiguous(), seq[a:b].contiguous(), bt,
                                                 kc, vc, nh, nkv, hd, dtype) for a, b in cuts])
        res.append((q, kc, vc))
    for a, b in zip(res[0], res[1]):
        assert torch.equal(a, b)


def test_argmax_is_the_first_maximum():
    lg = rnd(9, 1000)
    lg[2, 700] = lg[2, 30] = 9.0
    lg[5, :] = 1.0
    got = ops().sample(lg.to(DEV)).cpu().tolist()
    want = [int(np.argmax(r)) for r in lg.numpy()]
    assert got == want and got[2] == 30 and got[5] == 0


@pytest.mark.parametrize("V", [300, 5000, 151936])
def test_sampling_kernel_equals_the_plain_sampler(V):
    """Many rows, every setting: the same picks and the same random states."""
    rows = 12
    lg = rnd(rows, V, scale=2.0, seed=V)
    lg[3, 17] = lg[3, 5] = lg[3].max() + 1       # a tie at the top
    lg[4, 100:103] = lg[4].topk(5).values[4]     # ties around a top_k cut of 5
    settings = [(0.8, 20, 0.8, 0.0), (0.7, 0, 0.0, 0.0), (1.0, 5, 0.0, 0.0), (1.5, 0, 0.9, 0.05),
                (0.3, 50, 1.0, 0.2), (2.0, 3, 0.5, 0.0), (0.0, 0, 0.0, 0.0), (1.0, 3000, 0.0, 0.0)]
    o = ops()
    cap = 1 << (V - 1).bit_length()
    big_k = torch.empty(rows, cap, dtype=torch.int64, device=DEV)
    big_p = torch.empty(rows, cap, dtype=torch.float32, device=DEV)
    dl = lg.to(DEV)
    for si, (t, k, p, mp) in enumerate(settings):
        seeds = [(1 << 63) + 12345 * (si + 1) + r for r in range(rows)]
        slot = torch.arange(rows, dtype=torch.int32).flip(0).contiguous()   # row r uses slot 11 - r
        # state of slot s is the seed of the row that uses it
        state = torch.empty(rows, dtype=torch.int64)
        for r in range(rows):
            s = seeds[r]
            state[slot[r]] = s - (1 << 64) if s >= (1 << 63) else s
        state = state.to(DEV)
        full = lambda val, dt: torch.full((rows,), val, dtype=dt, device=DEV)
        forced = torch.zeros(rows, dtype=torch.int32, device=DEV)
        for rep in range(2):
            got = o.sample(dl, row_slot=slot.to(DEV), temperature=full(t, torch.float32),
                           top_k=full(k, torch.int32), top_p=full(p, torch.float32),
                           min_p=full(mp, torch.float32), rng=state, big_keys=big_k,
                           big_probs=big_p, forced=forced).cpu().tolist()
            for r in range(rows):
                tok, seeds[r] = plain.sample(lg[r].numpy(), t, k, p, mp, seeds[r])
                assert got[r] == tok, (V, (t, k, p, mp), rep, r)
            back = [(int(x) + (1 << 64)) % (1 << 64) for x in state.cpu().tolist()]
            assert [back[int(slot[r])] for r in range(rows)] == seeds


TC_SHAPES = [(1, 128, 64), (8, 200, 96), (16, 6144, 2560), (17, 130, 200), (33, 2560, 4096),
             (64, 384, 64), (100, 331, 80), (129, 300, 128), (300, 200, 2560), (700, 1000, 1096),
             (3, 151936, 256)]


@pytest.mark.parametrize("n,m,k", TC_SHAPES)
def test_gemm_tensor_core(n, m, k):
    """The tcgen05 product against a double-precision product, at every tile
    shape (tokens 1 .. 700), with rows and features that fill no tile and k that
    is no multiple of 64, and with k cut into parts."""
    a, w = rnd(n, k, dtype=torch.bfloat16), rnd(m, k, dtype=torch.bfloat16, seed=3)
    want = (a.double() @ w.double().T).float()
    o = ops()
    got = o.linear(a.to(DEV), w.to(DEV))
    assert o.gemm_tc_error() == 0
    assert got.shape[1:] == (n, m)
    S = got.shape[0]
    assert S == o.lib().jb_gemm_tc_splits(n, m, k)
    if n <= 128 and m <= 6144 and k >= 2048:
        assert S > 1                      # few tokens, long rows: k is cut
    got = got.double().sum(0).float().cpu()
    assert (got - want).abs().max() <= 2e-6 * math.sqrt(k) * max(1.0, want.abs().max())
    # and the plain kernel agrees with it
    simt = o.linear(a.to(DEV), w.to(DEV), force_simt=True)[0].cpu()
    assert (got - simt).abs().max() <= 2e-6 * math.sqrt(k) * max(1.0, want.abs().max())


def test_gemm_tensor_core_finds_one_large_product():
    """A single large entry far along k, in the last rows and features: it lands
    in the right place of the output and nowhere else."""
    n, m, k = 300, 260, 1096
    a = torch.zeros(n, k, dtype=torch.bfloat16)
    w = torch.zeros(m, k, dtype=torch.bfloat16)
    a[299, 1090] = 3.0
    w[259, 1090] = 5.0
    a[7, 3] = 2.0
    w[128, 3] = -4.0
    got = ops().linear(a.to(DEV), w.to(DEV)).sum(0).cpu()
    want = torch.zeros(n, m)
    want[299, 259] = 15.0
    want[7, 128] = -8.0
    assert torch.equal(got, want)


@pytest.mark.parametrize("n,ff,k", [(5, 100, 64), (128, 224, 96), (129, 136, 80), (600, 300, 2560),
                                    (1, 64, 64), (16, 136, 80), (17, 200, 256), (33, 72, 1000),
                                    (64, 1000, 2560), (8, 1984, 512), (65, 100, 128)])
def test_gemm_tensor_core_swiglu(n, ff, k):
    """Up to 64 rows in tiles of 64 gate and 64 up features, above in tiles of 128
    and 128; feature counts that leave the last tile partly empty."""
    a = rnd(n, k, dtype=torch.bfloat16)
    w = rnd(2 * ff, k, dtype=torch.bfloat16, seed=5, scale=0.3)
    a[n - 1] *= 60.0                      # gates of a few hundred, of both signs
    got = ops().linear_swiglu(a.to(DEV), w.to(DEV))
    assert ops().gemm_tc_error() == 0
    gu = a.double() @ w.double().T
    g, u = gu[:, :ff], gu[:, ff:]
    want = (g / (1 + torch.exp(-g)) * u).float()
    assert got.dtype == torch.bfloat16 and got.shape == (n, ff)
    err = (got.float().cpu() - want).abs().max(dim=1).values      # row by row: row 1 is large
    assert bool((err <= 2 ** -8 * want.abs().max(dim=1).values).all())


def test_products_that_the_tensor_core_kernel_refuses_go_the_plain_way():
    o = ops()
    a, w = rnd(4, 100, dtype=torch.bfloat16), rnd(30, 100, dtype=torch.bfloat16)   # 100 % 8 != 0
    got = o.linear(a.to(DEV), w.to(DEV))
    assert got.shape == (1, 4, 30)
    want = (a.double() @ w.double().T).float()
    assert (got[0].cpu() - want).abs().max() <= 1e-5 * want.abs().max()
    assert o.linear_swiglu(a.to(DEV), w.to(DEV)) is None


def _paged_many(ks, vs, n_pages, seed=0):
    """Several sequences' keys and values laid out in shuffled pages."""
    nkv, hd = ks[0].shape[1:]
    kc = (torch.randn(n_pages, nkv, 64, hd) * 3).to(ks[0].dtype)    # stale finite values elsewhere
    vc = (torch.randn(n_pages, nkv, 64, hd) * 3).to(ks[0].dtype)
    order = np.random.default_rng(seed).permutation(n_pages).tolist()
    need = max((k.shape[0] + 63) // 64 for k in ks)
    bt = torch.full((len(ks), (need + 7) // 8 * 8), -1, dtype=torch.int32)
    for i, (k, v) in enumerate(zip(ks, vs)):
        for p in range((k.shape[0] + 63) // 64):
            page = order.pop()
            bt[i, p] = page
            cnt = min(64, k.shape[0] - 64 * p)
            kc[page, :, :cnt] = k[64 * p:64 * p + cnt].transpose(0, 1)
            vc[page, :, :cnt] = v[64 * p:64 * p + cnt].transpose(0, 1)
    return kc, vc, bt


@pytest.mark.parametrize("nh,nkv,hd,window", [(8, 2, 128, 0), (32, 8, 128, 0), (8, 1, 128, 0),
                                              (6, 2, 64, 0), (5, 1, 128, 70), (4, 4, 64, 200),
                                              (64, 8, 128, 0), (12, 4, 128, 129)])
def test_attention_tensor_core_prefill(nh, nkv, hd, window):
    """Whole prompts of unequal lengths in one call, and tokens appended to
    sequences that already hold some, on the tensor-core kernel."""
    o = ops()
    lens, pos0 = [300, 1, 129, 64, 40], [0, 0, 0, 0, 170]     # the last one goes on from 170
    qs, ks, vs = [], [], []
    for i, (n, p0) in enumerate(zip(lens, pos0)):
        qs.append(rnd(p0 + n, nh, hd, dtype=torch.bfloat16, seed=10 * i))
        ks.append(rnd(p0 + n, nkv, hd, dtype=torch.bfloat16, seed=10 * i + 1))
        vs.append(rnd(p0 + n, nkv, hd, dtype=torch.bfloat16, seed=10 * i + 2))
    want = torch.cat([plain.attention(q.float(), k.float(), v.float(), window)[p0:]
                      for q, k, v, p0 in zip(qs, ks, vs, pos0)])
    q = torch.cat([q[p0:] for q, p0 in zip(qs, pos0)])
    kc, vc, bt = _paged_many(ks, vs, 20)
    row_pos = torch.cat([torch.arange(p0, p0 + n) for n, p0 in zip(lens, pos0)]).int()
    row_seq = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).int()
    row0 = np.concatenate([[0], np.cumsum(lens)])
    per = o.attention_block_positions(nh, nkv)
    blocks = o.attention_blocks(row0[:-1], pos0, lens, per, torch.device(DEV))
    chunk = o.attention_chunk()
    mc = 299 // chunk + 1
    got = o.attention(q.to(DEV), kc.to(DEV), vc.to(DEV), row_pos.to(DEV), row_seq.to(DEV),
                      bt.to(DEV), window, 1 / math.sqrt(hd), mc, blocks=blocks).cpu().float()
    assert o.attn_tc_error() == 0
    err = (got - want).abs().max() / want.abs().max()
    assert err <= 2 ** -7, err           # P and the output are bfloat16
    simt = o.attention(q.to(DEV), kc.to(DEV), vc.to(DEV), row_pos.to(DEV), row_seq.to(DEV),
                       bt.to(DEV), window, 1 / math.sqrt(hd), mc, force_simt=True).cpu().float()
    assert (got - simt).abs().max() / want.abs().max() <= 2 ** -7


@pytest.mark.parametrize("nh,nkv,hd,window", [(32, 8, 128, 0), (8, 1, 128, 0), (6, 2, 64, 0),
                                              (5, 1, 128, 70), (64, 8, 128, 300)])
def test_attention_tensor_core_decode(nh, nkv, hd, window):
    """One new token for each of several sequences of very different lengths."""
    o = ops()
    lens = [1, 64, 65, 128, 129, 700, 2050, 333]
    qs, ks, vs = [], [], []
    for i, n in enumerate(lens):
        qs.append(rnd(n, nh, hd, dtype=torch.bfloat16, seed=7 * i))
        ks.append(rnd(n, nkv, hd, dtype=torch.bfloat16, seed=7 * i + 1))
        vs.append(rnd(n, nkv, hd, dtype=torch.bfloat16, seed=7 * i + 2))
    want = torch.stack([plain.attention(q.float(), k.float(), v.float(), window)[-1]
                        for q, k, v in zip(qs, ks, vs)])
    q = torch.stack([q[-1] for q in qs])
    kc, vc, bt = _paged_many(ks, vs, 70, seed=3)
    row_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32)
    row_seq = torch.arange(len(lens), dtype=torch.int32)
    chunk = o.attention_chunk()
    for mc in (2049 // chunk + 1, 4096 // chunk):          # exact, and a looser bound
        got = o.attention(q.to(DEV), kc.to(DEV), vc.to(DEV), row_pos.to(DEV), row_seq.to(DEV),
                          bt.to(DEV), window, 1 / math.sqrt(hd), mc, decode=True).cpu().float()
        assert o.attn_tc_error() == 0
        err = (got - want).abs().max() / want.abs().max()
        assert err <= 2 ** -7, (mc, err)


@pytest.mark.parametrize("nh,nkv,window,S,normed,rotated,w_dtype", [
    (32, 8, 0, 6, True, True, torch.bfloat16), (8, 1, 0, 1, True, True, torch.float32),
    (5, 1, 70, 3, True, False, torch.bfloat16), (64, 4, 300, 2, False, True, torch.bfloat16),
    (12, 2, 0, 5, False, False, torch.float32)])
def test_attention_decode_makes_q_and_the_new_key_itself(nh, nkv, window, S, normed, rotated,
                                                         w_dtype):
    """The decode kernel that is given the q,k,v product's partial sums makes q and,
    in the CTA that holds the new position's chunk, that position's key and value,
    and writes them to the cache: output and caches equal, bit for bit, those of the
    rope kernel followed by the attention kernel.  New positions at a page's first
    and last place, at a chunk's first place and alone in the sequence; with and
    without norm and rotation; a layer that only reads its cache."""
    o = ops()
    hd = 128
    lens = [1, 64, 65, 128, 129, 700, 2050, 333]
    n = len(lens)
    ks = [rnd(m, nkv, hd, dtype=torch.bfloat16, seed=9 * i + 1) for i, m in enumerate(lens)]
    vs = [rnd(m, nkv, hd, dtype=torch.bfloat16, seed=9 * i + 2) for i, m in enumerate(lens)]
    kc, vc, bt = _paged_many(ks, vs, 70, seed=4)        # the last positions will be overwritten
    width = (nh + 2 * nkv) * hd
    qkv = rnd(S, n, width, seed=77, scale=2.0)
    qw = (1 + 0.2 * rnd(hd, seed=5)).to(w_dtype) if normed else None
    kw = (1 + 0.2 * rnd(hd, seed=6)).to(w_dtype) if normed else None
    if rotated:
        ang = torch.arange(4096)[:, None] * (10000.0 ** (-torch.arange(hd // 2) / (hd // 2)))[None]
        cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    else:
        cos = sin = None
    row_pos = torch.tensor([m - 1 for m in lens], dtype=torch.int32).to(DEV)
    row_seq = torch.arange(n, dtype=torch.int32).to(DEV)
    dev = lambda t: None if t is None else t.to(DEV)
    chunk = o.attention_chunk()
    mc = 2049 // chunk + 1
    if window:
        mc = min(mc, (window - 1) // chunk + 2)
    scale = 1 / math.sqrt(hd)
    for append in (True, False):
        k1, v1, k2, v2 = kc.to(DEV), vc.to(DEV), kc.to(DEV), vc.to(DEV)
        q = o.qk_norm_rope_append(qkv.to(DEV), dev(qw), dev(kw), 1e-6, cos, sin, row_pos, row_seq,
                                  bt.to(DEV), k1 if append else None, v1 if append else None,
                                  nh, nkv, hd, torch.bfloat16)
        want = o.attention(q, k1, v1, row_pos, row_seq, bt.to(DEV), window, scale, mc, decode=True)
        got = o.attention_decode_qkv(qkv.to(DEV), dev(qw), dev(kw), 1e-6, cos, sin, k2, v2, append,
                                     row_pos, row_seq, bt.to(DEV), window, scale, mc, nh)
        assert got is not None and o.attn_tc_error() == 0
        assert torch.equal(k1, k2) and torch.equal(v1, v2)
        assert torch.equal(k1, kc.to(DEV)) != append        # the key was written, or it was not
        assert torch.equal(got, want)
        assert float(want.float().abs().max()) > 0.1


def test_attention_tensor_core_prefill_moves_its_reference():
    """The prefill kernel keeps a row's exponent reference until a chunk's maximum
    runs more than 2^8 ahead, then scales the row's output, which lies in tensor
    memory.  Here the keys of the first chunk score 0, those of the second 2^9.5
    above them and one key of the third another 2^9.5: the 128 keys of an earlier
    chunk together still weigh a good part of what follows, so a wrong factor would
    show."""
    o = ops()
    n, nh, nkv, hd = 400, 8, 2, 128
    q = torch.zeros(n, nh, hd)
    k = torch.zeros(n, nkv, hd)
    v = rnd(n, nkv, hd).to(torch.bfloat16).float()
    q[:, :, 3] = 8.0
    step = 9.5 * math.sqrt(hd) / (8.0 * 1.4426950408889634)
    k[128:256, :, 3] = step
    k[260, :, 3] = 2 * step
    k = k.bfloat16().float()
    want = plain.attention(q.double(), k.double(), v.double(), 0).float()
    kc, vc, bt = _paged_many([k.bfloat16()], [v.bfloat16()], 9, seed=2)
    pos = torch.arange(n, dtype=torch.int32)
    seq = torch.zeros(n, dtype=torch.int32)
    per = o.attention_block_positions(nh, nkv)
    blocks = o.attention_blocks([0], [0], [n], per, torch.device(DEV))
    mc = (n - 1) // o.attention_chunk() + 1
    got = o.attention(q.bfloat16().to(DEV), kc.to(DEV), vc.to(DEV), pos.to(DEV), seq.to(DEV),
                      bt.to(DEV), 0, 1 / math.sqrt(hd), mc, blocks=blocks).cpu().float()
    assert o.attn_tc_error() == 0
    for rows in (slice(0, 128), slice(128, 260), slice(260, n)):     # 0, 1, 2 moves
        err = (got[rows] - want[rows]).abs().max() / want[rows].abs().max()
        assert err <= 2 ** -7, (rows, float(err))
    # the earlier chunks do weigh: without them the answers are others
    alone = v[260].repeat_interleave(nh // nkv, 0)
    assert (want[300] - alone).abs().max() > 10 * 2 ** -7 * want[300].abs().max()
    alone = v[128:131].mean(0).repeat_interleave(nh // nkv, 0)
    assert (want[130] - alone).abs().max() > 3 * 2 ** -7 * want[130].abs().max()


def test_attention_tensor_core_finds_a_far_key():
    """As for the plain kernel: one key among 700 stands out, with and without a
    window, for prefill rows and for a decoded token."""
    o = ops()
    n, nh, nkv, hd = 700, 8, 2, 128
    q = torch.zeros(n, nh, hd)
    k = torch.zeros(n, nkv, hd)
    v = rnd(n, nkv, hd).to(torch.bfloat16).float()
    q[:, :, 3] = 24.0
    k[133, :, 3] = 24.0
    kc, vc, bt = _paged_many([k.bfloat16()], [v.bfloat16()], 12, seed=5)
    pos = torch.arange(n, dtype=torch.int32)
    seq = torch.zeros(n, dtype=torch.int32)
    chunk = o.attention_chunk()
    per = o.attention_block_positions(nh, nkv)
    blocks = o.attention_blocks([0], [0], [n], per, torch.device(DEV))
    for window in (0, 200):
        mc = (n - 1) // chunk + 1
        got = o.attention(q.bfloat16().to(DEV), kc.to(DEV), vc.to(DEV), pos.to(DEV), seq.to(DEV),
                          bt.to(DEV), window, 1 / math.sqrt(hd), mc, blocks=blocks).cpu().float()
        last_seeing = n - 1 if not window else 133 + window - 1
        for r in (133, 134, 300, last_seeing):
            assert (got[r, 5] - v[133, 1]).abs().max() <= 2 ** -7, (window, r)
        if window:
            r = last_seeing + 1
            want = v[r + 1 - window:r + 1, 0].mean(0)
            assert (got[r, 3] - want).abs().max() <= 2 ** -6, (window, r)
        assert (got[99, 0] - v[:100, 0].mean(0)).abs().max() <= 2 ** -6
        # the same rows as decoded tokens
        for r in (133, last_seeing, last_seeing + 1 if window else 500):
            one = o.attention(q[r:r + 1].bfloat16().to(DEV), kc.to(DEV), vc.to(DEV),
                              pos[r:r + 1].to(DEV), seq[:1].to(DEV), bt.to(DEV), window,
                              1 / math.sqrt(hd), mc, decode=True).cpu().float()
            assert (one[0] - got[r]).abs().max() <= 2 ** -6, (window, r)
    assert o.attn_tc_error() == 0
