"""Each CUDA kernel alone against its plain PyTorch reference, at sizes other than the engine's."""

from __future__ import annotations

import pytest
import torch

import kernel_refs as ref
from acvram_b200.kernels.ops import QUERY_TILE

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=2e-5, atol=2e-5) if dtype == torch.float32 else dict(rtol=1.6e-2, atol=1.6e-2)


@pytest.fixture(scope="module")
def ops():
    from acvram_b200.kernels import ops
    ops.library()
    return ops


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, device="cuda", generator=g) * scale).to(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,V,T", [(72, 331, 9), (4096, 1000, 3), (50, 77, 1)])
def test_embed(ops, dtype, H, V, T):
    table = rnd(V, H, dtype=dtype)
    tok = torch.randint(0, V, (T,), device="cuda", dtype=torch.int32)
    out = torch.empty(T, H, device="cuda", dtype=dtype)
    ops.embed(table, tok, out)
    assert torch.equal(out, table[tok.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,H,eps", [(5, 72, 1e-6), (3, 4096, 1e-5), (2, 5120, 1e-6), (1, 13000, 1e-5), (17, 50, 1e-3)])
def test_add_rmsnorm(ops, dtype, T, H, eps):
    x = rnd(T, H, dtype=dtype, seed=1)
    d = rnd(T, H, dtype=dtype, seed=2)
    w = 1 + 0.1 * rnd(H, seed=3)
    # with the residual sum
    x1, x2 = x.clone(), x.clone()
    o1 = ops.add_rmsnorm(x1, d, w, eps, torch.empty_like(x))
    o2 = ref.add_rmsnorm(x2, d, w, eps, torch.empty_like(x))
    torch.testing.assert_close(x1, x2, **tol(dtype))
    torch.testing.assert_close(o1, o2, **tol(dtype))
    # without, and on chosen rows only
    rows = torch.tensor([T - 1, 0], device="cuda", dtype=torch.int32)
    x3 = x.clone()
    o3 = ops.add_rmsnorm(x3, d, w, eps, torch.empty(2, H, device="cuda", dtype=dtype), rows)
    o4 = ref.add_rmsnorm(x.clone(), d, w, eps, torch.empty(2, H, device="cuda", dtype=dtype), rows)
    assert torch.equal(x3, x), "the rows form must leave x as it is"
    torch.testing.assert_close(o3, o4, **tol(dtype))
    o5 = ops.add_rmsnorm(x.clone(), None, w, eps, torch.empty_like(x))
    o6 = ref.add_rmsnorm(x.clone(), None, w, eps, torch.empty_like(x))
    torch.testing.assert_close(o5, o6, **tol(dtype))


def test_rmsnorm_breaking_arm(ops):
    """The comparison can see a fault: a wrong eps moves the result beyond the tolerance."""
    x = rnd(4, 96, scale=0.01, seed=4)
    w = torch.ones(96, device="cuda")
    good = ops.add_rmsnorm(x.clone(), None, w, 1e-6, torch.empty_like(x))
    bad = ref.add_rmsnorm(x.clone(), None, w, 1e-4, torch.empty_like(x))
    assert (good - bad).abs().max() > 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,I", [(7, 176), (2, 12288), (1, 5), (33, 1000)])
def test_swiglu(ops, dtype, T, I):
    gu = rnd(T, 2 * I, dtype=dtype, scale=3.0, seed=5)
    gu[0, 0] = 80.0   # extremes: exp(-g) under- and overflows
    gu[0, 1] = -80.0
    o1 = ops.swiglu(gu, torch.empty(T, I, device="cuda", dtype=dtype))
    o2 = ref.swiglu(gu, torch.empty(T, I, device="cuda", dtype=dtype))
    torch.testing.assert_close(o1, o2, **tol(dtype))
    assert torch.isfinite(o1.float()).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T,N", [(1, 17), (9, 331), (300, 4096)])
def test_add_bias(ops, dtype, T, N):
    out = rnd(T, N + 5, dtype=dtype, seed=21)[:, :N]          # a row stride that is not the width
    bias = rnd(N, seed=22)
    want = out.clone()
    ref.add_bias(want, bias)
    ops.add_bias(out, bias)
    torch.testing.assert_close(out, want, **tol(dtype))


def test_table_update(ops):
    """The (row, column, page) triples of a step reach the block table on the device; what lies outside is skipped."""
    table = torch.full((5, 7), -1, dtype=torch.int32, device="cuda")
    triples = torch.tensor([[0, 0, 11], [4, 6, 12], [2, 3, 14], [5, 0, 15], [0, 7, 16], [-1, 2, 17], [1, 1, 99]],
                           dtype=torch.int32, device="cuda").reshape(-1)
    ops.table_update(table, triples, 6)             # the seventh triple is not part of the step
    want = torch.full((5, 7), -1, dtype=torch.int32)
    want[0, 0], want[4, 6], want[2, 3] = 11, 12, 14
    assert torch.equal(table.cpu(), want)


def _paged_setup(B, lens, NKV, D, page, dtype, n_pages, seed, shuffle=True):
    """Random block tables over a shuffled pool; returns (k_pages, v_pages, table[B, W])."""
    g = torch.Generator().manual_seed(seed)
    W = max((l + page - 1) // page for l in lens)
    perm = torch.randperm(n_pages, generator=g) if shuffle else torch.arange(n_pages)
    table = torch.full((B, W), -1, dtype=torch.int32)
    used = 0
    for b, l in enumerate(lens):
        n = (l + page - 1) // page
        table[b, :n] = perm[used:used + n].to(torch.int32)
        used += n
    assert used <= n_pages
    kp = torch.zeros(n_pages, NKV, page, D, device="cuda", dtype=dtype)
    vp = torch.zeros_like(kp)
    return kp, vp, table.cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("NH,NKV,D,rot,page", [(5, 1, 48, 48, 16), (6, 2, 32, 32, 8), (8, 8, 64, 32, 4), (4, 2, 128, 128, 16),
                                              (3, 3, 16, 16, 32)])
def test_qk_norm_rope_append(ops, dtype, NH, NKV, D, rot, page):
    lens = [19, 3, 40]
    q_lens = [5, 3, 1]   # the last tokens of each request are this step's
    B = len(lens)
    kp, vp, table = _paged_setup(B, lens, NKV, D, page, dtype, 16, seed=7)
    kp2, vp2 = kp.clone(), vp.clone()
    pos = torch.cat([torch.arange(l - q, l) for l, q in zip(lens, q_lens)]).to(torch.int32).cuda()
    seq = torch.cat([torch.full((q,), b) for b, q in enumerate(q_lens)]).to(torch.int32).cuda()
    T = pos.numel()
    qkv = rnd(T, (NH + 2 * NKV) * D, dtype=dtype, seed=8)
    qw, kw = 1 + 0.1 * rnd(D, seed=9), 1 + 0.1 * rnd(D, seed=10)
    inv = 1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    ang = torch.outer(torch.arange(64, dtype=torch.float32), inv)
    cs = torch.cat((ang.cos(), ang.sin()), -1).cuda()
    a, b = qkv.clone(), qkv.clone()
    ops.qk_norm_rope_append(a, NH, NKV, D, qw, kw, 1e-6, cs, pos, seq, table, kp, vp)
    ref.qk_norm_rope_append(b, NH, NKV, D, qw, kw, 1e-6, cs, pos, seq, table, kp2, vp2)
    torch.testing.assert_close(a[:, :NH * D], b[:, :NH * D], **tol(dtype))
    torch.testing.assert_close(kp, kp2, **tol(dtype))
    torch.testing.assert_close(vp, vp2, **tol(dtype))
    # steps alone: norm only (no table, no pages), then append only
    c, d = qkv.clone(), qkv.clone()
    ops.qk_norm_rope_append(c, NH, NKV, D, qw, kw, 1e-6, None, pos, seq, None, None, None)
    ref.qk_norm_rope_append(d, NH, NKV, D, qw, kw, 1e-6, None, pos, seq, None, None, None)
    torch.testing.assert_close(c, d, **tol(dtype))
    kp3, vp3 = torch.zeros_like(kp), torch.zeros_like(vp)
    ops.qk_norm_rope_append(c, NH, NKV, D, None, None, 0.0, None, pos, seq, table, kp3, vp3)
    kp4, vp4 = torch.zeros_like(kp), torch.zeros_like(vp)
    ref.qk_norm_rope_append(d, NH, NKV, D, None, None, 0.0, None, pos, seq, table, kp4, vp4)
    torch.testing.assert_close(kp3, kp4, **tol(dtype))
    torch.testing.assert_close(vp3, vp4, **tol(dtype))


def test_append_skips_negative_page(ops):
    """A page index < 0 writes nothing (it must not wrap to the last page)."""
    NH, NKV, D, page = 2, 1, 16, 4
    kp = torch.zeros(4, NKV, page, D, device="cuda")
    vp = torch.zeros_like(kp)
    table = torch.full((1, 2), -1, dtype=torch.int32, device="cuda")
    qkv = rnd(1, (NH + 2 * NKV) * D, seed=11)
    pos = torch.tensor([5], dtype=torch.int32, device="cuda")
    seq = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.qk_norm_rope_append(qkv, NH, NKV, D, None, None, 0.0, None, pos, seq, table, kp, vp)
    assert kp.abs().sum() == 0 and vp.abs().sum() == 0


def _attention_case(ops, fn, dtype, NH, NKV, D, page, lens, q_lens, window, seed, spike=None):
    B = len(lens)
    n_pages = sum((l + page - 1) // page for l in lens) + 3
    kp, vp, table = _paged_setup(B, lens, NKV, D, page, dtype, n_pages, seed)
    # fill the pages of each request with random keys and values
    g = torch.Generator(device="cuda").manual_seed(seed + 1)
    for b, l in enumerate(lens):
        for j in range(l):
            pg = int(table[b, j // page])
            kp[pg, :, j % page] = torch.randn(NKV, D, device="cuda", generator=g).to(dtype)
            vp[pg, :, j % page] = torch.randn(NKV, D, device="cuda", generator=g).to(dtype)
    pos = torch.cat([torch.arange(l - q, l) for l, q in zip(lens, q_lens)]).to(torch.int32).cuda()
    seq = torch.cat([torch.full((q,), b) for b, q in enumerate(q_lens)]).to(torch.int32).cuda()
    T = pos.numel()
    q = rnd(T, (NH + 2 * NKV) * D, dtype=dtype, seed=seed + 2)
    if spike is not None:
        # make one far key dominate for the last query of request 0: a kernel that loses that
        # key (a page's edge, a tile's edge) is far off, not a little
        b, j = spike
        pg = int(table[b, j // page])
        last = sum(q_lens[:b + 1]) - 1
        for h in range(NH):
            kv = h // (NH // NKV)
            q[last, h * D:(h + 1) * D] = (kp[pg, kv, j % page].float() * 4.0).to(dtype)
    out1 = torch.zeros(T, NH * D, device="cuda", dtype=dtype)
    out2 = torch.zeros_like(out1)
    fn(q, out1, kp, vp, pos, seq, table, NH, NKV, D, D ** -0.5, window)
    ref.attention_generic(q, out2, kp, vp, pos, seq, table, NH, NKV, D, D ** -0.5, window)
    return out1, out2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("NH,NKV,D,page,window", [(5, 1, 48, 16, 0), (6, 2, 32, 8, 0), (4, 4, 16, 4, 0), (8, 2, 128, 16, 0),
                                                 (4, 2, 64, 16, 21), (6, 3, 80, 8, 7), (2, 1, 256, 16, 0)])
def test_attention_generic(ops, dtype, NH, NKV, D, page, window):
    o1, o2 = _attention_case(ops, ops.attention_generic, dtype, NH, NKV, D, page, lens=[150, 33, 1, 64],
                             q_lens=[37, 33, 1, 2], window=window, seed=20)
    torch.testing.assert_close(o1, o2, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_generic_far_key(ops, dtype):
    """One far key among hundreds carries the answer."""
    for j in (0, 15, 16, 255, 256, 300):
        o1, o2 = _attention_case(ops, ops.attention_generic, dtype, 4, 2, 64, 16, lens=[301, 40], q_lens=[1, 3],
                                 window=0, seed=30 + j, spike=(0, j))
        torch.testing.assert_close(o1, o2, **tol(dtype))


@pytest.mark.parametrize("in_dtype,out_dtype", [(torch.float32, torch.float32), (torch.bfloat16, torch.float32),
                                                (torch.bfloat16, torch.bfloat16)])
@pytest.mark.parametrize("M,N,K", [(1, 331, 80), (7, 100, 72), (65, 130, 200), (3, 1000, 4096), (128, 64, 16)])
def test_gemm_simt(ops, in_dtype, out_dtype, M, N, K):
    a = rnd(M, K, dtype=in_dtype, seed=40)
    w = rnd(N, K, dtype=in_dtype, scale=0.05, seed=41)
    out = ops.gemm_simt(a, w, torch.empty(M, N, device="cuda", dtype=out_dtype))
    want = (a.double() @ w.double().T)
    t = dict(rtol=1e-4, atol=1e-4) if out_dtype == torch.float32 else tol(out_dtype)
    torch.testing.assert_close(out.double(), want, **t)


def test_gemm_simt_rows_independent(ops):
    """A row's result does not depend on the other rows of the batch (bit for bit)."""
    a = rnd(37, 300, seed=42)
    w = rnd(91, 300, scale=0.05, seed=43)
    whole = ops.gemm_simt(a, w, torch.empty(37, 91, device="cuda"))
    one = ops.gemm_simt(a[5:6].contiguous(), w, torch.empty(1, 91, device="cuda"))
    assert torch.equal(whole[5:6], one)


@pytest.mark.parametrize("R,V", [(1, 331), (5, 151936), (3, 1000), (64, 4097)])
def test_argmax(ops, R, V):
    lg = rnd(R, V, seed=50)
    lg[0, V - 1] = lg[0, 3] = 50.0   # equal maxima: the lowest index wins
    out = ops.argmax(lg, torch.empty(R, device="cuda", dtype=torch.int32))
    assert out.tolist() == lg.argmax(-1).tolist()
    assert out[0].item() == 3


# ----------------------------------------------------------------------------- tensor-core attention (bfloat16)
class _Ctx:
    pass


def _tc_case(ops, NH, NKV, D, page, lens, q_lens, window, seed, n_splits=None, spike=None, k_growth=0.0):
    """A mixed batch through ops.attention (decode kernel for one-token requests, tile kernel for portions)."""
    dtype = torch.bfloat16
    B = len(lens)
    n_pages = sum((l + page - 1) // page for l in lens) + 3
    kp, vp, table = _paged_setup(B, lens, NKV, D, page, dtype, n_pages, seed)
    g = torch.Generator(device="cuda").manual_seed(seed + 1)
    for b, l in enumerate(lens):
        for j in range(l):
            pg = int(table[b, j // page])
            kp[pg, :, j % page] = (torch.randn(NKV, D, device="cuda", generator=g) * (1.0 + k_growth * j)).to(dtype)
            vp[pg, :, j % page] = torch.randn(NKV, D, device="cuda", generator=g).to(dtype)
    ctx = _Ctx()
    ctx.positions = torch.cat([torch.arange(l - q, l) for l, q in zip(lens, q_lens)]).to(torch.int32).cuda()
    ctx.seq_of_token = torch.cat([torch.full((q,), b) for b, q in enumerate(q_lens)]).to(torch.int32).cuda()
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    ctx.cu_q = torch.tensor(cu, dtype=torch.int32).cuda()
    ctx.kv_len = torch.tensor(lens, dtype=torch.int32).cuda()
    dec = [b for b, q in enumerate(q_lens) if q == 1]
    tiles = [(b, s) for b, q in enumerate(q_lens) if q > 1 for s in range(0, q, QUERY_TILE)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    ctx.work = {"dec_tokens": i32([cu[b] for b in dec]), "dec_seqs": i32(dec), "n_dec": len(dec),
                "tile_seq": i32([t[0] for t in tiles]), "tile_q0": i32([t[1] for t in tiles]), "n_tiles": len(tiles),
                "max_dec_kv": max([lens[b] for b in dec], default=0), "n_splits": n_splits}
    T = cu[-1]
    q = rnd(T, (NH + 2 * NKV) * D, dtype=dtype, seed=seed + 2)
    if spike is not None:
        b, j = spike
        pg = int(table[b, j // page])
        last = cu[b + 1] - 1
        for h in range(NH):
            q[last, h * D:(h + 1) * D] = (kp[pg, h // (NH // NKV), j % page].float() * 3.0).to(dtype)
    out1 = torch.full((T, NH * D), 7.0, device="cuda", dtype=dtype)
    out2 = torch.zeros_like(out1)
    assert ops.tensor_core_attention_takes(dtype, NH, NKV, D)
    ops.attention(q, out1, kp, vp, ctx, table, NH, NKV, D, D ** -0.5, window)
    ref.attention_generic(q, out2, kp, vp, ctx.positions, ctx.seq_of_token, table, NH, NKV, D, D ** -0.5, window)
    return out1, out2


@pytest.mark.parametrize("NH,NKV,D,page", [(8, 2, 128, 16), (6, 2, 64, 8), (5, 1, 64, 16), (16, 1, 128, 32), (4, 4, 128, 4),
                                          (3, 3, 64, 16)])
@pytest.mark.parametrize("n_splits", [1, 2, 5, 8, None])
def test_attention_decode_kernel(ops, NH, NKV, D, page, n_splits):
    o1, o2 = _tc_case(ops, NH, NKV, D, page, lens=[1, 77, 300, 64, 65, 513], q_lens=[1] * 6, window=0, seed=60,
                      n_splits=n_splits)
    torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


@pytest.mark.parametrize("NH,NKV,D,page", [(8, 2, 128, 16), (6, 2, 64, 8), (5, 1, 64, 16), (4, 4, 128, 4)])
def test_attention_chunk_kernel(ops, NH, NKV, D, page):
    # whole prompts, portions after a cached prefix, a portion of two tokens, tiles that end mid-way
    o1, o2 = _tc_case(ops, NH, NKV, D, page, lens=[150, 33, 200, 64, 130, 2], q_lens=[150, 2, 71, 64, 65, 2], window=0,
                      seed=61)
    torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


@pytest.mark.parametrize("window", [1, 7, 64, 100])
def test_tensor_core_attention_window_and_mixed_batch(ops, window):
    o1, o2 = _tc_case(ops, 8, 2, 128, 16, lens=[150, 90, 300, 17, 64], q_lens=[150, 1, 70, 1, 2], window=window, seed=62)
    torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


def test_tensor_core_attention_far_key(ops):
    """One far key among hundreds carries the answer: at a page's edge, a tile's edge, a split's edge."""
    for j in (0, 15, 16, 63, 64, 127, 128, 447, 448, 600):
        for q_lens in ([1, 1], [5, 3]):
            o1, o2 = _tc_case(ops, 4, 2, 128, 16, lens=[601, 40], q_lens=q_lens, window=0, seed=70 + j, spike=(0, j))
            torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


def test_decode_kernel_twice_leaves_its_counters_clean(ops):
    """The split counters go back to zero, so a second call with other shapes is right too."""
    for seed, lens in ((80, [500, 300]), (81, [129, 700, 90])):
        o1, o2 = _tc_case(ops, 8, 2, 128, 16, lens=lens, q_lens=[1] * len(lens), window=0, seed=seed, n_splits=4)
        torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


def _decode_direct(ops, NH, NKV, D, page, lens, n_splits, cluster_merge, seed, spike=None):
    """The split-KV kernel called by itself (every page filled at random), against the float32 reference."""
    dtype = torch.bfloat16
    B = len(lens)
    n_pages = sum((l + page - 1) // page for l in lens) + 3
    kp, vp, table = _paged_setup(B, lens, NKV, D, page, dtype, n_pages, seed)
    kp.copy_(rnd(*kp.shape, dtype=dtype, seed=seed + 1))
    vp.copy_(rnd(*vp.shape, dtype=dtype, seed=seed + 2))
    q = rnd(B, (NH + 2 * NKV) * D, dtype=dtype, seed=seed + 3)
    if spike is not None:
        b, j = spike
        pg = int(table[b, j // page])
        for h in range(NH):
            q[b, h * D:(h + 1) * D] = (kp[pg, h // (NH // NKV), j % page].float() * 3.0).to(dtype)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32).cuda()
    kv_len, ar = i32(lens), i32(list(range(B)))
    out1 = torch.full((B, NH * D), 7.0, device="cuda", dtype=dtype)
    out2 = torch.zeros_like(out1)
    splits = n_splits or ops.decode_plan(B, NH, NKV, D, page, max(lens))[0]
    ops.attention_decode(q, out1, kp, vp, ar, ar, B, kv_len, table, NH, NKV, D, D ** -0.5, 0, splits, max(lens),
                         cluster_merge=cluster_merge)
    ref.attention_generic(q, out2, kp, vp, i32([l - 1 for l in lens]), ar, table, NH, NKV, D, D ** -0.5, 0)
    return out1, out2, splits


@pytest.mark.parametrize("n_splits", [3, 9, 16])
def test_decode_attention_merge_through_scratch_memory(ops, n_splits):
    """Partial results in scratch memory and the merge by the CTA that arrives last (what more than 8 splits, i.e.
    long contexts, use; up to 8 splits ordinarily merge inside a cluster): twice in a row with different shapes,
    so that a counter that did not return to zero or a partial result left over from the first call would show."""
    for seed, NH, NKV, D, page, lens in ((82, 8, 2, 128, 16, [700, 300, 1, 2100]), (83, 6, 2, 64, 8, [129, 1500, 90]),
                                         (84, 8, 2, 128, 16, [640, 33])):
        o1, o2, _ = _decode_direct(ops, NH, NKV, D, page, lens, n_splits, cluster_merge=False, seed=seed)
        torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


@pytest.mark.parametrize("n_splits", [2, 6, 8])
def test_decode_attention_merge_inside_clusters(ops, n_splits):
    """The splits of a request are the CTAs of a cluster: rank 0 keeps its own partial result, the others write theirs
    where rank 0's queries lay.  One far key carries the answer of request 0, in rank 0's part, at the edges of the
    parts and in the last one; 4 and 16 query heads to a kv-head (the partial results are smaller and larger than the
    queries' buffer)."""
    for NH, NKV in ((8, 2), (16, 1)):
        lens = [3000, 517, 40]
        per = -(-max(lens) // n_splits)
        for j in (0, 7, per - 1, per, 2999):
            o1, o2, _ = _decode_direct(ops, NH, NKV, 128, 16, lens, n_splits, cluster_merge=True, seed=90 + j % 5, spike=(0, j))
            torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


def test_decode_attention_long_context_chooses_many_splits(ops):
    """About 60 000 keys: the split count that serving computes is above 8, the merge goes through scratch memory
    and block-table entries beyond the part cached in shared memory are read; one far key at a split's edge carries
    the answer for request 0."""
    lens = [60000, 517]
    n, in_clusters = ops.decode_plan(len(lens), 8, 2, 128, 16, max(lens))
    assert n > 8 and not in_clusters
    per = -(-max(lens) // n)
    for j in (per - 1, per, 5 * per, 59999, 0):
        o1, o2, splits = _decode_direct(ops, 8, 2, 128, 16, lens, None, cluster_merge=True, seed=85 + j % 7, spike=(0, j))
        assert splits == n
        torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


# ----------------------------------------------------------------------------- tcgen05 matrix product
GEMM_SHAPES = [
    # (M, N, K): decode-like (swapped roles) and prefill-like, with edges that fill no tile
    (1, 256, 128), (8, 6144, 4096), (5, 331, 72), (16, 128, 64), (17, 200, 264), (64, 1000, 512), (100, 384, 200),
    (128, 256, 4096), (129, 256, 128), (300, 520, 136), (2048, 512, 1024), (515, 4096, 256),
]


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tc(ops, M, N, K, out_dtype):
    x = rnd(M, K, dtype=torch.bfloat16, seed=90)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=91)
    out = torch.full((M, N), 3.0, device="cuda", dtype=out_dtype)
    ops.gemm_tc(x, w, out)
    want = x.double() @ w.double().T
    assert ops.gemm_status() == 0
    t = dict(rtol=1e-4, atol=1e-4) if out_dtype == torch.float32 else tol(torch.bfloat16)
    torch.testing.assert_close(out.double(), want, **t)


@pytest.mark.parametrize("M,K", [(8, 512), (1, 4096), (300, 256)])
def test_gemm_tc_at_the_real_vocabulary(ops, M, K):
    """The output head of the real models: 151 936 rows of weights, float32 logits (1187 tiles of 128 rows)."""
    N = 151936
    x = rnd(M, K, dtype=torch.bfloat16, seed=98)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=99)
    out = torch.full((M, N), 3.0, device="cuda", dtype=torch.float32)
    ops.gemm_tc(x, w, out, static_weights=True)
    assert ops.gemm_status() == 0
    for n0 in range(0, N, 32768):        # the reference in pieces: a double copy of the whole weight is not needed
        want = x.double() @ w[n0:n0 + 32768].double().T
        torch.testing.assert_close(out[:, n0:n0 + 32768].double(), want, rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("plan", [(1, 16, 1), (1, 16, 4), (1, 32, 3), (1, 64, 2), (1, 128, 5), (0, 64, 1), (0, 128, 2),
                                  (0, 256, 1), (0, 256, 3), (0, 160, 1), (0, 192, 1), (0, 224, 1), (0, 160, 2),
                                  (0, 256, 1, 6, 4), (0, 256, 1, 2, 4)])          # the last two: pairs of CTAs on 256 x 256
def test_gemm_tc_every_tile_shape_and_split(ops, plan):
    M, N, K = (50 if plan[0] else 300), 700, 1160
    if plan[0] and M > plan[1]:
        M = plan[1] - 3
    x = rnd(M, K, dtype=torch.bfloat16, seed=92)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=93)
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.zeros(M, N, device="cuda", dtype=out_dtype)
        ops.gemm_tc(x, w, out, plan)
        assert ops.gemm_status() == 0
        t = dict(rtol=1e-4, atol=1e-4) if out_dtype == torch.float32 else tol(torch.bfloat16)
        torch.testing.assert_close(out.double(), x.double() @ w.double().T, **t)


@pytest.mark.parametrize("M,plan", [(8, None), (8, (1, 16, 4, 4, 0)), (300, None), (300, (0, 256, 1, 4, 4))])
def test_gemm_tc_wait_that_runs_out_leaves_its_code_and_returns(ops, M, plan):
    """A bounded wait made to run out, without a fault: the product is told to poll each barrier a few thousand
    times at most and never to load one k-block.  It has to give up, free what it holds and return, with the
    wait's code in the status word; after the counters are cleared the next launch of the same shape is right.
    M = 8: swapped roles, the splits of K as a cluster / through the work space; M = 300: tokens on the rows, a CTA
    or a pair of CTAs to a tile (in a pair both CTAs' waits run out, each by itself)."""
    N, K = 512, 4096
    x = rnd(M, K, dtype=torch.bfloat16, seed=190)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=191)
    want = x.double() @ w.double().T
    assert ops.gemm_status() == 0
    ops.gemm_tc_test_fault(1 << 12, 5)
    ops.gemm_tc(x, w, torch.zeros(M, N, device="cuda", dtype=torch.float32), plan)
    torch.cuda.synchronize()                 # returns: the kernel ended by itself
    assert ops.gemm_status() in (1, 2, 3, 4)
    ops.reset_after_failure()
    assert ops.gemm_status() == 0
    for _ in range(2):
        out = torch.zeros(M, N, device="cuda", dtype=torch.float32)
        ops.gemm_tc(x, w, out, plan)
        torch.testing.assert_close(out.double(), want, rtol=1e-4, atol=1e-4)
    assert ops.gemm_status() == 0


def test_gemm_tc_strided_rows_and_repeat(ops):
    """x as a column slice of a wider matrix (row stride > K), twice in a row (split counters return to zero)."""
    big = rnd(40, 1024, dtype=torch.bfloat16, seed=94)
    x = big[:, 256:768]
    w = rnd(384, 512, dtype=torch.bfloat16, scale=0.05, seed=95)
    for _ in range(2):
        out = torch.zeros(40, 384, device="cuda", dtype=torch.float32)
        ops.gemm_tc(x, w, out, (1, 64, 4))
        torch.testing.assert_close(out.double(), x.double() @ w.double().T, rtol=1e-4, atol=1e-4)
    assert ops.gemm_status() == 0


def test_gemm_tc_rows_do_not_depend_on_the_batch(ops):
    """The same token gives the same output row alone and among others (same tile shape and split)."""
    x = rnd(16, 512, dtype=torch.bfloat16, seed=96)
    w = rnd(640, 512, dtype=torch.bfloat16, scale=0.05, seed=97)
    whole = ops.gemm_tc(x, w, torch.zeros(16, 640, device="cuda", dtype=torch.float32), (1, 16, 2))
    one = ops.gemm_tc(x[3:4], w, torch.zeros(1, 640, device="cuda", dtype=torch.float32), (1, 16, 2))
    assert torch.equal(whole[3:4], one)


@pytest.mark.parametrize("plan", [None, (1, 16, 1), (1, 16, 3), (1, 64, 2), (0, 256, 1), (0, 128, 2), (0, 64, 1), (0, 256, 1, 6, 4)])
@pytest.mark.parametrize("M,I,K", [(8, 352, 512), (40, 1000, 264), (300, 520, 1160)])
def test_gemm_tc_fused_swiglu(ops, plan, M, I, K):
    """The paired epilogue equals the stacked product followed by the SwiGLU kernel, bit for bit."""
    if plan is not None and plan[0] == 1 and M > plan[1]:
        pytest.skip("more tokens than the tile's narrow side")
    x = rnd(M, K, dtype=torch.bfloat16, seed=98)
    wg = rnd(I, K, dtype=torch.bfloat16, scale=0.05, seed=99)
    wu = rnd(I, K, dtype=torch.bfloat16, scale=0.05, seed=100)
    pairs = torch.stack([wg, wu], dim=1).reshape(2 * I, K).contiguous()
    got = ops.gemm_tc(x, pairs, torch.zeros(M, I, device="cuda", dtype=torch.bfloat16), plan, swiglu_pairs=True)
    gu = ops.gemm_tc(x, torch.cat([wg, wu]).contiguous(), torch.zeros(M, 2 * I, device="cuda", dtype=torch.bfloat16), plan)
    want = ops.swiglu(gu, torch.zeros(M, I, device="cuda", dtype=torch.bfloat16))
    assert ops.gemm_status() == 0
    assert torch.equal(got, want)
    torch.testing.assert_close(got, ref.swiglu((x.float() @ torch.cat([wg, wu]).float().T).bfloat16(),
                                               torch.zeros(M, I, device="cuda", dtype=torch.bfloat16)), **tol(torch.bfloat16))


@pytest.mark.parametrize("M,N,K", [(2100, 2304, 200), (5000, 520, 136), (257, 256, 64), (256, 4104, 72), (9000, 264, 4096)])
def test_gemm_tc_pairs_of_ctas(ops, M, N, K):
    """Tiles of 256 x 256 on pairs of CTAs (tcgen05 cta_group::2): more tiles than pairs (a pair walks several, the
    accumulator buffers alternate), groups of tile rows of which the last is short, edges that fill no tile, one
    k-block and many; and the plan picks this form by itself for a prompt's shapes."""
    x = rnd(M, K, dtype=torch.bfloat16, seed=196)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=197)
    want = x.double() @ w.double().T
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.full((M, N), 3.0, device="cuda", dtype=out_dtype)
        ops.gemm_tc(x, w, out, (0, 256, 1, 6, ops.GEMM_PAIR), static_weights=out_dtype == torch.bfloat16)
        assert ops.gemm_status() == 0
        t = dict(rtol=1e-4, atol=1e-4) if out_dtype == torch.float32 else tol(torch.bfloat16)
        torch.testing.assert_close(out.double(), want, **t)
    assert ops.gemm_tc_plan(2048, 4096, 4096, 148)[4:] == (ops.GEMM_PAIR,)
    assert len(ops.gemm_tc_plan(1056, 34816, 5120, 148)) == 4       # 1280 rows of pair tiles for 1056 tokens: not worth it


def test_tensor_core_attention_growing_scores(ops):
    """Keys whose scores grow along a long prompt: the running maximum moves in every tile of keys, far enough
    that the rows of O are rescaled again and again (and by different amounts in the rows of one warp)."""
    for q_lens, lens in (([700, 130], [700, 400]), ([257, 2], [900, 514])):
        o1, o2 = _tc_case(ops, 6, 2, 128, 16, lens=lens, q_lens=q_lens, window=0, seed=91, k_growth=1.0 / 20.0)
        torch.testing.assert_close(o1, o2, **tol(torch.bfloat16))


@pytest.mark.parametrize("NH,NKV,D,T,K", [(32, 8, 128, 8, 4096), (6, 2, 64, 5, 264), (5, 1, 64, 17, 128), (4, 4, 128, 1, 512),
                                          (3, 1, 128, 32, 136),
                                          # many tokens: tokens on the tensor-memory lanes, whole heads inside a thread's row
                                          (8, 2, 128, 300, 512), (6, 2, 64, 129, 264), (5, 1, 64, 700, 128), (3, 1, 128, 257, 136)])
@pytest.mark.parametrize("normed,rotated,pair", [(True, True, False), (False, True, False), (True, False, False), (True, True, True)])
def test_gemm_tc_qkv_epilogue(ops, NH, NKV, D, T, K, normed, rotated, pair):
    """The stacked projection with norm, rotation and append in its own kernel against the projection followed by the
    rotation kernel: the same queries, and the same keys and values in the same pages (the sums of squares are added
    in another order, so a rounding may move here and there)."""
    page, n_pages = 16, 12
    N = (NH + 2 * NKV) * D
    x = rnd(T, K, dtype=torch.bfloat16, seed=150)
    w = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=151)
    qw = (1.0 + 0.1 * rnd(D, dtype=torch.float32, seed=152)) if normed else None
    kw = (1.0 + 0.1 * rnd(D, dtype=torch.float32, seed=153)) if normed else None
    table_rows = max(200, T)
    ang = torch.rand(table_rows, D // 2, device="cuda") * 6.28
    cos_sin = torch.cat([ang.cos(), ang.sin()], dim=1).contiguous() if rotated else None
    # tokens of three requests at scattered positions; one token's page is missing (-1)
    seq = torch.tensor([i % 3 for i in range(T)], dtype=torch.int32, device="cuda")
    pos = torch.tensor([(7 * i + 3) % 150 if T <= 32 else i // 3 for i in range(T)], dtype=torch.int32, device="cuda")
    per_request = int(pos.max()) // page + 1
    n_pages = 3 * per_request + 2
    table = torch.randperm(n_pages, device="cuda").to(torch.int32)[:3 * per_request].view(3, per_request).contiguous()
    if T > 2:
        table[int(seq[2]), int(pos[2]) // page] = -1
    if not ops.gemm_tc_qkv_takes(x, w, D, cos_sin, torch.empty(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16)):
        pytest.skip("no fused form for this plan")
    if pair and T <= 128:
        pytest.skip("pairs of CTAs serve the tokens-on-rows form")
    plan = (0, 256, 1, 6, ops.GEMM_PAIR) if pair else None
    kp1 = torch.zeros(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16)
    vp1, kp2, vp2 = torch.zeros_like(kp1), torch.zeros_like(kp1), torch.zeros_like(kp1)
    want = ops.gemm_tc(x, w, torch.zeros(T, N, device="cuda", dtype=torch.bfloat16))
    ops.qk_norm_rope_append(want, NH, NKV, D, qw, kw, 1e-6, cos_sin, pos, seq, table, kp1, vp1)
    got = torch.zeros(T, N, device="cuda", dtype=torch.bfloat16)
    ops.gemm_tc_qkv(x, w, got, NH, NKV, D, qw, kw, 1e-6, cos_sin, pos, seq, table, kp2, vp2, plan=plan)
    assert ops.gemm_status() == 0
    q1, q2 = want[:, :NH * D], got[:, :NH * D]
    torch.testing.assert_close(q2, q1, **tol(torch.bfloat16))
    torch.testing.assert_close(kp2, kp1, **tol(torch.bfloat16))
    assert torch.equal(vp2, vp1)
    assert (q2 != q1).float().mean() < 0.02 and (kp2 != kp1).float().mean() < 0.02
