"""Each CUDA kernel alone against its plain torch statement, at sizes the tiny models do not
have: head sizes in steps of 16, group sizes that are no power of two, widths and vocabularies
that are no power of two, page sizes 4 to 64, windows, and inputs made so that one far key or
one page's edge decides the result."""

from __future__ import annotations

from types import SimpleNamespace

import pytest
import torch

import plain_llama
import plain_ops

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def ops():
    from llmserve_triton_kernels_b200 import ops as o

    return o


def tol(dtype, scale=1.0):
    return dict(atol=(2e-6 if dtype == torch.float32 else 1.6e-2) * scale, rtol=(1e-5 if dtype == torch.float32 else 1.6e-2))


def rnd(*shape, dtype=torch.float32, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * std).to(dtype).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden,n", [(300, 72, 5), (1000, 2048, 33), (17, 16, 1)])
def test_embed(dtype, vocab, hidden, n):
    table = rnd(vocab, hidden, dtype=dtype)
    ids = torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(1)).to(torch.int32).to(DEV)
    got = ops().embed(ids, table)
    assert got.dtype == torch.float32
    torch.testing.assert_close(got, plain_ops.embed(ids, table), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,n", [(72, 7), (2048, 19), (5000, 3), (16, 1)])
@pytest.mark.parametrize("eps", [1e-5, 1e-2])
def test_rmsnorm_with_residual_sum(dtype, hidden, n, eps):
    resid = rnd(n, hidden, seed=2)
    delta = rnd(n, hidden, dtype=dtype, seed=3)
    weight = 1 + rnd(hidden, seed=4, std=0.1)
    want_resid = resid.clone()
    want = plain_ops.rmsnorm(want_resid, weight, eps, delta=delta, out_dtype=dtype)
    got = ops().rmsnorm(resid, weight, eps, delta=delta, out_dtype=dtype)
    torch.testing.assert_close(resid, want_resid, atol=1e-6, rtol=1e-6)  # the sum was written back
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))
    # chosen rows only: nothing is written back
    rows = torch.tensor([n - 1, 0], dtype=torch.int32, device=DEV)
    before = resid.clone()
    got_rows = ops().rmsnorm(resid, weight, eps, delta=delta, rows=rows, out_dtype=dtype)
    torch.testing.assert_close(resid, before, atol=0, rtol=0)
    want_rows = plain_ops.rmsnorm(before.clone(), weight, eps, delta=delta, rows=rows, out_dtype=dtype)
    torch.testing.assert_close(got_rows.float(), want_rows.float(), **tol(dtype))
    # without a delta
    torch.testing.assert_close(
        ops().rmsnorm(resid, weight, eps, out_dtype=dtype).float(),
        plain_ops.rmsnorm(resid.clone(), weight, eps, out_dtype=dtype).float(), **tol(dtype))


@pytest.mark.parametrize("m,n,k", [(1, 40, 24), (7, 172, 64), (65, 129, 173), (130, 64, 2048), (3, 1000, 5)])
def test_linear_float32_is_true_32_bit_and_row_independent(m, n, k):
    x, w = rnd(m, k, seed=5), rnd(n, k, seed=6)
    got = ops().linear(x, w)
    want = (x.double() @ w.double().t()).float()
    # ~8 standard deviations of the rounding of a sum of K/16 partial sums of unit-variance terms
    torch.testing.assert_close(got, want, atol=4e-6 * k**0.5, rtol=1e-5)
    # a row's result is bit-identical whatever else is in the batch
    alone = ops().linear(x[m - 1 : m].contiguous(), w)
    assert torch.equal(alone[0], got[m - 1])


@pytest.mark.parametrize(
    "m,n,k",
    [(1, 48, 64), (9, 344, 96), (130, 2560, 2048), (64, 100, 172), (8, 2560, 2048), (64, 11264, 2048), (33, 2048, 5632),
     (5, 40, 72), (17, 100, 48), (3, 64, 88), (16, 17, 8), (1, 32000, 2048), (2048, 2048, 5632), (257, 129, 8), (128, 128, 64),
     (1000, 3000, 1096), (5, 2048, 5632), (8, 1000, 3008), (1, 2368, 6144), (13, 2048, 5632), (16, 4096, 11008),
     (7, 3000, 28672)],
)
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("policy", ["own", "auto"])
def test_linear_bfloat16(m, n, k, out_dtype, policy, monkeypatch):
    """``own``: products of 128 rows and more on the tcgen05 kernel; ``auto``: as in serving (plain products of more
    than 16 rows are the library's)."""
    monkeypatch.setattr(ops(), "_GEMM_POLICY", policy)
    x, w = rnd(m, k, dtype=torch.bfloat16, seed=7), rnd(n, k, dtype=torch.bfloat16, seed=8, std=0.05)
    got = ops().linear(x, w, out_dtype=out_dtype)
    assert got.dtype == out_dtype
    want = x.double() @ w.double().t()
    torch.testing.assert_close(got.double(), want, atol=2e-2 * 0.05 * k**0.5, rtol=1e-2)


@pytest.mark.parametrize("m,inter,k", [(1, 5632, 2048), (8, 172 * 8, 64), (16, 100, 96), (5, 16, 8), (17, 100, 96), (300, 5632, 2048),
                                       (129, 200, 72), (2048, 1000, 256), (64, 5632, 2048), (127, 172 * 8, 64), (33, 100, 96),
                                       (50, 102, 104), (3, 1184, 4096), (8, 500, 2304), (16, 1184, 4096), (11, 3000, 14336)])
@pytest.mark.parametrize("policy", ["own", "auto"])
def test_linear_swiglu_fused_for_few_rows(m, inter, k, policy, monkeypatch):
    monkeypatch.setattr(ops(), "_GEMM_POLICY", policy)
    x = rnd(m, k, dtype=torch.bfloat16, seed=31)
    w = rnd(2 * inter, k, dtype=torch.bfloat16, seed=32, std=0.05)
    got = ops().linear_swiglu(x, w)
    gate_up = x.double() @ w.double().t()
    want = torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]
    torch.testing.assert_close(got.double(), want, atol=2e-2 * 0.05 * k**0.5, rtol=2e-2)


@pytest.mark.parametrize("m", [1, 3, 5, 8, 11, 16])
@pytest.mark.parametrize("inter", [5632, 1184])
def test_weight_streaming_product_when_warps_reach_their_first_box_early(m, inter):
    """A short k (x stays in registers, no meeting of the CTA before the first product) with fewer rows than warps:
    the warps without a row to scale reach their first box of weights while it is still on its way, and with several
    tiles a CTA the slot is asked for again as soon as it is read.  Repeated, with a factored norm and without, since
    what goes wrong here goes wrong in some runs only."""
    o = ops()
    k, parts, eps = 2048, 128, 1e-5
    w = rnd(2 * inter, k, dtype=torch.bfloat16, seed=61, std=0.02)
    for rep in range(6):
        resid = rnd(m, k, seed=62 + rep, std=1.0 + rep % 3)
        norm_w = 1 + rnd(k, seed=70, std=0.1)
        xw = (resid * norm_w).to(torch.bfloat16)
        ss = resid.view(m, parts, k // parts).pow(2).sum(-1).t().contiguous()
        scale = torch.rsqrt(resid.double().pow(2).mean(-1, keepdim=True) + eps)
        for x_in, x_plain in ((o.NormedInput(xw, ss, eps), xw.double() * scale), (xw, xw.double())):
            got = o.linear_swiglu(x_in, w)
            gate_up = x_plain @ w.double().t()
            want = torch.nn.functional.silu(gate_up[:, :inter]) * gate_up[:, inter:]
            torch.testing.assert_close(got.double(), want, atol=0.03, rtol=0.02)


@pytest.mark.parametrize("m,hidden,k,n_next", [(1, 2048, 5632, 2560), (8, 2048, 2048, 11264), (16, 96, 256, 40), (3, 72, 64, 172),
                                              (5, 128, 320, 100), (128, 96, 256, 40), (300, 2048, 5632, 2560), (2048, 2048, 2048, 11264),
                                              (131, 72, 24, 172), (8, 2048, 5632, 2560), (7, 1000, 3008, 172), (16, 2048, 5632, 2560),
                                              (12, 4096, 11008, 100)])
def test_residual_sink_and_factored_norm(m, hidden, k, n_next):
    """A product that adds into the residual stream and hands it on in factored normalised form,
    and the next product that consumes that form: together they must equal
    ``resid += x w^T``, the RMS norm of it, and the next product, done plainly."""
    o = ops()
    x = rnd(m, k, dtype=torch.bfloat16, seed=41)
    w = rnd(hidden, k, dtype=torch.bfloat16, seed=42, std=0.05)
    resid = rnd(m, hidden, seed=43)
    norm_w = 1 + rnd(hidden, seed=44, std=0.1)
    w_next = rnd(n_next, hidden, dtype=torch.bfloat16, seed=45, std=0.05)
    eps = 1e-5
    want_resid = resid.double() + x.double() @ w.double().t()
    want_norm = want_resid * torch.rsqrt(want_resid.pow(2).mean(-1, keepdim=True) + eps) * norm_w.double()
    want_next = want_norm @ w_next.double().t()

    before = resid.clone()
    sink = o.ResidualSink(resid, norm_w, eps)
    # few rows: the weight-streaming kernel; many: the own tcgen05 kernel's end (kept under test; serving lets the
    # library's product add into the stream, below)
    handed = sink.linear(x, w) if m <= 16 else sink.linear_tcgen05(x, w)
    assert isinstance(handed, o.NormedInput)
    torch.testing.assert_close(resid.double(), want_resid, atol=2e-2 * 0.05 * k**0.5, rtol=1e-2)
    torch.testing.assert_close(handed.materialize().double(), want_norm, atol=3e-2, rtol=2e-2)
    if m > 16:
        stream = before.clone()
        assert o.ResidualSink(stream, None, 0.0).linear(x, w) is o.ADDED
        torch.testing.assert_close(stream.double(), want_resid, atol=2e-2 * 0.05 * k**0.5, rtol=1e-2)
    got_next = o.linear(handed, w_next, out_dtype=torch.float32)
    torch.testing.assert_close(got_next.double(), want_next, atol=3e-2 * 0.05 * hidden**0.5, rtol=2e-2)
    if n_next % 2 == 0:
        got_act = o.linear_swiglu(handed, w_next)
        half = n_next // 2
        want_act = torch.nn.functional.silu(want_next[:, :half]) * want_next[:, half:]
        # d(silu(g) u) <= |u| dg + |silu(g)| du, with dg and du bounded as for got_next above
        bound = 3e-2 * 0.05 * hidden**0.5 * (1 + float(want_next.abs().max()))
        torch.testing.assert_close(got_act.double(), want_act, atol=bound, rtol=3e-2)


@pytest.mark.parametrize("m,H,KV,D,hidden,page_size,rotate", [(1, 32, 4, 64, 2048, 16, True), (8, 4, 2, 16, 64, 8, True),
                                                            (16, 3, 1, 32, 192, 4, True), (5, 6, 3, 128, 320, 16, False),
                                                            (2, 5, 0, 48, 128, 1, True), (9, 32, 4, 64, 2048, 16, True),
                                                            (4, 8, 2, 64, 4096, 16, True), (12, 8, 2, 128, 4096, 16, True)])
def test_linear_qkv_rope_fused_for_few_rows(m, H, KV, D, hidden, page_size, rotate):
    """Projection, rotation and cache write in one kernel against the three done plainly."""
    o = ops()
    x = rnd(m, hidden, dtype=torch.bfloat16, seed=51)
    w = rnd((H + 2 * KV) * D, hidden, dtype=torch.bfloat16, seed=52, std=0.1)
    cos, sin = plain_llama.rope_cos_sin(torch.arange(200), D, 1234.0)
    table = torch.cat((cos[:, : D // 2], sin[:, : D // 2]), dim=-1).contiguous().to(DEV) if rotate else None
    positions = torch.randint(0, 200, (m,), generator=torch.Generator().manual_seed(3)).to(torch.int32).to(DEV)
    pages = 12
    slot_map = torch.randperm(pages * page_size, generator=torch.Generator().manual_seed(4))[:m].to(torch.int32).to(DEV)
    pool_a = torch.zeros(pages, 2, max(KV, 1), page_size, D, dtype=torch.bfloat16, device=DEV) if KV else None
    pool_b = pool_a.clone() if KV else None
    got_q = o.linear_qkv_rope(x, w, positions, table, slot_map if KV else None, pool_a, H, KV, D, write_kv=KV > 0)
    assert got_q is not None
    # a width that is no multiple of 64 (the weights travel in pieces of 64) is not taken: the caller goes the other way
    assert o.linear_qkv_rope(x[:, :40].contiguous(), w[:, :40].contiguous(), positions, table, slot_map if KV else None, pool_a, H, KV, D,
                             write_kv=KV > 0) is None
    qkv = plain_ops.linear(x, w, out_dtype=torch.float32)  # the plain chain keeps 32 bits until the stores
    plain_ops.rope_kv_write(qkv, positions, table, slot_map if KV else None, pool_b, H, KV, D, write_kv=KV > 0)
    scale = float(qkv.abs().max())
    torch.testing.assert_close(got_q.float(), qkv[:, : H * D], atol=1e-2 * scale, rtol=1.6e-2)
    if KV:
        torch.testing.assert_close(pool_a.float(), pool_b.float(), atol=1e-2 * scale, rtol=1.6e-2)
        assert float(pool_a.float().abs().sum()) > 0


def make_cache(requests, KV, D, page_size, dtype, seed=0, shuffle=True):
    """A pool with the keys and values of ``requests`` (list of context lengths) on shuffled pages."""
    pages_of = [-(-n // page_size) for n in requests]
    total = sum(pages_of) + 3
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed)) if shuffle else torch.arange(total)
    pool = torch.zeros(total, 2, KV, page_size, D, dtype=dtype, device=DEV)
    width = max(pages_of)
    table = torch.zeros(len(requests), width, dtype=torch.int32)
    keys, values, at = [], [], 0
    for r, n in enumerate(requests):
        k, v = rnd(n, KV, D, seed=seed + 10 + r), rnd(n, KV, D, seed=seed + 50 + r)
        keys.append(k)
        values.append(v)
        table[r, : pages_of[r]] = perm[at : at + pages_of[r]].to(torch.int32)
        at += pages_of[r]
    return pool, table.to(DEV), keys, values


def fill_pool(pool, table, keys, values, page_size):
    for r, (k, v) in enumerate(zip(keys, values)):
        for j in range(k.shape[0]):
            page, off = int(table[r, j // page_size]), j % page_size
            pool[page, 0, :, off] = k[j].to(pool.dtype)
            pool[page, 1, :, off] = v[j].to(pool.dtype)


def step_ctx(ctx_lens, q_lens):
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    token_request = [r for r, q in enumerate(q_lens) for _ in range(q)]
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    return SimpleNamespace(cu_tokens=i32(cu), context_lens=i32(ctx_lens), token_request=i32(token_request))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize(
    "H,KV,D,page_size,window",
    [(4, 2, 16, 16, None), (3, 1, 32, 8, None), (6, 2, 48, 4, None), (8, 8, 64, 16, 9), (5, 5, 80, 32, None),
     (12, 4, 128, 64, 33), (2, 1, 256, 16, None), (7, 7, 112, 16, 1), (5, 5, 20, 8, None), (4, 2, 100, 16, 7), (3, 1, 6, 4, None)],
)
def test_paged_attention_mixed_batch(dtype, H, KV, D, page_size, window):
    ctx_lens, q_lens = [70, 1, 33, 129, 17], [5, 1, 33, 1, 2]  # a portion, a first token, a whole prompt, decodes
    pool, table, keys, values = make_cache(ctx_lens, KV, D, page_size, dtype)
    fill_pool(pool, table, keys, values, page_size)
    ctx = step_ctx(ctx_lens, q_lens)
    n = sum(q_lens)
    q = rnd(n, H * D + 24, dtype=dtype, seed=99)  # rows are wider than the query heads, as in a fused projection
    kw = dict(num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5, window=window)
    got = ops().paged_attention(q, pool, table, ctx, **kw)
    want = plain_ops.paged_attention(q, pool, table, ctx, **kw)
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize(
    "H,KV,D,page_size,window",
    [(32, 4, 64, 16, None), (8, 2, 128, 16, None), (6, 2, 32, 8, 50), (4, 4, 16, 4, None), (16, 2, 64, 64, 130),
     (3, 1, 128, 32, 700)],
)
@pytest.mark.parametrize("general_kernel", [False, True])
def test_paged_attention_long_portions_bfloat16(H, KV, D, page_size, window, general_kernel, monkeypatch):
    """Portions of hundreds of tokens beside decode tokens at contexts beyond a thousand: the
    tensor-core kernel's 64-row tiles, its split keys and their merge; and the general kernel
    on the same inputs."""
    monkeypatch.setattr(ops(), "_FORCE_GENERIC_ATTENTION", general_kernel)
    ctx_lens, q_lens = [500, 333, 64, 1200, 130], [300, 333, 3, 1, 2]
    pool, table, keys, values = make_cache(ctx_lens, KV, D, page_size, torch.bfloat16, seed=21)
    pool_filled = torch.zeros_like(pool)
    for r, (k, v) in enumerate(zip(keys, values)):  # vectorised fill
        n = k.shape[0]
        j = torch.arange(n, device=DEV)
        page = table[r].long()[j // page_size]
        pool_filled[page, 0, :, j % page_size] = k.to(torch.bfloat16)
        pool_filled[page, 1, :, j % page_size] = v.to(torch.bfloat16)
    ctx = step_ctx(ctx_lens, q_lens)
    q = rnd(sum(q_lens), (H + 2 * KV) * D, dtype=torch.bfloat16, seed=98)
    kw = dict(num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5, window=window)
    got = ops().paged_attention(q, pool_filled, table, ctx, **kw)
    want = plain_ops.paged_attention(q, pool_filled, table, ctx, **kw)
    torch.testing.assert_close(got.float(), want.float(), **tol(torch.bfloat16))


def _filled(ctx_lens, KV, D, page_size, seed, key_scale=1.0):
    pool, table, keys, values = make_cache(ctx_lens, KV, D, page_size, torch.bfloat16, seed=seed)
    filled = torch.zeros_like(pool)
    for r, (k, v) in enumerate(zip(keys, values)):
        j = torch.arange(k.shape[0], device=DEV)
        page = table[r].long()[j // page_size]
        filled[page, 0, :, j % page_size] = (k * key_scale).to(torch.bfloat16)
        filled[page, 1, :, j % page_size] = v.to(torch.bfloat16)
    return filled, table, keys, values


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("H,KV,page_size,window", [(32, 4, 16, None), (8, 8, 8, None), (6, 2, 32, 200), (4, 1, 64, 64), (2, 2, 16, 1),
                                                   (3, 1, 16, 129)])
def test_paged_attention_tcgen05_portions(H, KV, page_size, window, D, monkeypatch):
    """Portions of 128 tokens and more at head sizes 64 and 128 run on tcgen05 (128-token tiles of one head, 64 keys a
    time): whole prompts of exactly one and two tiles, portions behind hundreds of cached tokens, ragged ends,
    windows that end inside a tile, beside short portions and decode tokens that take the other kernels."""
    ctx_lens, q_lens = [128, 700, 1700, 129, 5, 256, 40], [128, 572, 1000, 129, 1, 256, 40]
    pool, table, _, _ = _filled(ctx_lens, KV, D, page_size, seed=31)
    ctx = step_ctx(ctx_lens, q_lens)
    q = rnd(sum(q_lens), (H + 2 * KV) * D, dtype=torch.bfloat16, seed=97)
    kw = dict(num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5, window=window)
    launched = {}
    real = ops()._launch

    def recording(name, *a):
        launched[name] = real(name, *a)
        return launched[name]

    monkeypatch.setattr(ops(), "_launch", recording)
    got = ops().paged_attention(q, pool, table, ctx, **kw)
    assert launched == {"llm_attention_tcgen05": 0, "llm_attention_mma_routed": 0}
    ops().check_device_errors()
    want = plain_ops.paged_attention(q, pool, table, ctx, **kw)
    torch.testing.assert_close(got.float(), want.float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("far_key", [0, 63, 64, 499, 500, 563, 564, 627, 628, 899])
def test_paged_attention_tcgen05_finds_one_far_key(far_key, D):
    """A portion of 400 tokens behind 500 cached ones; one key is made to match every query.  Every token at or
    behind that key must return the key's value, whichever tile, page or stage of the ring the key lies in."""
    H, KV, page_size, n, q_len = 4, 2, 16, 900, 400
    pool, table, keys, values = make_cache([n], KV, D, page_size, torch.bfloat16, seed=3)
    direction = torch.nn.functional.normalize(rnd(D, seed=6), dim=0)
    keys[0][:] = keys[0] * 0.05
    keys[0][far_key] = direction * 24
    fill_pool(pool, table, keys, values, page_size)
    q = rnd(q_len, H * D, dtype=torch.bfloat16, seed=5, std=0.1)
    q.view(q_len, H, D)[:] = (direction * 24).to(torch.bfloat16)
    ctx = step_ctx([n], [q_len])
    kw = dict(num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5)
    got = ops().paged_attention(q, pool, table, ctx, **kw).float()
    ops().check_device_errors()
    first = max(0, far_key - (n - q_len))  # the first token of the portion that sees the key
    want = values[0][far_key].to(torch.bfloat16).float().repeat_interleave(H // KV, dim=0).reshape(1, H * D)
    torch.testing.assert_close(got[first:], want.expand(q_len - first, -1), atol=2e-2, rtol=2e-2)
    plain = plain_ops.paged_attention(q, pool, table, ctx, **kw).float()
    torch.testing.assert_close(got, plain, **tol(torch.bfloat16))


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("rise", [0.02, 0.08, 0.3])
def test_paged_attention_tcgen05_scores_that_keep_rising(rise, D):
    """The tcgen05 kernel keeps its output in tensor memory and rescales a row only when its maximum has risen by more than
    2^8 since the row's shift was last set.  Here every key scores higher than the one before it, by ``rise`` nats a
    key: the shift is left behind and follows in jumps (every 277, 69 or 18 keys), several times inside one portion, and the keys just before a jump carry weights of up to 2^8 against the stale shift.  A jump that is missed,
    scaled wrongly or applied a tile late shows against the plain attention, whose weights fall off over the last few
    keys only."""
    H, KV, page_size, n, q_len = 4, 2, 16, 1100, 600
    pool, table, keys, values = make_cache([n], KV, D, page_size, torch.bfloat16, seed=8)
    direction = torch.nn.functional.normalize(rnd(D, seed=9), dim=0)
    ramp = torch.arange(n, device=DEV, dtype=torch.float32) * rise  # the score of key j, before the scale by 1/sqrt(D)
    keys[0][:] = keys[0] * 0.02 + (ramp[:, None, None] * direction) * (D**0.5 / 8.0)
    fill_pool(pool, table, keys, values, page_size)
    q = rnd(q_len, H * D, dtype=torch.bfloat16, seed=10, std=0.05)
    q.view(q_len, H, D)[:] += (direction * 8.0).to(torch.bfloat16)
    ctx = step_ctx([n], [q_len])
    kw = dict(num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5)
    got = ops().paged_attention(q, pool, table, ctx, **kw).float()
    ops().check_device_errors()
    plain = plain_ops.paged_attention(q, pool, table, ctx, **kw).float()
    torch.testing.assert_close(got, plain, **tol(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far_key,n", [(0, 701), (15, 701), (16, 701), (511, 701), (512, 701), (700, 701), (0, 2101), (1023, 2101),
                                       (1024, 2101), (2100, 2101)])
def test_paged_attention_finds_one_far_key(dtype, far_key, n):
    """One key among hundreds (or two thousand: several splits of the keys, merged) is made to match
    the query: the output must be that key's value.  A kernel that loses a key at a page's edge,
    a chunk's edge or a split's edge would return an average."""
    H, KV, D, page_size = 4, 2, 64, 16
    pool, table, keys, values = make_cache([n], KV, D, page_size, dtype, seed=3)
    q = rnd(1, H * D, dtype=dtype, seed=5, std=0.1)
    direction = torch.nn.functional.normalize(rnd(D, seed=6), dim=0)
    q.view(H, D)[:] = (direction * 24).to(dtype)
    keys[0][:] = keys[0] * 0.05
    keys[0][far_key] = direction * 24
    fill_pool(pool, table, keys, values, page_size)
    ctx = step_ctx([n], [1])
    got = ops().paged_attention(q, pool, table, ctx, num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5)
    want = values[0][far_key].to(dtype).float().repeat_interleave(H // KV, dim=0).reshape(1, H * D)
    torch.testing.assert_close(got.float(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("H,KV,D", [(8, 4, 64), (4, 4, 32), (8, 4, 128)])
def test_paged_attention_many_requests_each_finds_its_far_key(H, KV, D, monkeypatch):
    """Forty decoding requests with four key/value heads: more (request, head) pairs than the GPU has SMs, which takes
    the split-key kernel's eight-warp shape with 128-key tiles, two CTAs to an SM.  Contexts run from 1 to 2,100 keys;
    in every request one key — the first, the last, one at a tile's or a split's edge — is made to match the query, and
    the output must be that key's value.  The general kernel is run on the same inputs."""
    page_size, R = 16, 40
    g = torch.Generator().manual_seed(9)
    ctx_lens = [1, 2, 15, 16, 17, 127, 128, 129, 255, 256, 257, 383, 384, 385, 511, 512, 513, 1023, 1024, 1025, 2047, 2048, 2100]
    ctx_lens += torch.randint(1, 2101, (R - len(ctx_lens),), generator=g).tolist()
    far = []
    for i, n in enumerate(ctx_lens):
        choices = [0, n - 1, n // 2, min(n - 1, 127), min(n - 1, 128), max(0, n - 129), max(0, n - 128)]
        far.append(choices[i % len(choices)])
    pool, table, keys, values = make_cache(ctx_lens, KV, D, page_size, torch.bfloat16, seed=13)
    direction = torch.nn.functional.normalize(rnd(D, seed=6), dim=0)
    for r in range(R):
        keys[r][:] = keys[r] * 0.05
        keys[r][far[r]] = direction * 24
    filled = torch.zeros_like(pool)
    for r, (k, v) in enumerate(zip(keys, values)):
        j = torch.arange(k.shape[0], device=DEV)
        page = table[r].long()[j // page_size]
        filled[page, 0, :, j % page_size] = k.to(torch.bfloat16)
        filled[page, 1, :, j % page_size] = v.to(torch.bfloat16)
    q = (direction * 24).to(torch.bfloat16).repeat(R, H).contiguous()
    ctx = step_ctx(ctx_lens, [1] * R)
    kw = dict(num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5)
    want = torch.stack([values[r][far[r]].to(torch.bfloat16).float().repeat_interleave(H // KV, dim=0).reshape(H * D) for r in range(R)])
    for general in (False, True):
        monkeypatch.setattr(ops(), "_FORCE_GENERIC_ATTENTION", general)
        got = ops().paged_attention(q, filled, table, ctx, **kw).float()
        bad = (got - want).abs().amax(dim=1) > 2e-2 + 2e-2 * want.abs().amax(dim=1)
        assert not bad.any(), f"general={general}: requests {bad.nonzero().flatten().tolist()} with contexts {[ctx_lens[i] for i in bad.nonzero().flatten().tolist()]}"
    # and with ordinary inputs against the plain statement
    monkeypatch.setattr(ops(), "_FORCE_GENERIC_ATTENTION", False)
    q2 = rnd(R, H * D, dtype=torch.bfloat16, seed=77)
    pool2, table2, _, _ = _filled(ctx_lens, KV, D, page_size, seed=14)
    torch.testing.assert_close(ops().paged_attention(q2, pool2, table2, ctx, **kw).float(),
                               plain_ops.paged_attention(q2, pool2, table2, ctx, **kw).float(), **tol(torch.bfloat16))


@pytest.mark.parametrize("splits", [2, 5])
def test_paged_attention_64_row_shape_with_split_keys_and_merge(splits):
    """The library's C interface lets the 64-row shape split its keys over CTAs too, merged by a kernel of its own
    (the Python side never asks for it).  Called directly: portions of 40 and 9 tokens behind a thousand keys, beside a
    decode token of the split-key shape."""
    import ctypes

    o = ops()
    lib = o.library()
    H, KV, D, page_size = 8, 2, 64, 16
    ctx_lens, q_lens = [1100, 700, 900], [40, 9, 1]
    pool, table, _, _ = _filled(ctx_lens, KV, D, page_size, seed=41)
    ctx = step_ctx(ctx_lens, q_lens)
    n = sum(q_lens)
    q = rnd(n, H * D, dtype=torch.bfloat16, seed=42)
    out = torch.zeros((n, H * D), dtype=torch.bfloat16, device=DEV)
    scratch_o = torch.empty(n * H * splits * D, dtype=torch.float32, device=DEV)
    scratch_ml = torch.empty(n * H * splits * 2, dtype=torch.float32, device=DEV)
    counters = torch.zeros(len(q_lens) * KV, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), pool.data_ptr(), table.data_ptr(), table.shape[1],
            ctx.token_request.data_ptr(), ctx.cu_tokens.data_ptr(), ctx.context_lens.data_ptr(), len(q_lens), n, H, KV, D, page_size, 0,
            float(D**-0.5), max(q_lens) * (H // KV), 1, splits, splits, scratch_o.data_ptr(), scratch_ml.data_ptr(), counters.data_ptr()]
    assert lib.llm_attention_mma(*args, stream) == 0
    torch.cuda.synchronize()
    want = plain_ops.paged_attention(q, pool, table, ctx, num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5)
    torch.testing.assert_close(out.float(), want.float(), **tol(torch.bfloat16))
    assert int(counters.abs().sum()) == 0  # left zeroed for the next call
    # requests left to another kernel and split keys of the 64-row shape do not go together: refused, nothing launched
    assert lib.llm_attention_mma_routed(*args, 128, stream) == 10001


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 16, 17, 40])
def test_paged_attention_window_edge(dtype, window):
    """The key just outside the window shouts; the key just inside whispers.  The result must
    not contain the value of the key outside."""
    H, KV, D, page_size, n = 2, 1, 32, 8, 100
    pool, table, keys, values = make_cache([n], KV, D, page_size, dtype, seed=4)
    direction = torch.nn.functional.normalize(rnd(D, seed=6), dim=0)
    q = (direction * 20).repeat(H).reshape(1, H * D).to(dtype)
    keys[0][:] = keys[0] * 0.01
    keys[0][n - 1 - window] = direction * 20  # outside: position p - window
    values[0][n - 1 - window] = 1000.0
    fill_pool(pool, table, keys, values, page_size)
    ctx = step_ctx([n], [1])
    kw = dict(num_heads=H, num_kv_heads=KV, head_dim=D, scale=D**-0.5, window=window)
    got = ops().paged_attention(q, pool, table, ctx, **kw)
    want = plain_ops.paged_attention(q, pool, table, ctx, **kw)
    assert got.float().abs().max() < 100
    torch.testing.assert_close(got.float(), want.float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,D,page_size", [(4, 2, 16, 16), (3, 1, 32, 8), (5, 5, 80, 4), (32, 4, 64, 16)])
@pytest.mark.parametrize("rotate", [True, False])
def test_rope_kv_write(dtype, H, KV, D, page_size, rotate):
    n, theta, max_pos = 11, 500000.0, 300
    positions = torch.tensor([0, 1, 2, 7, 8, 9, 255, 299, 31, 32, 33], dtype=torch.int32, device=DEV)
    cos, sin = plain_llama.rope_cos_sin(torch.arange(max_pos), D, theta)
    table = torch.cat((cos[:, : D // 2], sin[:, : D // 2]), dim=-1).contiguous().to(DEV) if rotate else None
    qkv = rnd(n, (H + 2 * KV) * D, dtype=dtype, seed=11)
    pages = 8
    slot_map = torch.randperm(pages * page_size, generator=torch.Generator().manual_seed(2))[:n].to(torch.int32).to(DEV)
    pool_a = torch.zeros(pages, 2, KV, page_size, D, dtype=dtype, device=DEV)
    pool_b = pool_a.clone()
    qkv_a, qkv_b = qkv.clone(), qkv.clone()
    ops().rope_kv_write(qkv_a, positions, table, slot_map, pool_a, H, KV, D)
    plain_ops.rope_kv_write(qkv_b, positions, table, slot_map, pool_b, H, KV, D)
    torch.testing.assert_close(qkv_a.float(), qkv_b.float(), **tol(dtype))
    torch.testing.assert_close(pool_a.float(), pool_b.float(), **tol(dtype))
    if rotate:  # and against the reference's own formulation with concatenated halves
        q = qkv[:, : H * D].float().view(n, H, D).transpose(0, 1).cpu()
        c, s = cos[positions.cpu().long()], sin[positions.cpu().long()]
        want = plain_llama.apply_rope(q, c, s).transpose(0, 1).reshape(n, H * D)
        torch.testing.assert_close(qkv_a[:, : H * D].float().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,inter", [(3, 172), (17, 5632), (1, 16)])
def test_swiglu(dtype, n, inter):
    gate_up = rnd(n, 2 * inter, dtype=dtype, seed=12, std=3.0)
    torch.testing.assert_close(ops().swiglu(gate_up).float(), plain_ops.swiglu(gate_up).float(), **tol(dtype, 3.0))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,cols,pad", [(3, 172, 0), (17, 2560, 8), (1, 5, 3), (300, 100, 0)])
def test_add_bias(dtype, n, cols, pad):
    wide = rnd(n, cols + pad, dtype=dtype, seed=17)
    x = wide[:, :cols]  # rows wider than the columns that take the bias
    bias = rnd(cols, dtype=dtype, seed=18)
    want = (x.float() + bias.float()).to(dtype)
    before = wide.clone()
    got = ops().add_bias(x, bias)
    assert got.data_ptr() == x.data_ptr()
    torch.testing.assert_close(x.float(), want.float(), atol=0, rtol=0)
    torch.testing.assert_close(wide[:, cols:], before[:, cols:], atol=0, rtol=0)


@pytest.mark.parametrize("rows,vocab", [(1, 256), (5, 32000), (3, 50257), (2, 7)])
def test_argmax_lowest_index_among_equals(rows, vocab):
    logits = rnd(rows, vocab, seed=13)
    logits[0, vocab // 2] = 50.0
    logits[0, vocab - 1] = 50.0
    got = ops().argmax(logits)
    assert got.tolist() == torch.argmax(logits.cpu(), dim=-1).tolist()
    assert got[0].item() == vocab // 2


@pytest.mark.parametrize("vocab", [77, 384, 32000, 50257, 128256, 330001])  # the last does not fit in the shared memory of a cluster
def test_sample_matches_plain_sampler(vocab):
    rows = 12
    logits = rnd(rows, vocab, seed=14, std=2.0)
    temperature = torch.tensor([0.0, 0.8, 0.8, 1.0, 1.5, 0.3, 0.8, 0.8, 1.0, 1.0, 0.7, 2.0], device=DEV)
    top_k = torch.tensor([0, 0, 50, 1, 0, 0, 5, 0, 200, 0, 40, 0], dtype=torch.int32, device=DEV)
    top_p = torch.tensor([1.0, 1.0, 1.0, 1.0, 0.9, 1.0, 1.0, 0.5, 0.95, 1e-6, 0.8, 1.0], device=DEV)
    seeds = torch.arange(100, 100 + rows, dtype=torch.int64, device=DEV)
    for counter in (0, 1, 17):
        counters = torch.full((rows,), counter, dtype=torch.int64, device=DEV)
        got = ops().sample(logits, temperature, top_k, top_p, seeds, counters).tolist()
        want = plain_ops.sample(logits, temperature, top_k, top_p, seeds, counters).tolist()
        assert got == want
    assert got[0] == int(torch.argmax(logits[0]).item())  # temperature 0
    assert got[3] == int(torch.argmax(logits[3]).item())  # top_k = 1
    assert got[9] == int(torch.argmax(logits[9]).item())  # a tiny top_p keeps the top token only


def test_tokens_also_written_to_pinned_host_memory():
    rows, vocab = 6, 1000
    logits = rnd(rows, vocab, seed=16)
    host = torch.full((rows,), -1, dtype=torch.int32).pin_memory()
    got = ops().argmax(logits, host_out=host)
    torch.cuda.synchronize()
    assert host.tolist() == got.tolist() == torch.argmax(logits.cpu(), dim=-1).tolist()
    host.fill_(-1)
    t = torch.full((rows,), 0.7, device=DEV)
    k = torch.full((rows,), 20, dtype=torch.int32, device=DEV)
    p = torch.full((rows,), 0.9, device=DEV)
    seeds = torch.arange(rows, dtype=torch.int64, device=DEV)
    counters = torch.zeros(rows, dtype=torch.int64, device=DEV)
    got = ops().sample(logits, t, k, p, seeds, counters, host_out=host)
    torch.cuda.synchronize()
    assert host.tolist() == got.tolist() == plain_ops.sample(logits, t, k, p, seeds, counters).tolist()


@pytest.mark.parametrize("words,head", [(5, 0), (1092, 8), (70000, 64), (300, 300)])
def test_fetch_words_from_pinned_memory(words, head):
    host = torch.randint(-(2**31), 2**31 - 1, (words,), dtype=torch.int32).pin_memory()
    dev = torch.zeros(words, dtype=torch.int32, device=DEV)
    for round_ in range(2):  # the same addresses with new contents: nothing stale may be read
        host.copy_(torch.randint(-(2**31), 2**31 - 1, (words,), dtype=torch.int32))
        first = torch.arange(head, dtype=torch.int32, device=DEV) + 7 * round_
        ops().fetch_words(host, dev, first if head else None)
        torch.cuda.synchronize()
        want = host.clone()
        want[:head] = first.cpu()
        assert torch.equal(dev.cpu(), want)


def test_sample_follows_the_distribution():
    vocab, draws = 50, 4000
    logits = rnd(1, vocab, seed=15).repeat(draws, 1).contiguous()
    t = torch.full((draws,), 0.9, device=DEV)
    k = torch.full((draws,), 10, dtype=torch.int32, device=DEV)
    p = torch.full((draws,), 1.0, device=DEV)
    seeds = torch.full((draws,), 77, dtype=torch.int64, device=DEV)
    counters = torch.arange(draws, dtype=torch.int64, device=DEV)
    got = ops().sample(logits, t, k, p, seeds, counters).cpu().long()
    probs = plain_llama.filtered_probs(logits[0].cpu(), 0.9, top_k=10)
    freq = torch.bincount(got, minlength=vocab).double() / draws
    assert freq[probs == 0].sum() == 0  # nothing outside the top 10
    assert (freq - probs.double()).abs().max() < 0.03
