"""Each CUDA kernel alone against its plain statement, at sizes other than the
engine's tiny models: widths and vocabularies that are no power of two, head sizes
in steps of 16, odd head counts and groups, sharp attention data, page edges."""
import math

import pytest
import torch

from plain.plain_kernels import PlainKernels, philox_uniform

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def close(a, b, atol, rtol=0.0):
    a, b = a.double(), b.double()
    assert torch.isfinite(a).all() and torch.isfinite(b).all(), "non-finite values: the inputs are broken"
    err = (a - b).abs()
    bound = atol + rtol * b.abs()
    assert bool((err <= bound).all()), f"max err {float(err.max())}, at {int(err.argmax())}, bound {atol}+{rtol}*|b|"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,vocab", [(72, 301), (1000, 50), (3584, 777)])
def test_embed(cuda_kernels, dtype, hidden, vocab):
    table = rnd(vocab, hidden, dtype=dtype)
    ids = torch.randint(0, vocab, (37,), dtype=torch.int32, device=DEV)
    assert torch.equal(cuda_kernels.embed(table, ids, vocab), PlainKernels().embed(table, ids, vocab))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,hidden,eps", [(1, 64, 1e-6), (19, 200, 1e-5), (5, 3584, 1e-6), (3, 5000, 3e-4)])
def test_rmsnorm_and_fused_add(cuda_kernels, dtype, rows, hidden, eps):
    x = rnd(rows, hidden, seed=1, scale=0.05)
    w = 1.0 + rnd(hidden, seed=2, scale=0.3)
    want = PlainKernels(wide=True).rmsnorm(x, w, eps, torch.float64)
    got = cuda_kernels.rmsnorm(x, w, eps, dtype)
    close(got, want, atol=2e-6, rtol=2e-6 if dtype == torch.float32 else 2 ** -8)
    delta = rnd(rows, hidden, dtype=dtype, seed=3, scale=0.05)
    x1, x2 = x.clone(), x.clone()
    want = PlainKernels(wide=True).add_rmsnorm(x1, delta, w, eps, torch.float64)
    got = cuda_kernels.add_rmsnorm(x2, delta, w, eps, dtype)
    assert torch.equal(x1, x2), "the residual stream after the add differs"
    close(got, want, atol=2e-6, rtol=2e-6 if dtype == torch.float32 else 2 ** -8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,inter", [(3, 176), (17, 321), (2, 18944)])
def test_silu_mul(cuda_kernels, dtype, rows, inter):
    gu = rnd(rows, 2 * inter, dtype=dtype, seed=4, scale=2.0)
    want = PlainKernels(wide=True).silu_mul(gu.double())
    close(cuda_kernels.silu_mul(gu), want, atol=1e-6, rtol=1e-6 if dtype == torch.float32 else 2 ** -8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_add_gather_scatter(cuda_kernels, dtype):
    x = rnd(13, 100, seed=5)
    delta = rnd(13, 100, dtype=dtype, seed=6)
    want = x + delta.float()
    cuda_kernels.residual_add(x, delta)
    assert torch.equal(x, want)
    rows = torch.tensor([12, 0, 5, 5], dtype=torch.int32, device=DEV)
    assert torch.equal(cuda_kernels.gather_rows(x, rows), x[rows.long()])
    table = torch.zeros((4, 10), dtype=torch.int32, device=DEV)
    idx = torch.tensor([3, 17, 39], dtype=torch.int32, device=DEV)
    val = torch.tensor([7, 8, 9], dtype=torch.int32, device=DEV)
    cuda_kernels.scatter_i32(table, idx, val)
    assert table.view(-1)[idx.long()].tolist() == [7, 8, 9] and int(table.sum()) == 24


@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (7, 130, 50), (65, 257, 333), (130, 1000, 192), (3, 48, 17)])
def test_gemm_float32(cuda_kernels, M, N, K):
    a, w, b = rnd(M, K, seed=7), rnd(N, K, seed=8), rnd(N, seed=9)
    want = a.double() @ w.double().t() + b.double()
    close(cuda_kernels.linear(a, w, b), want, atol=1e-5 * math.sqrt(K), rtol=1e-6)
    # a row's result does not depend on what else is in the launch
    alone = cuda_kernels.linear(a[M // 2:M // 2 + 1].contiguous(), w, b)
    assert torch.equal(alone[0], cuda_kernels.linear(a, w, b)[M // 2])


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (7, 136, 48), (65, 264, 328), (8, 1000, 192), (3, 50, 17)])
def test_gemm_bfloat16(cuda_kernels, M, N, K, out_dtype):
    a, w = rnd(M, K, dtype=torch.bfloat16, seed=7), rnd(N, K, dtype=torch.bfloat16, seed=8)
    want = a.double() @ w.double().t()
    rtol = 2 ** -8 if out_dtype == torch.bfloat16 else 1e-5
    close(cuda_kernels.linear(a, w, out_dtype=out_dtype), want, atol=1e-4 * math.sqrt(K), rtol=rtol)
    close(cuda_kernels.linear_generic(a, w, out_dtype=out_dtype), want, atol=1e-4 * math.sqrt(K), rtol=rtol)


@pytest.mark.parametrize("M,N,K", [(1, 128, 64), (3, 80, 128), (8, 256, 512), (17, 1000, 200), (33, 300, 328), (64, 3584, 1024),
                                   (100, 130, 72), (128, 520, 4104), (5, 4608, 3584), (129, 264, 520), (200, 1000, 328),
                                   (256, 384, 4104)])
def test_gemm_tcgen05_few_rows(cuda_kernels, monkeypatch, M, N, K):
    """The weight-streaming tensor-core product: plain store (bfloat16 and float32 out, with
    bias), K split into partial sums and their consumers, and the fused silu(gate) * up."""
    monkeypatch.setattr(type(cuda_kernels), "SKINNY_MAX_ROWS", 256)    # the kernel's own limit, not the routing's
    from inferflux_b200.csrc import PartialSum
    a = rnd(M, K, dtype=torch.bfloat16, seed=20, scale=0.5)
    w = rnd(N, K, dtype=torch.bfloat16, seed=21, scale=0.1)
    b = rnd(N, seed=22)
    want = a.double() @ w.double().t()
    tol = 1e-4 * math.sqrt(K)
    close(cuda_kernels.linear_skinny(a, w, None, out_dtype=torch.bfloat16), want, atol=tol, rtol=2 ** -8)
    close(cuda_kernels.linear_skinny(a, w, b, out_dtype=torch.float32), want + b.double(), atol=tol, rtol=1e-5)
    kblocks = -(-K // 64)
    for splits in sorted({1, min(3, kblocks), min(10, kblocks)}):
        parts = cuda_kernels.linear_skinny(a, w, None, splits=splits, mode=1)
        assert parts.shape == (splits, M, N)
        close(parts.double().sum(0), want, atol=tol, rtol=1e-5)
        ps = PartialSum(parts, torch.bfloat16)
        close(cuda_kernels.materialize(ps, b), want + b.double(), atol=tol, rtol=2 ** -8)
        x = rnd(M, N, seed=23)
        x1, x2 = x.clone(), x.clone()
        cuda_kernels.residual_add(x1, ps)
        close(x1, x.double() + want, atol=tol, rtol=1e-5)
        wn = 1 + rnd(N, seed=24, scale=0.1)
        got = cuda_kernels.add_rmsnorm(x2, ps, wn, 1e-5, torch.bfloat16)
        ref = PlainKernels(wide=True).rmsnorm(x.double() + want, wn, 1e-5, torch.float64)
        assert torch.equal(x1, x2)
        close(got, ref, atol=1e-3, rtol=2 ** -7)
    if N % 2 == 0:
        half = N // 2
        g, u = want[:, :half], want[:, half:]
        got = cuda_kernels.linear_skinny(a, w, None, mode=2, n_out=half, up_row_offset=half)
        close(got, g / (1 + torch.exp(-g)) * u, atol=tol, rtol=2 ** -7)
        close(cuda_kernels.linear_swiglu(a, w), g / (1 + torch.exp(-g)) * u, atol=tol, rtol=2 ** -7)
    # the routing in `linear`: few rows go to this kernel, with or without partial sums
    r = cuda_kernels.linear(a, w, allow_partial=True)
    close(cuda_kernels.materialize(r), want, atol=tol, rtol=2 ** -8)
    cuda_kernels.check_errors()


@pytest.mark.parametrize("T,H,N", [(1, 64, 128), (8, 3584, 512), (33, 1000, 264), (128, 520, 130), (250, 520, 264)])
def test_prenormed_rows_through_the_product(cuda_kernels, monkeypatch, T, H, N):
    """The norm that leaves its row scale to the product: prenorm + linear equals
    add_rmsnorm + linear, for every epilogue of the few-rows product."""
    monkeypatch.setattr(type(cuda_kernels), "SKINNY_MAX_ROWS", 256)    # the kernel's own limit, not the routing's
    from inferflux_b200.csrc import PartialSum, ScaledRows
    x = rnd(T, H, seed=30)
    parts = PartialSum(rnd(3, T, H, seed=31, scale=0.3), torch.bfloat16)
    wn = 1 + rnd(H, seed=32, scale=0.2)
    w = rnd(N, H, dtype=torch.bfloat16, seed=33, scale=0.1)
    b = rnd(N, seed=34)
    x1, x2 = x.clone(), x.clone()
    rows = cuda_kernels.prenorm(x1, parts, wn, 1e-5, torch.bfloat16)
    assert isinstance(rows, ScaledRows)
    xs = x.double() + parts.parts.double().sum(0)
    hn = PlainKernels(wide=True).rmsnorm(xs, wn, 1e-5, torch.float64)
    close(x1, xs, atol=1e-5, rtol=1e-6)
    close(cuda_kernels.materialize_rows(rows), hn, atol=2e-3, rtol=2 ** -7)
    # the product works on the rounded rows x * w; its result is exact up to float32 accumulation
    scale = torch.rsqrt((xs * xs).mean(-1, keepdim=True) + 1e-5)
    want = (rows.pre.double() * scale) @ w.double().t()
    close(want, hn @ w.double().t(), atol=2e-3 * math.sqrt(H), rtol=2e-2)
    tol = 1e-4 * math.sqrt(H)
    close(cuda_kernels.linear(rows, w, b, out_dtype=torch.float32), want + b.double(), atol=tol, rtol=1e-5)
    close(cuda_kernels.materialize(cuda_kernels.linear(rows, w, allow_partial=True)), want, atol=tol, rtol=2 ** -8)
    if N % 2 == 0:
        g, u = want[:, :N // 2], want[:, N // 2:]
        close(cuda_kernels.linear_swiglu(rows, w), g / (1 + torch.exp(-g)) * u, atol=tol, rtol=2 ** -7)
    # a plain tensor delta and no delta at all
    d16 = rnd(T, H, dtype=torch.bfloat16, seed=35)
    r2 = cuda_kernels.prenorm(x2, d16, wn, 1e-5, torch.bfloat16)
    close(cuda_kernels.materialize_rows(r2), PlainKernels(wide=True).rmsnorm(x.double() + d16.double(), wn, 1e-5, torch.float64),
          atol=2e-3, rtol=2 ** -7)
    r3 = cuda_kernels.prenorm(x2, None, wn, 1e-5, torch.bfloat16)
    close(cuda_kernels.materialize_rows(r3), PlainKernels(wide=True).rmsnorm(x2.double(), wn, 1e-5, torch.float64),
          atol=2e-3, rtol=2 ** -7)
    cuda_kernels.check_errors()


def test_rope_append_from_partial_sums(cuda_kernels):
    from inferflux_b200.csrc import PartialSum
    from inferflux_b200.parts.base import RotaryTable
    nq, nkv, d, page = 6, 2, 32, 8
    lens, spans = [40, 9], [7, 1]
    ctx, cache, slots = make_cache_case(torch.bfloat16, nkv, d, page, lens, spans, num_pages=12, seed=1)
    T, width = ctx.num_tokens, (nq + 2 * nkv) * d
    parts = rnd(3, T, width, seed=2)
    bias = rnd(width, seed=3)
    inv = (1.0 / (1e4 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    rotary = RotaryTable(inv, d, False)
    kv0 = cache.kv.clone()
    q1 = cuda_kernels.rope_append(PartialSum(parts, torch.bfloat16), bias, rotary, nq, nkv, d, ctx, cache)
    kv1 = cache.kv.clone()
    cache.kv = kv0
    q2 = PlainKernels(wide=True).rope_append(parts.sum(0).double(), bias, rotary, nq, nkv, d, ctx, cache)
    close(q1, q2, atol=2e-2, rtol=2 ** -7)
    close(kv1, cache.kv, atol=2e-2, rtol=2 ** -7)


# ---------------------------------------------------------------------- attention

class _Ctx:
    pass


def make_cache_case(dtype, nkv, d, page, lens, spans, num_pages, seed, shuffle=True):
    """A cache filled by hand: `lens[r]` tokens stored for request r, of which the
    last `spans[r]` are this step's queries.  Pages are handed out in a shuffled
    order so that logical and physical order differ."""
    from inferflux_b200.cache.manager import CacheView
    g = torch.Generator().manual_seed(seed)
    R = len(lens)
    max_blocks = max(-(-n // page) for n in lens) + 1
    order = torch.randperm(num_pages, generator=g).tolist() if shuffle else list(range(num_pages))
    table = torch.full((R + 2, max_blocks), -1, dtype=torch.int32)
    slots = list(range(R, 0, -1))                       # slots differ from batch order
    for r, n in enumerate(lens):
        for b in range(-(-n // page)):
            table[slots[r], b] = order.pop()
    kv = torch.zeros((num_pages, 2, nkv, page, d), dtype=dtype)
    ctx = _Ctx()
    positions, token_req = [], []
    for r, (n, s) in enumerate(zip(lens, spans)):
        positions += list(range(n - s, n))
        token_req += [r] * s
    ctx.positions = torch.tensor(positions, dtype=torch.int32, device=DEV)
    ctx.token_req = torch.tensor(token_req, dtype=torch.int32, device=DEV)
    ctx.req_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    ctx.num_tokens = len(positions)
    # the work lists of the attention kernels, as the kernel table makes them for a step
    ctx.spans = [(n - s_, s_) for n, s_ in zip(lens, spans)]
    ctx.slots_host = slots
    from inferflux_b200.csrc import CudaKernels
    ctx.extra, ctx.extra_len = {}, {}
    for name, vals in CudaKernels.attention_sections(CudaKernels, ctx).items():
        ctx.extra[name] = torch.tensor(vals, dtype=torch.int32, device=DEV)
        ctx.extra_len[name] = len(vals)
    ctx.max_kv_len = max(lens)
    cache = CacheView(kv.to(DEV), table.to(DEV), page, None, True, 0)
    return ctx, cache, slots


def fill_cache(cache, lens, slots, nkv, d, dtype, seed, sharp_every=0):
    """Random keys and values for every stored position; returns them per request."""
    g = torch.Generator().manual_seed(seed)
    page = cache.page_size
    stored = []
    for r, n in enumerate(lens):
        K = torch.randn(n, nkv, d, generator=g).to(dtype)
        V = torch.randn(n, nkv, d, generator=g).to(dtype)
        stored.append((K, V))
        for p in range(n):
            pg = int(cache.block_table[slots[r], p // page])
            cache.kv[pg, 0, :, p % page, :] = K[p].to(DEV)
            cache.kv[pg, 1, :, p % page, :] = V[p].to(DEV)
    return stored


def attention_oracle(q, stored, lens, spans, nq, nkv, d, window, scale):
    out = []
    t = 0
    for r, (n, s) in enumerate(zip(lens, spans)):
        K, V = stored[r][0].double(), stored[r][1].double()
        for pos in range(n - s, n):
            first = max(0, pos - window + 1) if window else 0
            for h in range(nq):
                g = h // (nq // nkv)
                sc = (K[first:pos + 1, g] @ q[t, h].double().cpu()) * scale
                out.append(torch.softmax(sc, 0) @ V[first:pos + 1, g])
            t += 1
    return torch.stack(out).view(-1, nq * d)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (4, 2, 16, 4, None), (6, 2, 32, 8, None), (7, 1, 128, 16, None), (5, 5, 48, 16, 21),
    (28, 4, 128, 16, None), (12, 2, 64, 32, 100), (3, 1, 80, 8, 7), (2, 1, 256, 16, None),
    (34, 2, 32, 16, None), (4, 2, 144, 16, None), (8, 1, 96, 5, 33), (6, 3, 112, 64, None)])
def test_attention_over_pages(cuda_kernels, dtype, nq, nkv, d, page, window):
    """Mixed spans (prompt portions beside single tokens) over shuffled pages, with
    sharp data: one far key per query dominates, so a key that is missed, read from
    the wrong page or masked wrongly changes the result."""
    lens = [1, 37, 130, 64, 259, 16, 1500, 200]
    spans = [1, 1, 50, 64, 3, 2, 1, 150]
    ctx, cache, slots = make_cache_case(dtype, nkv, d, page, lens, spans, num_pages=sum(-(-n // page) for n in lens) + 3,
                                        seed=3)
    stored = fill_cache(cache, lens, slots, nkv, d, dtype, seed=4)
    T = ctx.num_tokens
    q = rnd(T, nq, d, dtype=dtype, seed=5, scale=0.3)
    # plant: query t of head h looks hard at one key inside its range (often the first or last it may see)
    t = 0
    for r, (n, s) in enumerate(zip(lens, spans)):
        for pos in range(n - s, n):
            first = max(0, pos - window + 1) if window else 0
            target = [first, pos, (first + pos) // 2][t % 3]
            for h in range(nq):
                g = h // (nq // nkv)
                q[t, h] = (stored[r][0][target, g].float() * (12.0 / math.sqrt(d))).to(dtype).to(DEV)
            t += 1
    scale = 1.0 / math.sqrt(d)
    want = attention_oracle(q, stored, lens, spans, nq, nkv, d, window, scale)
    got = cuda_kernels.attention(q.view(T, nq * d), nq, nkv, d, window, scale, ctx, cache)
    close(got.cpu(), want, atol=2e-5 if dtype == torch.float32 else 2e-2, rtol=1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("nq,nkv,d,page,window", [(14, 2, 128, 16, None), (4, 1, 64, 32, None), (8, 2, 128, 16, 2300)])
def test_attention_decode_one_token_over_a_cluster_of_sixteen(cuda_kernels, nq, nkv, d, page, window):
    """One or two decoded tokens with thousands of keys: the key range is cut over the largest
    cluster the kernel takes, and the planted key may lie in any block of it."""
    dtype = torch.bfloat16
    lens, spans = [2600, 2333], [1, 1]
    assert cuda_kernels.decode_splits(2, nkv, 2333, cuda_kernels.lib.ifx_attention_decode_max_splits(d, page)) == 16
    for target_of in (lambda first, pos: first, lambda first, pos: pos, lambda first, pos: first + (pos - first) * 5 // 16,
                      lambda first, pos: first + (pos - first) * 15 // 16):
        ctx, cache, slots = make_cache_case(dtype, nkv, d, page, lens, spans,
                                            num_pages=sum(-(-n // page) for n in lens) + 3, seed=23)
        stored = fill_cache(cache, lens, slots, nkv, d, dtype, seed=24)
        q = rnd(2, nq, d, dtype=dtype, seed=25, scale=0.3)
        for t, n in enumerate(lens):
            pos = n - 1
            first = max(0, pos - window + 1) if window else 0
            for h in range(nq):
                g = h // (nq // nkv)
                q[t, h] = (stored[t][0][target_of(first, pos), g].float() * (12.0 / math.sqrt(d))).to(dtype).to(DEV)
        scale = 1.0 / math.sqrt(d)
        want = attention_oracle(q, stored, lens, spans, nq, nkv, d, window, scale)
        got = cuda_kernels.attention(q.view(2, nq * d), nq, nkv, d, window, scale, ctx, cache)
        close(got.cpu(), want, atol=2e-2, rtol=2e-2)
    cuda_kernels.check_errors()


@pytest.mark.parametrize("nq,nkv,d,page,window", [(14, 2, 128, 16, None), (6, 1, 64, 32, None), (7, 1, 128, 16, 12500)])
def test_attention_decode_one_token_over_thirteen_thousand_keys(cuda_kernels, nq, nkv, d, page, window):
    """One decoded token far into a long context: few blocks, each with hundreds of keys a warp, which is where
    the decode kernel runs with rings twice as deep.  The planted key may lie anywhere in the range."""
    dtype = torch.bfloat16
    lens, spans = [13000], [1]
    ctx, cache, slots = make_cache_case(dtype, nkv, d, page, lens, spans, num_pages=-(-lens[0] // page) + 3, seed=33)
    stored = fill_cache(cache, lens, slots, nkv, d, dtype, seed=34)
    scale = 1.0 / math.sqrt(d)
    pos = lens[0] - 1
    first = max(0, pos - window + 1) if window else 0
    for target in (first, pos, first + 17, first + (pos - first) // 3, pos - 1, first + (pos - first) * 11 // 16):
        q = rnd(1, nq, d, dtype=dtype, seed=35, scale=0.3)
        for h in range(nq):
            q[0, h] = (stored[0][0][target, h // (nq // nkv)].float() * (12.0 / math.sqrt(d))).to(dtype).to(DEV)
        want = attention_oracle(q, stored, lens, spans, nq, nkv, d, window, scale)
        got = cuda_kernels.attention(q.view(1, nq * d), nq, nkv, d, window, scale, ctx, cache)
        close(got.cpu(), want, atol=2e-2, rtol=2e-2)
    cuda_kernels.check_errors()


@pytest.mark.parametrize("nq,nkv,d,page,window", [
    (4, 2, 128, 16, None), (6, 1, 64, 16, None), (4, 4, 128, 32, 200), (3, 1, 64, 64, 129), (2, 1, 96, 16, 300)])
def test_attention_long_portions(cuda_kernels, monkeypatch, nq, nkv, d, page, window):
    """Portions of several hundred tokens behind several hundred cached ones: many key tiles
    for each tile of queries, whole ones and ragged ones, and a window that ends inside them."""
    dtype = torch.bfloat16
    lens = [700, 513, 1, 390]
    spans = [300, 513, 1, 131]
    ctx, cache, slots = make_cache_case(dtype, nkv, d, page, lens, spans, num_pages=sum(-(-n // page) for n in lens) + 5,
                                        seed=13)
    stored = fill_cache(cache, lens, slots, nkv, d, dtype, seed=14)
    T = ctx.num_tokens
    q = rnd(T, nq, d, dtype=dtype, seed=15, scale=0.3)
    t = 0
    for r, (n, s) in enumerate(zip(lens, spans)):
        for pos in range(n - s, n):
            first = max(0, pos - window + 1) if window else 0
            target = [first, pos, (first + pos) // 2, max(first, pos - 127), max(first, pos - 128)][t % 5]
            for h in range(nq):
                g = h // (nq // nkv)
                q[t, h] = (stored[r][0][target, g].float() * (12.0 / math.sqrt(d))).to(dtype).to(DEV)
            t += 1
    scale = 1.0 / math.sqrt(d)
    want = attention_oracle(q, stored, lens, spans, nq, nkv, d, window, scale)
    got = cuda_kernels.attention(q.view(T, nq * d), nq, nkv, d, window, scale, ctx, cache)
    close(got.cpu(), want, atol=2e-2, rtol=2e-2)
    # the mma.sync kernel that takes the other head sizes gives the same on these
    monkeypatch.setattr(cuda_kernels, "tensor_core_prefill", False)
    other = cuda_kernels.attention(q.view(T, nq * d), nq, nkv, d, window, scale, ctx, cache)
    close(other.cpu(), want, atol=2e-2, rtol=2e-2)
    cuda_kernels.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("many", [False, True])
@pytest.mark.parametrize("nq,nkv,d,rot,interleaved,bias", [
    (4, 2, 16, 16, False, True), (6, 2, 32, 32, False, False), (5, 1, 48, 24, True, True),
    (28, 4, 128, 128, False, True), (3, 3, 80, 0, False, True), (2, 1, 256, 256, False, True)])
def test_rope_append(cuda_kernels, dtype, nq, nkv, d, rot, interleaved, bias, many):
    from inferflux_b200.parts.base import RotaryTable
    page = 8
    lens, spans = [5, 300, 41, 17], [5, 1, 30, 2]
    if many:
        lens, spans = [70, 300, 41, 17], [70, 100, 30, 2]        # enough tokens for the one-block-per-token kernel
    ctx, cache, slots = make_cache_case(dtype, nkv, d, page, lens, spans, num_pages=60, seed=6)
    ref_cache_kv = cache.kv.clone()
    T = ctx.num_tokens
    qkv = rnd(T, (nq + 2 * nkv) * d, dtype=dtype, seed=7)
    b = rnd((nq + 2 * nkv) * d, seed=8, scale=0.5) if bias else None
    rotary = None
    if rot:
        inv = (1.0 / (1e6 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(DEV)
        rotary = RotaryTable(inv, rot, interleaved)
    q_got = cuda_kernels.rope_append(qkv, b, rotary, nq, nkv, d, ctx, cache)
    got_kv = cache.kv.clone()
    cache.kv = ref_cache_kv
    q_want = PlainKernels(wide=True).rope_append(qkv, b, rotary, nq, nkv, d, ctx, cache)
    tol = dict(atol=3e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=1e-2, rtol=2 ** -7)
    close(q_got, q_want, **tol)
    close(got_kv, cache.kv, **tol)
    assert int((got_kv != 0).any(-1).sum()) == int((cache.kv != 0).any(-1).sum()), "rows written differ"


# ----------------------------------------------------------------------- sampling

@pytest.mark.parametrize("rows,vocab", [(1, 512), (5, 1000), (64, 152064), (3, 777)])
def test_argmax_first_index_wins(cuda_kernels, rows, vocab):
    logits = rnd(rows, vocab, seed=10)
    logits[0, vocab // 3] = 50.0
    logits[0, vocab - 1] = 50.0                      # a tie: the lower index is the answer
    got = cuda_kernels.argmax(logits)
    assert got.tolist() == torch.argmax(logits, -1).tolist()
    assert int(got[0]) == vocab // 3


def test_sampling_matches_plain(cuda_kernels):
    from plain.plain_kernels import PlainKernels
    rows, vocab = 12, 3001
    logits = rnd(rows, vocab, seed=11, scale=3.0)
    f = lambda v: torch.tensor(v, dtype=torch.float32, device=DEV)
    i = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    temperature = f([0.8, 1.0, 0.0, 1.3, 0.5, 1.0, 1.0, 0.7, 1.0, 2.0, 1.0, 0.9])
    top_k = i([0, 40, 0, 0, 5, 0, 1, 0, 100, 0, 0, 3])
    top_p = f([1.0, 1.0, 1.0, 0.9, 1.0, 0.5, 1.0, 0.95, 0.8, 1.0, 0.1, 1.0])
    min_p = f([0, 0, 0, 0, 0, 0, 0, 0.05, 0, 0.2, 0, 0])
    seed_lo = torch.arange(rows, dtype=torch.int64).add(12345).to(torch.int32).to(DEV)
    seed_hi = torch.zeros(rows, dtype=torch.int32, device=DEV)
    agree = 0
    for step in range(6):
        st = torch.full((rows,), step, dtype=torch.int32, device=DEV)
        got = cuda_kernels.sample(logits, temperature, top_k, top_p, min_p, seed_lo, seed_hi, st).tolist()
        want = PlainKernels().sample(logits.cpu(), temperature.cpu(), top_k.cpu(), top_p.cpu(), min_p.cpu(),
                                     seed_lo.cpu(), seed_hi.cpu(), st.cpu()).tolist()
        agree += sum(int(a == b) for a, b in zip(got, want))
        assert got[2] == int(torch.argmax(logits[2])) and got[6] == int(torch.argmax(logits[6]))
        # whatever is drawn must lie inside the kept set
        from plain.plain_kernels import kept_mask
        for r in range(rows):
            if float(temperature[r]) > 0:
                p = torch.softmax(logits[r].cpu() / float(temperature[r]), -1)
                keep = kept_mask(p, int(top_k[r]), float(top_p[r]), float(min_p[r]))
                assert bool(keep[got[r]]) or float(p[got[r]]) >= 0.999 * float(p[keep].min())
    assert agree >= 6 * rows - 2, f"only {agree} of {6 * rows} draws agree with the plain sampler"


@pytest.mark.parametrize("vocab", [700, 9001, 152064])
def test_sampling_over_many_blocks_against_one_block(cuda_kernels, vocab):
    """The many-block sampler (radix descent on counts and fixed-point masses) draws what the
    one-block sampler (bisection on float sums) draws, up to elements that sit on a threshold;
    whatever it draws lies in the kept set; twice in a row (its scratch must be left zero)."""
    from plain.plain_kernels import kept_mask
    rows = 24
    logits = rnd(rows, vocab, seed=51, scale=2.5)
    logits[3, 17] = logits[3, 400]                       # ties at a threshold
    g = torch.Generator().manual_seed(5)
    temperature = (torch.rand(rows, generator=g) * 1.5 + 0.3)
    temperature[5] = 0.0
    top_k = torch.tensor([0, 1, 5, 50, 0, 0, 0, 1000, 3, 0, 0, 20] * 2, dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 1.0, 0.9, 0.5, 0.3, 0.95, 0.8, 1.0, 0.05, 0.999, 0.7] * 2)
    min_p = torch.tensor([0, 0, 0, 0, 0, 0, 0.05, 0, 0.3, 0, 0, 0.01] * 2, dtype=torch.float32)
    seed_lo = torch.arange(rows, dtype=torch.int32) + 77
    z = torch.zeros(rows, dtype=torch.int32)
    dev = lambda t: t.to(DEV)
    from plain.plain_kernels import philox_uniform

    def near_a_boundary(r, step, a, b):
        """Two samplers may differ on a row only where float32 rounding decides: the draw falls within 2e-5 of
        the total mass of a boundary between two kept tokens, or a token sits on a threshold."""
        pr = torch.softmax(logits[r].cpu().double() / float(temperature[r]), -1)
        keep = kept_mask(pr.float(), int(top_k[r]), float(top_p[r]), float(min_p[r]))
        if not (bool(keep[a]) and bool(keep[b])):
            edge = float(pr[keep].min())
            return min(abs(float(pr[a]) - edge), abs(float(pr[b]) - edge)) <= 1e-3 * edge
        c = torch.cumsum(torch.where(keep, pr, torch.zeros_like(pr)), 0)
        target = philox_uniform(int(seed_lo[r]), 0, step) * float(c[-1])
        lo, hi = min(a, b), max(a, b)
        return float((c[lo:hi] - target).abs().min()) <= 2e-5 * float(c[-1])

    plain = PlainKernels(wide=True)
    for step in range(8):
        st = torch.full((rows,), step, dtype=torch.int32)
        args = [dev(temperature), dev(top_k), dev(top_p), dev(min_p), dev(seed_lo), dev(z), dev(st)]
        got = cuda_kernels.sample(logits, *args).tolist()
        again = cuda_kernels.sample(logits, *args).tolist()
        assert got == again, "the same call drew differently the second time"
        few = cuda_kernels.sample(logits[:5].contiguous(), *[a[:5].contiguous() for a in args]).tolist()
        assert few == got[:5], "a row drew differently in a smaller batch"
        one = cuda_kernels.sample_one_block(logits, *args).tolist()
        want = plain.sample(logits.cpu(), temperature, top_k, top_p, min_p, seed_lo, z, st).tolist()
        for r in range(rows):                                 # against the one-block kernel and the plain statement
            for other, name in ((one[r], "one-block kernel"), (want[r], "plain sampler")):
                assert got[r] == other or (float(temperature[r]) > 0 and near_a_boundary(r, step, got[r], other)), \
                    f"step {step} row {r}: drew {got[r]}, the {name} {other}"
        assert got[5] == int(torch.argmax(logits[5]))
        for r in range(rows):
            if float(temperature[r]) > 0:
                p = torch.softmax(logits[r].cpu() / float(temperature[r]), -1)
                keep = kept_mask(p, int(top_k[r]), float(top_p[r]), float(min_p[r]))
                assert bool(keep[got[r]]) or float(p[got[r]]) >= 0.999 * float(p[keep].min()), (r, got[r])
    # filters the caller says nobody uses are not applied: the plain temperature draw
    plain = cuda_kernels.sample(logits, dev(temperature), dev(top_k), dev(top_p), dev(min_p * 0), dev(seed_lo), dev(z), dev(z),
                                features=0).tolist()
    want = cuda_kernels.sample_one_block(logits, dev(temperature), dev(top_k * 0), dev(top_p * 0 + 1), dev(min_p * 0),
                                         dev(seed_lo), dev(z), dev(z)).tolist()
    assert sum(int(a == b) for a, b in zip(plain, want)) >= rows - 1


def test_sampling_distribution_and_batch_independence(cuda_kernels):
    vocab = 50
    logits = torch.log(torch.arange(1, vocab + 1, dtype=torch.float32)).repeat(4096, 1).to(DEV)
    n = logits.shape[0]
    f = lambda v: torch.full((n,), v, dtype=torch.float32, device=DEV)
    z = torch.zeros(n, dtype=torch.int32, device=DEV)
    seeds = torch.arange(n, dtype=torch.int32, device=DEV)
    got = cuda_kernels.sample(logits, f(1.0), z, f(1.0), f(0.0), seeds, z, z)
    freq = torch.bincount(got.long(), minlength=vocab).float() / n
    want = torch.arange(1, vocab + 1, dtype=torch.float32) / (vocab * (vocab + 1) / 2)
    assert float((freq.cpu() - want).abs().max()) < 0.015
    # the same request (seed, step) draws the same token alone as in a batch
    alone = cuda_kernels.sample(logits[7:8].contiguous(), f(1.0)[:1], z[:1], f(1.0)[:1], f(0.0)[:1],
                                seeds[7:8].contiguous(), z[:1], z[:1])
    assert int(alone[0]) == int(got[7])
    assert abs(philox_uniform(7, 0, 0) - 0.5) <= 0.5


def test_penalties_and_bias(cuda_kernels):
    logits = rnd(2, 100, seed=12)
    want = logits.clone().cpu()
    tokens = torch.tensor([[5, 9, -1], [7, -1, -1]], dtype=torch.int32)
    counts = torch.tensor([[2, 1, 0], [3, 0, 0]], dtype=torch.int32)
    rep, freq, pres = torch.tensor([1.3, 1.0]), torch.tensor([0.1, 0.5]), torch.tensor([0.2, 0.0])
    PlainKernels().penalties(want, tokens, counts, rep, freq, pres)
    cuda_kernels.penalties(logits, tokens.to(DEV), counts.to(DEV), rep.to(DEV), freq.to(DEV), pres.to(DEV))
    close(logits.cpu(), want, atol=1e-6)
    rows = torch.tensor([0, 1, 1], dtype=torch.int32, device=DEV)
    toks = torch.tensor([3, 3, 99], dtype=torch.int32, device=DEV)
    bias = torch.tensor([1.5, -2.0, 100.0], device=DEV)
    cuda_kernels.logit_bias(logits, rows, toks, bias)
    want[0, 3] += 1.5; want[1, 3] -= 2.0; want[1, 99] += 100.0
    close(logits.cpu(), want, atol=1e-6)


@pytest.mark.parametrize("M,N,K", [(1, 256, 64), (130, 520, 264), (257, 1000, 1536), (512, 4608, 3584), (300, 256, 8960)])
def test_many_rows_tensor_core_product_and_its_swiglu(cuda_kernels, M, N, K):
    """The tcgen05 product for prompt portions (128 x 256 tiles, persistent blocks, two accumulators in
    tensor memory): plain store, and silu(gate) * up from stacked weights, at sizes with ragged edges."""
    a = rnd(M, K, dtype=torch.bfloat16, seed=40, scale=0.5)
    w = rnd(N, K, dtype=torch.bfloat16, seed=41, scale=0.1)
    want = a.double() @ w.double().t()
    tol = 1e-4 * math.sqrt(K)
    close(cuda_kernels.linear_tiles(a, w), want, atol=tol, rtol=2 ** -8)
    if N % 2 == 0:
        half = N // 2
        g, u = want[:, :half], want[:, half:]
        close(cuda_kernels.linear_tiles(a, w, swiglu=True), g / (1 + torch.exp(-g)) * u, atol=tol, rtol=2 ** -7)
    cuda_kernels.check_errors()
