"""Each CUDA kernel alone against a plain PyTorch reference, at sizes other than the engine's."""

import math

import numpy as np
import pytest
import torch

from tests.plain import llama

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=2e-2, atol=2e-2)


def dev(t):
    return t.cuda()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, width, vocab", [(1, 8, 3), (17, 100, 331), (129, 2048, 1000), (5, 7, 11)])
def test_embedding_and_gather(dtype, rows, width, vocab):
    from tesseract_b200 import kernels

    torch.manual_seed(0)
    table = torch.randn(vocab, width).to(dtype)
    tokens = torch.randint(0, vocab, (rows,), dtype=torch.int32)
    out = torch.empty(rows, width, dtype=dtype, device="cuda")
    kernels.embedding(dev(tokens), dev(table), out)
    assert torch.equal(out.cpu(), table[tokens.long()])
    picked = torch.empty(rows, width, dtype=dtype, device="cuda")
    index = torch.randint(0, rows, (rows,), dtype=torch.int32)
    kernels.gather_rows(dev(index), out, picked)
    assert torch.equal(picked.cpu(), table[tokens.long()][index.long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, width, eps", [(1, 16, 1e-5), (3, 100, 1e-6), (64, 2048, 1e-5), (7, 4100, 1e-3)])
def test_rms_norm_and_fused_add(dtype, rows, width, eps):
    from tesseract_b200 import kernels

    torch.manual_seed(1)
    x = (torch.randn(rows, width) * 3).to(dtype)
    u = torch.randn(rows, width).to(dtype)
    w = 1 + 0.1 * torch.randn(width)
    out = torch.empty(rows, width, dtype=dtype, device="cuda")
    kernels.rms_norm(dev(x), dev(w), eps, out)
    want = llama.rms_norm(x.double(), w.double(), eps)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype))
    res = dev(x.clone())
    kernels.add_rms_norm(res, dev(u), dev(w), eps, out, res)
    c = x.double() + u.double()
    torch.testing.assert_close(out.cpu().double(), llama.rms_norm(c, w.double(), eps), **tol(dtype))
    torch.testing.assert_close(res.cpu().double(), c, **tol(dtype))       # the residual holds the rounded sum
    if dtype == torch.bfloat16:
        assert torch.equal(res.cpu(), (x.float() + u.float()).to(torch.bfloat16))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows, inter", [(1, 8), (5, 200), (33, 8192), (2, 333)])
def test_silu_mul(dtype, rows, inter):
    from tesseract_b200 import kernels

    torch.manual_seed(2)
    gu = (torch.randn(rows, 2 * inter) * 2).to(dtype)
    out = torch.empty(rows, inter, dtype=dtype, device="cuda")
    kernels.silu_mul(dev(gu), out)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    torch.testing.assert_close(out.cpu().double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


@pytest.mark.parametrize("m, n, k", [(1, 1, 1), (3, 5, 7), (64, 64, 16), (65, 130, 33), (200, 96, 96), (17, 331, 72),
                                     (2, 1000, 2048)])
def test_gemm_f32(m, n, k):
    from tesseract_b200 import kernels

    torch.manual_seed(3)
    a, w = torch.randn(m, k), torch.randn(n, k)
    out = torch.empty(m, n, device="cuda")
    kernels.gemm_f32_nt(dev(a), dev(w), out)
    want = a.double() @ w.double().T
    torch.testing.assert_close(out.cpu().double(), want, rtol=1e-5, atol=1e-5 * math.sqrt(k))
    # a row's result does not depend on the rows around it, nor a column's on the other columns
    alone = torch.empty(1, n, device="cuda")
    kernels.gemm_f32_nt(dev(a[m - 1:m].contiguous()), dev(w), alone)
    assert torch.equal(alone[0], out[m - 1])
    # strided operands (a column slice of a wider buffer)
    wide = torch.randn(m, k + 5)
    strided = torch.empty(m, n, device="cuda")
    kernels.gemm_f32_nt(dev(wide)[:, 1:k + 1], dev(w), strided)
    torch.testing.assert_close(strided.cpu().double(), wide[:, 1:k + 1].double() @ w.double().T, rtol=1e-5,
                               atol=1e-5 * math.sqrt(k))


def test_gemm_f32_is_true_32_bit():
    """A product that a reduced-precision matrix mode (10-bit mantissa) would get visibly wrong."""
    from tesseract_b200 import kernels

    a = torch.full((4, 64), 1.0 + 2.0 ** -12)
    w = torch.full((8, 64), 1.0 + 2.0 ** -13)
    out = torch.empty(4, 8, device="cuda")
    kernels.gemm_f32_nt(dev(a), dev(w), out)
    want = 64 * (1.0 + 2.0 ** -12) * (1.0 + 2.0 ** -13)
    assert abs(out[0, 0].item() - want) < 1e-5 and abs(64.0 - want) > 1e-2


def paged_case(dtype, lengths, new, nh, nkv, d, page_size, seed, window=0):
    """A batch of sequences with ``lengths[i]`` keys, the last ``new[i]`` of them being this step's rows."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-n // page_size) for n in lengths)
    order = torch.randperm(total_pages + 3, generator=g)[:total_pages].tolist()     # scattered, non-identity pages
    order = [p + 1 for p in order]
    cache = torch.zeros(total_pages + 5, 2, nkv, page_size, d)
    columns = max(-(-n // page_size) for n in lengths)
    table = torch.zeros(len(lengths), columns, dtype=torch.int32)
    ks, vs, at = [], [], 0
    for s, n in enumerate(lengths):
        k, v = torch.randn(n, nkv, d, generator=g), torch.randn(n, nkv, d, generator=g)
        ks.append(k)
        vs.append(v)
        for logical in range(-(-n // page_size)):
            page = order[at]
            at += 1
            table[s, logical] = page
            span = slice(logical * page_size, min(n, (logical + 1) * page_size))
            cache[page, 0, :, :span.stop - span.start] = k[span].transpose(0, 1)
            cache[page, 1, :, :span.stop - span.start] = v[span].transpose(0, 1)
    positions, seq_of_row = [], []
    for s, (n, q) in enumerate(zip(lengths, new)):
        positions += list(range(n - q, n))
        seq_of_row += [s] * q
    q = torch.randn(len(positions), nh, d, generator=g)
    return dict(q=q.to(dtype), ks=[k.to(dtype) for k in ks], vs=[v.to(dtype) for v in vs], cache=cache.to(dtype),
                table=table, positions=torch.tensor(positions, dtype=torch.int32),
                seq_of_row=torch.tensor(seq_of_row, dtype=torch.int32), new=new, lengths=lengths)


def plain_paged_attention(case, scale, window=None):
    """Row by row with the plain whole-sequence attention: row at position p is row p of the full answer."""
    outs = []
    row = 0
    for s, (n, new) in enumerate(zip(case["lengths"], case["new"])):
        k, v = case["ks"][s].double(), case["vs"][s].double()
        q_full = torch.zeros(n, case["q"].shape[1], case["q"].shape[2], dtype=torch.float64)
        q_full[n - new:] = case["q"][row:row + new].double()
        outs.append(llama.attention(q_full, k, v, scale, window)[n - new:])
        row += new
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("lengths, new, nh, nkv, d, page_size, window", [
    ([1], [1], 1, 1, 16, 16, 0),
    ([17, 16, 15, 33], [1, 1, 1, 1], 6, 3, 48, 16, 0),            # decode rows, pages' edges
    ([40, 129, 2, 64], [40, 5, 2, 17], 4, 2, 16, 16, 0),          # portions of prompts at any offset
    ([300, 31], [1, 31], 3, 1, 32, 32, 0),                        # one kv head, larger pages
    ([100, 70], [30, 1], 8, 8, 64, 16, 0),                        # no grouping
    ([200, 90, 33], [16, 1, 33], 4, 2, 128, 64, 0),
    ([150, 64, 10], [20, 1, 10], 4, 2, 32, 16, 24),               # sliding window
    ([5], [5], 5, 5, 256, 16, 0),
])
def test_attention_rows(dtype, lengths, new, nh, nkv, d, page_size, window):
    from tesseract_b200 import kernels

    case = paged_case(dtype, lengths, new, nh, nkv, d, page_size, seed=len(lengths) + d)
    scale = 1.0 / math.sqrt(d)
    rows = case["q"].shape[0]
    out = torch.empty(rows, nh * d, dtype=dtype, device="cuda")
    kernels.attention_rows(dev(case["q"]).view(rows, nh * d), out, dev(case["cache"]), dev(case["positions"]),
                           dev(case["seq_of_row"]), dev(case["table"]), nh, nkv, d, page_size, window, scale)
    want = plain_paged_attention(case, scale, window or None).reshape(rows, nh * d)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 1, 24, 100])
def test_attention_rows_at_the_edges_of_what_a_row_sees(dtype, window):
    """Scores that rise by 8 with every key (the position as 16 * hi + lo in two dimensions, exact in bfloat16 too) give
    all the weight to the LAST key a row sees, falling ones to the FIRST: a mask off by one key at the row's own
    position or at the window's first key returns another key's value."""
    from tesseract_b200 import kernels

    nh, nkv, d, page_size = 4, 2, 32, 16
    lengths, new = [1, 17, 130, 300, 511], [1, 17, 40, 1, 64]
    for direction in (1.0, -1.0):
        case = paged_case(dtype, lengths, new, nh, nkv, d, page_size, seed=window)
        rows = case["q"].shape[0]
        q = torch.zeros(rows, nh, d)
        q[:, :, 3] = direction * 128.0
        q[:, :, 7] = direction * 8.0
        cache = case["cache"].float()
        for s, n in enumerate(lengths):
            k = torch.zeros(n, nkv, d)
            where = torch.arange(n)
            k[:, :, 3] = (where // 16).float()[:, None]
            k[:, :, 7] = (where % 16).float()[:, None]
            for logical in range(-(-n // page_size)):
                pg = int(case["table"][s, logical])
                span = slice(logical * page_size, min(n, (logical + 1) * page_size))
                cache[pg, 0, :, :span.stop - span.start] = k[span].transpose(0, 1)
        out = torch.empty(rows, nh * d, dtype=dtype, device="cuda")
        kernels.attention_rows(dev(q.to(dtype)).view(rows, nh * d), out, dev(cache.to(dtype)), dev(case["positions"]),
                               dev(case["seq_of_row"]), dev(case["table"]), nh, nkv, d, page_size, window, 1.0)
        for r in range(rows):
            s, position = int(case["seq_of_row"][r]), int(case["positions"][r])
            first = max(0, position - window + 1) if window else 0
            target = position if direction > 0 else first
            want = case["vs"][s][target].float().repeat_interleave(nh // nkv, dim=0).reshape(nh * d)
            torch.testing.assert_close(out[r].cpu().float(), want, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """One query and one far key are scaled so that a single score stands out: the row must return that key's value,
    wherever in the pages it lies (first key, a page's last slot, a page's first slot, the row's own position)."""
    from tesseract_b200 import kernels

    nh, nkv, d, page_size, n = 4, 2, 32, 16, 700
    for target in (0, 15, 16, 351, 687, 699):
        case = paged_case(dtype, [n], [1], nh, nkv, d, page_size, seed=target)
        q = torch.zeros(1, nh, d)
        q[0, :, 3] = 60.0
        k = case["ks"][0].float()
        k[:, :, 3] = 0.0
        k[target, :, 3] = 8.0
        page, slot = int(case["table"][0, target // page_size]), target % page_size
        cache = case["cache"].float()
        for logical in range(-(-n // page_size)):
            p = int(case["table"][0, logical])
            span = slice(logical * page_size, min(n, (logical + 1) * page_size))
            cache[p, 0, :, :span.stop - span.start] = k[span].transpose(0, 1)
        out = torch.empty(1, nh * d, dtype=dtype, device="cuda")
        kernels.attention_rows(dev(q.to(dtype)).view(1, nh * d), out, dev(cache.to(dtype)), dev(case["positions"]),
                               dev(case["seq_of_row"]), dev(case["table"]), nh, nkv, d, page_size, 0, 1.0)
        want = case["vs"][0][target].float().repeat_interleave(nh // nkv, dim=0).reshape(1, nh * d)
        torch.testing.assert_close(out.cpu().float(), want, rtol=1e-2, atol=1e-2)
        assert cache[page, 0, 0, slot, 3] == 8.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkv, d, page_size, scaling", [
    (4, 2, 16, 16, None), (3, 1, 32, 16, "llama3"), (6, 3, 48, 32, None), (2, 2, 128, 64, "llama3")])
def test_rope_kv_write(dtype, nh, nkv, d, page_size, scaling):
    from tesseract_b200 import kernels
    from tesseract_b200.parts.rotary import rotary_inverse_frequencies

    torch.manual_seed(5)
    scaling = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                   original_max_position_embeddings=64) if scaling else None
    inv_freq = rotary_inverse_frequencies(d, 500000.0 if scaling else 10000.0, scaling)
    begins, news = [0, 37, 1000], [20, 1, 3]
    positions = [p for b, n in zip(begins, news) for p in range(b, b + n)]
    seq_of_row = [s for s, n in enumerate(news) for _ in range(n)]
    rows = len(positions)
    columns = max(-(-(b + n) // page_size) for b, n in zip(begins, news))
    table = torch.zeros(3, columns, dtype=torch.int32)
    page = 1
    for s, (b, n) in enumerate(zip(begins, news)):
        for logical in range(b // page_size, -(-(b + n) // page_size)):
            table[s, logical] = page
            page += 1
    qkv = torch.randn(rows, (nh + 2 * nkv) * d).to(dtype)
    cache = torch.zeros(page + 1, 2, nkv, page_size, d, dtype=dtype, device="cuda")
    buf = dev(qkv.clone())
    kernels.rope_kv_write(buf, dev(torch.tensor(positions, dtype=torch.int32)),
                          dev(torch.tensor(seq_of_row, dtype=torch.int32)), dev(table),
                          dev(torch.from_numpy(inv_freq)), cache, nh, nkv, d, page_size)
    cos, sin = llama.rope_tables(positions, inv_freq)
    q = qkv[:, :nh * d].double().view(rows, nh, d)
    k = qkv[:, nh * d:(nh + nkv) * d].double().view(rows, nkv, d)
    v = qkv[:, (nh + nkv) * d:].view(rows, nkv, d)
    torch.testing.assert_close(buf.cpu()[:, :nh * d].double().view(rows, nh, d), llama.rotate_half(q, cos, sin),
                               **tol(dtype))
    k_rot = llama.rotate_half(k, cos, sin)
    host = cache.cpu()
    for r, (p, s) in enumerate(zip(positions, seq_of_row)):
        pg, slot = int(table[s, p // page_size]), p % page_size
        torch.testing.assert_close(host[pg, 0, :, slot].double(), k_rot[r], **tol(dtype))
        assert torch.equal(host[pg, 1, :, slot], v[r])                  # values are stored as they are
    assert torch.equal(buf.cpu()[:, nh * d:], qkv[:, nh * d:])          # k and v columns of the buffer are untouched
    assert host[0].abs().sum() == 0                                      # nothing strayed into the scratch page


@pytest.mark.parametrize("rows, vocab", [(1, 5), (4, 331), (3, 128256), (70, 1000)])
def test_argmax_lowest_index_on_ties(rows, vocab):
    from tesseract_b200 import kernels

    torch.manual_seed(6)
    logits = torch.randn(rows, vocab)
    logits[0, vocab // 2] = 50.0
    if vocab > 4:
        logits[0, vocab - 1] = 50.0            # a tie: the lower index wins
        logits[rows - 1, 1] = logits[rows - 1].max() + 1
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    kernels.argmax(dev(logits), out)
    want = [int(np.flatnonzero(r == r.max())[0]) for r in logits.numpy()]
    assert out.cpu().tolist() == want


@pytest.mark.parametrize("vocab", [7, 384, 5000, 128256])
def test_temperature_sampling_follows_the_inverse_cdf(vocab):
    from tesseract_b200 import kernels

    rng = np.random.default_rng(vocab)
    rows = 24
    logits = (rng.normal(size=(rows, vocab)) * 2).astype(np.float32)
    temps = rng.uniform(0.3, 1.5, size=rows).astype(np.float32)
    temps[3] = 0.0                              # a greedy row in the same call
    draws = rng.uniform(size=rows)
    draws[0], draws[1] = 0.0, 1.0 - 2.0 ** -53
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    kernels.sample(dev(torch.from_numpy(logits)), dev(torch.from_numpy(temps)), dev(torch.from_numpy(draws)), out)
    got = out.cpu().tolist()
    for r in range(rows):
        want = llama.sample_in_token_order(logits[r], float(temps[r]), float(draws[r]))
        if got[r] != want:
            scaled = logits[r] * (np.float32(1.0) / temps[r])
            cdf = np.cumsum(np.exp((scaled - scaled.max()).astype(np.float64)))
            cdf /= cdf[-1]
            assert abs(cdf[min(got[r], want)] - draws[r]) < 1e-9, f"row {r}: sampled {got[r]}, plain says {want}"
    # the empirical distribution of one row follows softmax(l / T)
    row = (rng.normal(size=(1, 16)) * 1.5).astype(np.float32)
    n = 4000
    many = torch.from_numpy(np.repeat(row, n, axis=0))
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    kernels.sample(dev(many), dev(torch.full((n,), 0.8)), dev(torch.from_numpy(rng.uniform(size=n))), out)
    freq = np.bincount(out.cpu().numpy(), minlength=16) / n
    p = np.exp(row[0] / 0.8 - (row[0] / 0.8).max())
    p /= p.sum()
    assert np.abs(freq - p).max() < 0.03


def test_kernels_refuse_what_they_cannot_do():
    from tesseract_b200 import kernels

    with pytest.raises(kernels.KernelError):
        kernels.rms_norm(torch.zeros(2, 8), torch.ones(8), 1e-5, torch.zeros(2, 8))          # not on the device
    with pytest.raises(kernels.KernelError):
        kernels.rms_norm(torch.zeros(2, 8, device="cuda", dtype=torch.float16), torch.ones(8, device="cuda"), 1e-5,
                         torch.zeros(2, 8, device="cuda", dtype=torch.float16))               # unsupported dtype
    q = torch.zeros(1, 2 * 20, device="cuda")
    with pytest.raises(kernels.KernelError):                                                   # head_dim 20
        kernels.attention_rows(q, torch.empty_like(q), torch.zeros(2, 2, 1, 16, 20, device="cuda"),
                               torch.zeros(1, dtype=torch.int32, device="cuda"),
                               torch.zeros(1, dtype=torch.int32, device="cuda"),
                               torch.zeros(1, 1, dtype=torch.int32, device="cuda"), 2, 1, 20, 16, 0, 1.0)


def run_attention_mma(case, nh, nkv, d, page_size, window, scale, splits):
    from tesseract_b200 import kernels

    rows = case["q"].shape[0]
    new, lengths = case["new"], case["lengths"]
    row_start = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32)
    seq_begin = torch.tensor([n - q for n, q in zip(lengths, new)], dtype=torch.int32)
    fold = nh // nkv
    out = torch.full((rows, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    kernels.attention_mma(dev(case["q"]).view(rows, nh * d), out, dev(case["cache"]), dev(row_start), dev(seq_begin),
                          dev(case["table"]), len(lengths), max(new), nh, nkv, d, page_size, window, scale,
                          any(n * fold > 16 for n in new), any(n * fold <= 16 for n in new), splits)
    return out


@pytest.mark.parametrize("lengths, nh, nkv, d, page_size, window, splits, scaling, write_kv", [
    ([1, 16, 17, 333], 6, 3, 48, 16, 0, 1, None, True),               # the new key first, last and alone in a page
    ([700, 64, 65, 1, 33], 32, 8, 64, 16, 0, 4, "llama3", True),      # splits as a cluster
    ([2100, 500], 8, 2, 128, 32, 0, 12, "llama3", True),              # splits through scratch memory
    ([150, 64, 10], 4, 2, 32, 16, 24, 2, None, True),                 # sliding window
    ([90, 41], 5, 5, 256, 16, 0, 2, None, True),                      # the widest head, no grouping
    ([129, 40], 4, 1, 16, 16, 0, 3, "none", True),                    # no rotation at all
    ([129, 40], 8, 2, 64, 16, 0, 3, "llama3", False),                 # reads a cache that another layer wrote
    ([7 + 5 * k for k in range(40)], 16, 8, 64, 16, 0, 1, "llama3", True),   # 320 CTAs: the four-warp form
])
def test_attention_decode_rope_equals_rope_then_attention(lengths, nh, nkv, d, page_size, window, splits, scaling,
                                                          write_kv):
    """The fused decode kernel against the two kernels it replaces: same output bits, same cache bits."""
    from tesseract_b200 import kernels
    from tesseract_b200.parts.rotary import rotary_inverse_frequencies

    case = paged_case(torch.bfloat16, lengths, [1] * len(lengths), nh, nkv, d, page_size, seed=21)
    n = len(lengths)
    inv_freq = None
    if scaling != "none":
        rope = dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                    original_max_position_embeddings=64) if scaling else None
        inv_freq = dev(torch.from_numpy(rotary_inverse_frequencies(d, 500000.0 if scaling else 10000.0, rope)))
    torch.manual_seed(3)
    qkv = dev(torch.randn(n, (nh + 2 * nkv) * d).to(torch.bfloat16))
    row_start = dev(torch.arange(n + 1, dtype=torch.int32))
    seq_begin = dev(torch.tensor([length - 1 for length in lengths], dtype=torch.int32))
    table, positions, seq_of_row = dev(case["table"]), dev(case["positions"]), dev(case["seq_of_row"])
    scale = 1.0 / math.sqrt(d)

    cache_a, qkv_a = dev(case["cache"]).clone(), qkv.clone()
    kernels.rope_kv_write(qkv_a, positions, seq_of_row, table, inv_freq, cache_a, nh, nkv, d, page_size,
                          write_kv=write_kv)
    out_a = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    kernels.attention_mma(qkv_a[:, :nh * d], out_a, cache_a, row_start, seq_begin, table, n, 1, nh, nkv, d, page_size,
                          window, scale, False, True, splits)

    cache_b = dev(case["cache"]).clone()
    out_b = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    kernels.attention_decode_rope(qkv, out_b, cache_b, row_start, seq_begin, table, n, nh, nkv, d, page_size, window,
                                  scale, inv_freq, write_kv, splits)
    torch.cuda.synchronize()
    assert not torch.isnan(out_b.float()).any()
    assert torch.equal(out_a, out_b)
    assert torch.equal(cache_a, cache_b)
    if not write_kv:
        assert torch.equal(cache_b, dev(case["cache"]))                # a reader leaves the cache alone


@pytest.mark.parametrize("lengths, new, nh, nkv, d, page_size, window, splits", [
    ([1], [1], 1, 1, 16, 16, 0, 1),
    ([17, 16, 15, 33], [1, 1, 1, 1], 6, 3, 48, 16, 0, 1),             # decode rows at pages' edges
    ([17, 16, 15, 333], [1, 1, 1, 1], 6, 3, 48, 16, 0, 3),            # the same, keys split three ways
    ([700, 64, 65, 1], [1, 1, 1, 1], 32, 8, 64, 16, 0, 8),            # more splits than some sequences have tiles
    ([900, 64, 65, 1], [1, 1, 2, 1], 32, 8, 64, 16, 0, 12),           # too many splits for a cluster: scratch memory
    ([500, 40], [1, 1], 8, 2, 128, 16, 0, 5),                          # five splits of a wide head as a cluster
    ([40, 129, 2, 64], [40, 5, 2, 17], 4, 2, 16, 16, 0, 2),           # long and short sequences in one batch
    ([300, 31], [1, 31], 3, 1, 32, 32, 0, 4),                          # one kv head, larger pages
    ([100, 70], [30, 1], 8, 8, 64, 16, 0, 1),                          # no grouping
    ([200, 90, 33], [16, 1, 33], 4, 2, 128, 64, 0, 2),
    ([150, 64, 10, 200], [20, 1, 10, 1], 4, 2, 32, 16, 24, 2),        # sliding window
    ([5, 300], [5, 2], 5, 5, 256, 16, 0, 2),
    ([260, 70], [200, 3], 2, 1, 80, 16, 0, 1),                         # a head size between the padded widths
    ([513], [513], 32, 8, 64, 16, 0, 1),                               # many tiles of one long prompt
    ([90, 5], [2, 1], 32, 2, 96, 16, 0, 2),                            # a group of 16 heads: one token fills a tile
    ([90, 50], [2, 1], 40, 2, 16, 16, 0, 1),                           # a group of 20: decode goes to the tile kernel
    ([3 + 2 * k for k in range(75)], [1] * 75, 8, 4, 64, 16, 0, 1),   # 300 CTAs without splits: the four-warp form
    ([1 + 3 * k for k in range(100)], [1] * 100, 6, 3, 32, 16, 0, 1), # the same at a narrower head
])
def test_attention_mma(lengths, new, nh, nkv, d, page_size, window, splits):
    case = paged_case(torch.bfloat16, lengths, new, nh, nkv, d, page_size, seed=sum(lengths) + d)
    scale = 1.0 / math.sqrt(d)
    out = run_attention_mma(case, nh, nkv, d, page_size, window, scale, splits)
    rows = case["q"].shape[0]
    want = plain_paged_attention(case, scale, window or None).reshape(rows, nh * d)
    torch.testing.assert_close(out.cpu().double(), want, rtol=2e-2, atol=2e-2)


def test_attention_mma_finds_one_far_key_among_hundreds():
    nh, nkv, d, page_size, n = 8, 2, 64, 16, 1500
    for target in (0, 15, 16, 63, 64, 777, 1487, 1499):
        for new, splits in ((1, 1), (1, 7), (40, 1)):
            case = paged_case(torch.bfloat16, [n], [new], nh, nkv, d, page_size, seed=target + new)
            q = torch.zeros(new, nh, d)
            q[:, :, 3] = 60.0
            case["q"] = q.to(torch.bfloat16)
            k = case["ks"][0].float()
            k[:, :, 3] = 0.0
            k[target, :, 3] = 8.0
            case["ks"][0] = k.to(torch.bfloat16)
            cache = case["cache"].float()
            for logical in range(-(-n // page_size)):
                pg = int(case["table"][0, logical])
                span = slice(logical * page_size, min(n, (logical + 1) * page_size))
                cache[pg, 0, :, :span.stop - span.start] = k[span].transpose(0, 1)
            case["cache"] = cache.to(torch.bfloat16)
            out = run_attention_mma(case, nh, nkv, d, page_size, 0, 1.0, splits)
            # every row at or after the target returns the target's value; earlier rows do not see it
            v = case["vs"][0][target].float().repeat_interleave(nh // nkv, dim=0).reshape(nh * d)
            first_pos = n - new
            for r in range(new):
                if first_pos + r >= target:
                    torch.testing.assert_close(out[r].cpu().float(), v, rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("d", [64, 128])
def test_attention_tcgen05_and_wide_decode_find_one_far_key_among_hundreds(d):
    """One key among 1,500 answers the query (its score stands out by construction): prompt rows on the tcgen05
    kernel and decode rows on the split kernel, at both head sizes, must return that key's value whichever block,
    page or split it lies in."""
    from tesseract_b200 import kernels

    nh, nkv, page_size, n = 8, 2, 16, 1500
    for target in (0, 63, 64, 127, 128, 777, 1471, 1499):
        for new, splits in ((40, 1), (1, 5)):
            case = paged_case(torch.bfloat16, [n], [new], nh, nkv, d, page_size, seed=target + new + d)
            q = torch.zeros(new, nh, d)
            q[:, :, d - 5] = 60.0
            case["q"] = q.to(torch.bfloat16)
            k = case["ks"][0].float()
            k[:, :, d - 5] = 0.0
            k[target, :, d - 5] = 8.0
            case["ks"][0] = k.to(torch.bfloat16)
            cache = case["cache"].float()
            for logical in range(-(-n // page_size)):
                pg = int(case["table"][0, logical])
                span = slice(logical * page_size, min(n, (logical + 1) * page_size))
                cache[pg, 0, :, :span.stop - span.start] = k[span].transpose(0, 1)
            case["cache"] = cache.to(torch.bfloat16)
            if new > 1:
                row_start = torch.tensor([0, new], dtype=torch.int32)
                seq_begin = torch.tensor([n - new], dtype=torch.int32)
                out = torch.full((new, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
                kernels.attention_tcgen05(dev(case["q"]).view(new, nh * d), out, dev(case["cache"]), dev(row_start),
                                          dev(seq_begin), dev(case["table"]), 1, new, nh, nkv, d, page_size, 0, 1.0,
                                          key_splits=1 + target % 4)      # alone, or shared by up to four CTAs
                assert kernels.tcgen05_error() == 0
            else:
                out = run_attention_mma(case, nh, nkv, d, page_size, 0, 1.0, splits)
            v = case["vs"][0][target].float().repeat_interleave(nh // nkv, dim=0).reshape(nh * d)
            first_pos = n - new
            for r in range(new):
                if first_pos + r >= target:
                    torch.testing.assert_close(out[r].cpu().float(), v, rtol=1e-2, atol=1e-2)


def test_silu_mul_interleaved_layout():
    from tesseract_b200 import kernels

    torch.manual_seed(7)
    for dtype in DTYPES:
        for rows, inter in ((3, 8), (5, 200), (17, 8192)):
            gate, up = (torch.randn(rows, inter) * 2).to(dtype), torch.randn(rows, inter).to(dtype)
            merged = torch.stack([gate.view(rows, inter // 8, 8), up.view(rows, inter // 8, 8)], dim=2)
            merged = merged.reshape(rows, 2 * inter).contiguous()
            out = torch.empty(rows, inter, dtype=dtype, device="cuda")
            kernels.silu_mul(dev(merged), out, interleaved=True)
            g, u = gate.double(), up.double()
            torch.testing.assert_close(out.cpu().double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("n, k", [(16, 32), (48, 96), (160, 64), (2048, 2048), (384, 320), (1024, 4096),
                                  (16384, 256), (5024, 96)])       # the last two: 32-feature tiles, several per CTA
def test_decode_linear_plain_and_f32(m, n, k):
    from tesseract_b200 import kernels

    torch.manual_seed(m * 1000 + n + k)
    x = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn(n, k) / math.sqrt(k)).to(torch.bfloat16)
    want = x.double() @ w.double().T
    out = torch.empty(m, n, dtype=torch.bfloat16, device="cuda")
    kernels.decode_linear(dev(w), out, x=dev(x))
    torch.testing.assert_close(out.cpu().double(), want, rtol=1e-2, atol=1e-2)
    out32 = torch.empty(m, n, dtype=torch.float32, device="cuda")
    kernels.decode_linear(dev(w), out32, x=dev(x), epilogue=kernels.EPI_F32)
    torch.testing.assert_close(out32.cpu().double(), want, rtol=1e-4, atol=1e-4)
    # a strided view of a wider buffer as input (a column slice)
    wide = torch.randn(m, k + 16).to(torch.bfloat16)
    kernels.decode_linear(dev(w), out32, x=dev(wide)[:, 8:k + 8], epilogue=kernels.EPI_F32)
    torch.testing.assert_close(out32.cpu().double(), wide[:, 8:k + 8].double() @ w.double().T, rtol=1e-4, atol=1e-4)
    # a row's result does not depend on the rows beside it
    alone = torch.empty(1, n, dtype=torch.float32, device="cuda")
    kernels.decode_linear(dev(w), alone, x=dev(x[m - 1:m].contiguous()), epilogue=kernels.EPI_F32)
    kernels.decode_linear(dev(w), out32, x=dev(x), epilogue=kernels.EPI_F32)
    assert torch.equal(alone[0], out32[m - 1])


@pytest.mark.parametrize("m, n, k, eps", [(1, 64, 64, 1e-5), (7, 160, 96, 1e-6), (8, 3072, 2048, 1e-5), (6, 16384, 2048, 1e-5),
                                          (13, 512, 1024, 1e-3), (16, 256, 2048, 1e-5), (5, 64, 4096, 1e-5)])
def test_decode_linear_fused_norm_and_swiglu(m, n, k, eps):
    from tesseract_b200 import kernels

    torch.manual_seed(m + n + k)
    res = (torch.randn(m, k) * 2).to(torch.bfloat16)
    upd = torch.randn(m, k).to(torch.bfloat16)
    nw = 1 + 0.1 * torch.randn(k)
    w = (torch.randn(n, k) / math.sqrt(k)).to(torch.bfloat16)

    def rounded(t):
        return t.to(torch.bfloat16).double()

    # norm only
    x = rounded(llama.rms_norm(res.double(), nw.double(), eps))
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    kernels.decode_linear(dev(w), out, residual=dev(res), norm_weight=dev(nw), eps=eps, epilogue=kernels.EPI_F32)
    torch.testing.assert_close(out.cpu().double(), x @ w.double().T, rtol=2e-2, atol=2e-2)
    # add + norm, new residual written apart
    c = res.double() + upd.double()
    x = rounded(llama.rms_norm(c, nw.double(), eps))
    new_res = torch.zeros(m, k, dtype=torch.bfloat16, device="cuda")
    res_dev = dev(res)
    kernels.decode_linear(dev(w), out, residual=res_dev, update=dev(upd), norm_weight=dev(nw), eps=eps,
                          residual_out=new_res, epilogue=kernels.EPI_F32)
    torch.testing.assert_close(out.cpu().double(), x @ w.double().T, rtol=2e-2, atol=2e-2)
    assert torch.equal(new_res.cpu(), (res.float() + upd.float()).to(torch.bfloat16))
    assert torch.equal(res_dev.cpu(), res)                                   # the old residual is left alone
    with pytest.raises(kernels.KernelError):
        kernels.decode_linear(dev(w), out, residual=res_dev, update=dev(upd), norm_weight=dev(nw), eps=eps,
                              residual_out=res_dev, epilogue=kernels.EPI_F32)
    # add + norm + gate/up + activation
    gate, up = w[: n // 2], w[n // 2:]
    merged = torch.stack([gate.view(n // 16, 8, k), up.view(n // 16, 8, k)], dim=1).reshape(n, k).contiguous()
    act = torch.empty(m, n // 2, dtype=torch.bfloat16, device="cuda")
    kernels.decode_linear(dev(merged), act, residual=res_dev, update=dev(upd), norm_weight=dev(nw), eps=eps,
                          residual_out=new_res, epilogue=kernels.EPI_SWIGLU)
    g, u = x @ gate.double().T, x @ up.double().T
    torch.testing.assert_close(act.cpu().double(), g / (1 + torch.exp(-g)) * u, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m, inner, hidden, wide, eps", [(8, 2048, 2048, 3072, 1e-5), (3, 96, 160, 64, 1e-6),
                                                         (13, 320, 512, 1024, 1e-5), (1, 8192, 2048, 16384, 1e-5),
                                                         (16, 64, 5024, 48, 1e-3)])
def test_decode_linear_prepares_the_following_norm(m, inner, hidden, wide, eps):
    """A product that also does the work of the norm behind it (new residual, rows times the norm's weights, sums
    of squares per tile), and the product behind that, which applies the norm's scale to its 32-bit sums: together
    add + RMSNorm + product, with one rounding of the operand as in the reference's order, placed before the scale
    instead of after it."""
    from tesseract_b200 import kernels

    torch.manual_seed(m + inner + hidden)
    bf = torch.bfloat16
    x = torch.randn(m, inner).to(bf)
    w_first = (torch.randn(hidden, inner) / math.sqrt(inner)).to(bf)
    res = (torch.randn(m, hidden) * 2).to(bf)
    nw = 1 + 0.1 * torch.randn(hidden)
    w_second = (torch.randn(wide, hidden) / math.sqrt(hidden)).to(bf)
    tiles = hidden // kernels.decode_linear_tile_features(hidden)
    res_out = torch.zeros(m, hidden, dtype=bf, device="cuda")
    rows = torch.zeros(m, hidden, dtype=bf, device="cuda")
    sums = torch.full((tiles, kernels.SS_STRIDE), float("nan"), device="cuda")
    res_dev = dev(res)
    kernels.decode_linear(dev(w_first), None, x=dev(x), prepare=(res_dev, dev(nw), res_out, rows, sums))
    o = (x.double() @ w_first.double().T).to(bf)                       # the product as it would be stored alone
    c = res.double() + o.double()
    close = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(res_out.cpu().double(), c, **close)
    torch.testing.assert_close(rows.cpu().double(), c * nw.double(), **close)
    assert torch.equal(res_dev.cpu(), res)                                  # the old residual is left alone
    got_sums = sums.cpu().double()
    assert torch.isfinite(got_sums).all() and (got_sums[:, m:] == 0).all()   # rows beyond M hold zeros
    torch.testing.assert_close(got_sums[:, :m].sum(0), (c * c).sum(1), rtol=2e-2, atol=1e-3)
    # the product behind: scale from the sums, operand as prepared
    out = torch.empty(m, wide, dtype=torch.float32, device="cuda")
    kernels.decode_linear(dev(w_second), out, x=rows, scaled_by=sums, eps=eps, epilogue=kernels.EPI_F32)
    exact_c = res_out.cpu().double()        # what the kernel itself rounded: its statistics come from the unrounded c
    s = torch.rsqrt(got_sums[:, :m].sum(0) / hidden + eps)[:, None]
    torch.testing.assert_close(out.cpu().double(), (rows.cpu().double() @ w_second.double().T) * s, rtol=1e-4, atol=1e-4)
    reference = llama.rms_norm(c, nw.double(), eps).to(bf).double() @ w_second.double().T
    torch.testing.assert_close(out.cpu().double(), reference, **close)
    if wide % 16 == 0 and (wide // 2) % 8 == 0:
        act = torch.empty(m, wide // 2, dtype=bf, device="cuda")
        kernels.decode_linear(dev(w_second), act, x=rows, scaled_by=sums, eps=eps, epilogue=kernels.EPI_SWIGLU)
        y = out.cpu().double().view(m, wide // 16, 2, 8)
        g, u = y[:, :, 0].reshape(m, wide // 2), y[:, :, 1].reshape(m, wide // 2)
        torch.testing.assert_close(act.cpu().double(), g / (1 + torch.exp(-g)) * u, **close)
    with pytest.raises(kernels.KernelError):       # the new residual needs a buffer of its own
        kernels.decode_linear(dev(w_first), None, x=dev(x), prepare=(res_dev, dev(nw), res_dev, rows, sums))


@pytest.mark.parametrize("m, n, k", [(8, 128256, 256), (3, 5024, 96), (16, 331 * 16, 64), (1, 48, 32)])
def test_two_stage_argmax_through_the_product_and_the_sampler(m, n, k):
    """The product that writes 32-bit logits leaves each CTA's best value per row and its lowest column; the
    sampler takes a greedy row's token from those alone and a sampled row's maximum (so the same token as without
    them); ties go to the lowest token wherever in the vocabulary they lie."""
    from tesseract_b200 import kernels

    torch.manual_seed(n + m)
    x = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn(n, k) / math.sqrt(k)).to(torch.bfloat16)
    # two identical weight rows far apart (in different tiles and CTAs) that row 0 scores highest: a tie
    tie_lo, tie_hi = 5, n - 3
    w[tie_lo] = w[tie_hi] = (x[0].float() * 4 / x[0].float().norm()).to(torch.bfloat16)
    out = torch.empty(m, n, dtype=torch.float32, device="cuda")
    shape = (kernels.decode_linear_ctas(n), kernels.SS_STRIDE)
    values = torch.full(shape, float("nan"), device="cuda")
    indices = torch.full(shape, -7, dtype=torch.int32, device="cuda")
    kernels.decode_linear(dev(w), out, x=dev(x), epilogue=kernels.EPI_F32, best=(values, indices))
    logits = out.cpu()
    got_best = values.cpu()[:, :m].max(0).values
    assert torch.equal(got_best, logits.max(1).values)
    temperature = torch.tensor([0.0 if r % 2 == 0 else 0.7 for r in range(m)], device="cuda")
    uniform = torch.tensor([0.1 + 0.8 * r / max(1, m - 1) for r in range(m)], dtype=torch.float64, device="cuda")
    with_parts = torch.full((m,), -1, dtype=torch.int32, device="cuda")
    without = torch.full((m,), -1, dtype=torch.int32, device="cuda")
    kernels.sample(out, temperature, uniform, with_parts, partials=(values, indices))
    kernels.sample(out, temperature, uniform, without)
    assert torch.equal(with_parts, without)
    assert int(with_parts[0]) == tie_lo and logits[0, tie_lo] == logits[0, tie_hi]
    for r in range(0, m, 2):
        row = logits[r]
        assert int(with_parts[r]) == int((row == row.max()).nonzero()[0])


def test_decode_linear_refuses_other_sizes():
    from tesseract_b200 import kernels

    assert not kernels.decode_linear_supported(17, 64, 64)
    assert not kernels.decode_linear_supported(4, 72, 64)
    assert not kernels.decode_linear_supported(4, 64, 72)
    assert kernels.decode_linear_supported(16, 128256, 2048, kernels.PRO_ADD_NORM)
    assert not kernels.decode_linear_supported(16, 64, 8192, kernels.PRO_ADD_NORM)      # rows would not fit shared memory
    with pytest.raises(kernels.KernelError):
        kernels.decode_linear(torch.zeros(64, 72, dtype=torch.bfloat16, device="cuda"),
                              torch.zeros(2, 64, dtype=torch.bfloat16, device="cuda"),
                              x=torch.zeros(2, 72, dtype=torch.bfloat16, device="cuda"))


@pytest.mark.parametrize("m, n, k", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (1, 256, 64), (130, 264, 72),
                                     (2048, 3072, 2048), (333, 1000, 520), (77, 16, 8), (64, 1000, 520),
                                     (96, 40000, 1024)])
@pytest.mark.parametrize("form", ["single", "pair", "pair448"])
def test_gemm_tcgen05(m, n, k, form):
    """Single CTAs on 128 x 256 tiles, CTA pairs on 256 x 256 tiles (tcgen05.mma.cta_group::2) and pairs on 256 x 448
    tiles (two products a step into one accumulator), each at every size: fewer rows than a tile, edges in every
    dimension, more tiles than CTAs (both accumulators in turn), a ring that turns many times."""
    from tesseract_b200 import kernels

    pair = dict(pair=form != "single", tile_width={"single": 0, "pair": 256, "pair448": 448}[form])

    torch.manual_seed(m + n + k)
    a = torch.randn(m, k).to(torch.bfloat16)
    w = (torch.randn(n, k) / math.sqrt(k)).to(torch.bfloat16)
    want = a.double() @ w.double().T
    out32 = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    kernels.gemm_tcgen05(dev(a), dev(w), out32, epilogue=kernels.EPI_F32, **pair)
    assert kernels.tcgen05_error() == 0, "a bounded wait inside the kernel ran out"
    torch.testing.assert_close(out32.cpu().double(), want, rtol=1e-4, atol=1e-4)
    out = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
    kernels.gemm_tcgen05(dev(a), dev(w), out, **pair)
    assert kernels.tcgen05_error() == 0
    torch.testing.assert_close(out.cpu().double(), want, rtol=1e-2, atol=1e-2)
    if n % 16 == 0:
        gate, up = w[: n // 2], w[n // 2:]
        merged = torch.stack([gate.view(n // 16, 8, k), up.view(n // 16, 8, k)], dim=1).reshape(n, k).contiguous()
        act = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
        kernels.gemm_tcgen05(dev(a), dev(merged), act, epilogue=kernels.EPI_SWIGLU, **pair)
        assert kernels.tcgen05_error() == 0
        g, u = a.double() @ gate.double().T, a.double() @ up.double().T
        torch.testing.assert_close(act.cpu().double(), g / (1 + torch.exp(-g)) * u, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("window", [0, 1, 100, 333])
@pytest.mark.parametrize("splits", [1, 3, 12])
def test_decode_attention_at_the_edges_of_what_a_row_sees(window, splits, d):
    """The same construction for single decode rows on the split kernel (the prompt kernel's test below explains it):
    sequences whose last key, and whose window's first key, fall at a page's first and last place, at a tile's and
    at a split's."""
    nh, nkv, page_size = 8, 2, 16
    lengths = [1, 16, 17, 130, 257, 300, 511, 640, 1025]
    for direction in (1.0, -1.0):
        case = paged_case(torch.bfloat16, lengths, [1] * len(lengths), nh, nkv, d, page_size, seed=window + splits + d)
        q = torch.zeros(len(lengths), nh, d)
        q[:, :, 3] = direction * 128.0
        q[:, :, 7] = direction * 8.0
        case["q"] = q.to(torch.bfloat16)
        cache = case["cache"].float()
        for s, n in enumerate(lengths):
            k = torch.zeros(n, nkv, d)
            where = torch.arange(n)
            k[:, :, 3] = (where // 16).float()[:, None]
            k[:, :, 7] = (where % 16).float()[:, None]
            case["ks"][s] = k.to(torch.bfloat16)
            for logical in range(-(-n // page_size)):
                pg = int(case["table"][s, logical])
                span = slice(logical * page_size, min(n, (logical + 1) * page_size))
                cache[pg, 0, :, :span.stop - span.start] = k[span].transpose(0, 1)
        case["cache"] = cache.to(torch.bfloat16)
        out = run_attention_mma(case, nh, nkv, d, page_size, window, 1.0, splits)
        for s, n in enumerate(lengths):
            first = max(0, n - window) if window else 0
            target = n - 1 if direction > 0 else first
            want = case["vs"][s][target].float().repeat_interleave(nh // nkv, dim=0).reshape(nh * d)
            torch.testing.assert_close(out[s].cpu().float(), want, rtol=1e-2, atol=1e-2,
                                       msg=lambda m: f"sequence of {n} keys (window {window}, scores "
                                                     f"{'rising' if direction > 0 else 'falling'}): {m}")


@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("n, new, window", [(700, 300, 0), (700, 300, 130), (1100, 420, 300), (520, 130, 1)])
def test_attention_tcgen05_at_the_edges_of_what_a_row_sees(n, new, window, d):
    """Scores that grow by 8 with every key (the position written into two dimensions as 16 * hi + lo, exact in
    bfloat16) make the LAST key a row sees take all the weight; scores that fall by 8 make the FIRST one take it.  A
    mask off by one key at either edge (the row's own position; the window's first key) returns the wrong key's
    value, whichever block, chunk or CTA the edge falls into."""
    from tesseract_b200 import kernels

    nh, nkv, page_size = 8, 2, 16
    for direction in (1.0, -1.0):
        case = paged_case(torch.bfloat16, [n], [new], nh, nkv, d, page_size, seed=n + new + window + d)
        k = torch.zeros(n, nkv, d)
        where = torch.arange(n)
        k[:, :, 3] = (where // 16).float()[:, None]
        k[:, :, 7] = (where % 16).float()[:, None]
        q = torch.zeros(new, nh, d)
        q[:, :, 3] = direction * 128.0
        q[:, :, 7] = direction * 8.0
        case["q"], case["ks"][0] = q.to(torch.bfloat16), k.to(torch.bfloat16)
        cache = case["cache"].float()
        for logical in range(-(-n // page_size)):
            pg = int(case["table"][0, logical])
            span = slice(logical * page_size, min(n, (logical + 1) * page_size))
            cache[pg, 0, :, :span.stop - span.start] = k[span].transpose(0, 1)
        case["cache"] = cache.to(torch.bfloat16)
        row_start = torch.tensor([0, new], dtype=torch.int32)
        seq_begin = torch.tensor([n - new], dtype=torch.int32)
        tiles = kernels.attention_tcgen05_tile_ctas(1, new, nh, nkv)
        for key_splits in (1, 2):
            if tiles * key_splits > 2 * kernels.sm_count():
                continue
            out = torch.full((new, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
            kernels.attention_tcgen05(dev(case["q"]).view(new, nh * d), out, dev(case["cache"]), dev(row_start),
                                      dev(seq_begin), dev(case["table"]), 1, new, nh, nkv, d, page_size, window, 1.0,
                                      key_splits=key_splits)
            assert kernels.tcgen05_error() == 0
            values = case["vs"][0].float()
            for r in range(new):
                position = n - new + r
                first = max(0, position - window + 1) if window else 0
                target = position if direction > 0 else first
                want = values[target].repeat_interleave(nh // nkv, dim=0).reshape(nh * d)
                torch.testing.assert_close(out[r].cpu().float(), want, rtol=1e-2, atol=1e-2,
                                           msg=lambda m: f"row at position {position} (window {window}, scores "
                                                         f"{'rising' if direction > 0 else 'falling'}, "
                                                         f"{key_splits} CTAs a tile): {m}")


@pytest.mark.parametrize("lengths, new, nh, nkv, page_size, window", [
    ([40], [40], 4, 4, 16, 0),                                  # a single block, rows beyond the sequence masked
    ([100, 70], [30, 1], 8, 8, 16, 0),                          # no grouping; the decode row is left to the other kernel
    ([513], [513], 32, 8, 16, 0),                               # many tiles and blocks of one long prompt
    ([700, 300, 129], [129, 300, 5], 8, 2, 16, 0),              # portions at offsets, blocks crossing page edges
    ([1000], [200], 4, 1, 64, 0),                               # one kv head, larger pages
    ([600, 90], [260, 90], 4, 2, 16, 100),                      # sliding window
    ([300], [17], 16, 1, 16, 0),                                # a group of 16: two tokens fill a tile row block
    ([333, 90], [200, 90], 4, 2, 8, 0),                         # the smallest pages: sixteen or eight copies a block
    ([500], [300], 6, 3, 32, 64),                               # pages of 32 keys, a window
    ([700], [300], 24, 8, 16, 0),                               # a group of three: tiles begin inside a position
    ([900, 40], [420, 40], 12, 4, 16, 200),                     # the same with a window over several blocks
])
@pytest.mark.parametrize("d", [64, 128])
def test_attention_tcgen05(lengths, new, nh, nkv, page_size, window, d):
    from tesseract_b200 import kernels

    case = paged_case(torch.bfloat16, lengths, new, nh, nkv, d, page_size, seed=sum(lengths))
    scale = 1.0 / math.sqrt(d)
    rows = case["q"].shape[0]
    row_start = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32)
    seq_begin = torch.tensor([n - q for n, q in zip(lengths, new)], dtype=torch.int32)
    out = torch.full((rows, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
    kernels.attention_tcgen05(dev(case["q"]).view(rows, nh * d), out, dev(case["cache"]), dev(row_start), dev(seq_begin),
                              dev(case["table"]), len(lengths), max(new), nh, nkv, d, page_size, window, scale)
    assert kernels.tcgen05_error() == 0, "a bounded wait inside the kernel ran out"
    want = plain_paged_attention(case, scale, window or None).reshape(rows, nh * d)
    fold = nh // nkv
    at = 0
    for n in new:
        got = out[at:at + n].cpu()
        if n * fold > 16:
            torch.testing.assert_close(got.double(), want[at:at + n], rtol=2e-2, atol=2e-2)
        else:
            assert torch.isnan(got.float()).all()           # short sequences are not this kernel's
        at += n
    # the same with every tile shared by several CTAs, each over a run of the tile's key blocks (some runs are empty:
    # early tiles have fewer blocks than CTAs), twice in a row (the arrival counters must be left as found)
    tiles = kernels.attention_tcgen05_tile_ctas(len(lengths), max(new), nh, nkv)
    for key_splits in (2, 3, 8):
        if tiles * key_splits > 2 * kernels.sm_count():
            continue
        for _ in range(2):
            shared = torch.full((rows, nh * d), float("nan"), dtype=torch.bfloat16, device="cuda")
            kernels.attention_tcgen05(dev(case["q"]).view(rows, nh * d), shared, dev(case["cache"]), dev(row_start),
                                      dev(seq_begin), dev(case["table"]), len(lengths), max(new), nh, nkv, d, page_size,
                                      window, scale, key_splits=key_splits)
            assert kernels.tcgen05_error() == 0
            at = 0
            for n in new:
                if n * fold > 16:
                    torch.testing.assert_close(shared[at:at + n].cpu().double(), want[at:at + n], rtol=2e-2, atol=2e-2)
                    torch.testing.assert_close(shared[at:at + n].float(), out[at:at + n].float(), rtol=2e-2, atol=1e-2)
                else:
                    assert torch.isnan(shared[at:at + n].float()).all()
                at += n


@pytest.mark.parametrize("m, n, k", [(64, 2048, 2048), (17, 3072, 2048), (128, 2048, 8192), (100, 200, 136),
                                     (33, 16384, 2048), (48, 20000, 64), (1, 128, 8), (96, 1152, 5120),
                                     (21, 201, 72)])
def test_skinny_tcgen05_against_a_plain_product(m, n, k):
    """The swapped-operand tcgen05 product for up to 128 rows against a 64-bit product: every split count (one tile
    per SM and fewer, K splits meeting in a cluster), several tiles per CTA, sizes that are no multiple of a tile,
    bfloat16 and 32-bit stores, and SwiGLU on interleaved rows."""
    from tesseract_b200 import kernels

    torch.manual_seed(m + n + k)
    bf = torch.bfloat16
    x = torch.randn(m, k).to(bf)
    w = (torch.randn(n, k) / math.sqrt(k)).to(bf)
    exact = x.double() @ w.double().T
    out32 = torch.full((m, n), float("nan"), device="cuda")
    kernels.skinny_tcgen05(dev(x), dev(w), out32, epilogue=kernels.EPI_F32)
    torch.testing.assert_close(out32.cpu().double(), exact, rtol=1e-4, atol=1e-4)
    out16 = torch.zeros(m, n, dtype=bf, device="cuda")
    kernels.skinny_tcgen05(dev(x), dev(w), out16)
    assert torch.equal(out16.cpu(), out32.cpu().to(bf))
    # rows with a stride of their own (a slice of a wider buffer)
    wide = torch.zeros(m, k + 64, dtype=bf, device="cuda")
    wide[:, 8:k + 8] = dev(x)
    again = torch.zeros(m, n, dtype=bf, device="cuda")
    kernels.skinny_tcgen05(wide[:, 8:k + 8], dev(w), again)
    assert torch.equal(again, out16)
    # and an output that is a column slice of a wider buffer (rows that do not start on 8-byte boundaries)
    framed = torch.full((m, n + 3), 7.0, dtype=bf, device="cuda")
    kernels.skinny_tcgen05(dev(x), dev(w), framed[:, 1:n + 1])
    assert torch.equal(framed[:, 1:n + 1], out16) and (framed[:, 0] == 7).all() and (framed[:, n + 1:] == 7).all()
    if n % 16 == 0:
        act = torch.zeros(m, n // 2, dtype=bf, device="cuda")
        kernels.skinny_tcgen05(dev(x), dev(w), act, epilogue=kernels.EPI_SWIGLU)
        y = out32.cpu().double().view(m, n // 16, 2, 8)
        g, u = y[:, :, 0].reshape(m, n // 2), y[:, :, 1].reshape(m, n // 2)
        torch.testing.assert_close(act.cpu().double(), g / (1 + torch.exp(-g)) * u, rtol=2e-2, atol=2e-2)
    assert kernels.tcgen05_error() == 0


@pytest.mark.parametrize("m, inner, hidden, wide, eps", [(64, 2048, 2048, 3072, 1e-5), (19, 96, 160, 64, 1e-6),
                                                         (128, 8192, 2048, 16384, 1e-5), (40, 64, 5024, 48, 1e-3),
                                                         (77, 320, 3072, 1024, 1e-5)])
def test_skinny_tcgen05_prepares_the_following_norm(m, inner, hidden, wide, eps):
    """The same two halves as decode_linear's, for up to 128 rows: a product that leaves the new residual, the rows
    times the following norm's weights and their sums of squares per tile of 128 features, and the product behind,
    which applies the norm's scale to its 32-bit sums."""
    from tesseract_b200 import kernels

    torch.manual_seed(m + inner + hidden)
    bf = torch.bfloat16
    x = torch.randn(m, inner).to(bf)
    w_first = (torch.randn(hidden, inner) / math.sqrt(inner)).to(bf)
    res = (torch.randn(m, hidden) * 2).to(bf)
    nw = 1 + 0.1 * torch.randn(hidden)
    w_second = (torch.randn(wide, hidden) / math.sqrt(hidden)).to(bf)
    res_out = torch.zeros(m, hidden, dtype=bf, device="cuda")
    rows = torch.zeros(m, hidden, dtype=bf, device="cuda")
    sums = torch.full(kernels.skinny_tcgen05_sums_shape(hidden), float("nan"), device="cuda")
    res_dev = dev(res)
    kernels.skinny_tcgen05(dev(x), dev(w_first), None, prepare=(res_dev, dev(nw), res_out, rows, sums))
    o = (x.double() @ w_first.double().T).to(bf)                       # the product as it would be stored alone
    c = res.double() + o.double()
    close = dict(rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(res_out.cpu().double(), c, **close)
    torch.testing.assert_close(rows.cpu().double(), c * nw.double(), **close)
    assert torch.equal(res_dev.cpu(), res)                                  # the old residual is left alone
    got_sums = sums.cpu().double()[:, :m]
    assert torch.isfinite(got_sums).all()
    torch.testing.assert_close(got_sums.sum(0), (c * c).sum(1), rtol=2e-2, atol=1e-3)
    out = torch.empty(m, wide, dtype=torch.float32, device="cuda")
    kernels.skinny_tcgen05(rows, dev(w_second), out, epilogue=kernels.EPI_F32, scaled_by=sums, eps=eps)
    s = torch.rsqrt(got_sums.sum(0) / hidden + eps)[:, None]
    torch.testing.assert_close(out.cpu().double(), (rows.cpu().double() @ w_second.double().T) * s, rtol=1e-4, atol=1e-4)
    reference = llama.rms_norm(c, nw.double(), eps).to(bf).double() @ w_second.double().T
    torch.testing.assert_close(out.cpu().double(), reference, **close)
    if wide % 16 == 0:
        act = torch.empty(m, wide // 2, dtype=bf, device="cuda")
        kernels.skinny_tcgen05(rows, dev(w_second), act, epilogue=kernels.EPI_SWIGLU, scaled_by=sums, eps=eps)
        y = out.cpu().double().view(m, wide // 16, 2, 8)
        g, u = y[:, :, 0].reshape(m, wide // 2), y[:, :, 1].reshape(m, wide // 2)
        torch.testing.assert_close(act.cpu().double(), g / (1 + torch.exp(-g)) * u, **close)
    with pytest.raises(kernels.KernelError):       # the new residual needs a buffer of its own
        kernels.skinny_tcgen05(dev(x), dev(w_first), None, prepare=(res_dev, dev(nw), res_dev, rows, sums))
    assert kernels.tcgen05_error() == 0
