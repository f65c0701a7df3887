"""Each kernel alone against a plain computation of the same operation, at sizes other than
the engine tests' (widths and vocabularies that are no power of two, head sizes from 16 to
256 in steps of 16, groups of heads, rows that do not fill a tile)."""

import math

import numpy as np
import pytest
import torch

import plain_gpt2 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


def dev(array, dtype=None):
    t = torch.as_tensor(np.asarray(array)).cuda()
    return t.to(dtype) if dtype is not None else t


def f64(t):
    return t.detach().double().cpu().numpy()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 200, 1600])
def test_embed(dtype, width):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(width)
    table, ptable = dev(rng.normal(size=(301, width)), dtype), dev(rng.normal(size=(77, width)), dtype)
    ids, pos = rng.integers(0, 301, 29), rng.integers(0, 77, 29)
    out = torch.empty(29, width, device="cuda")
    ops.embed(out, dev(ids, torch.int32), dev(pos, torch.int32), table, ptable)
    np.testing.assert_allclose(f64(out), f64(table)[ids] + f64(ptable)[pos], rtol=0, atol=1e-6)
    ops.embed(out, dev(ids, torch.int32), None, table, None)
    np.testing.assert_array_equal(f64(out), f64(table)[ids])
    ops.add_position_rows(out, dev(pos, torch.int32), ptable)
    np.testing.assert_allclose(f64(out), f64(table)[ids] + f64(ptable)[pos], rtol=0, atol=1e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width, eps", [(80, 1e-5), (768, 1e-6), (1600, 1e-3), (3000, 1e-5)])
def test_layernorm(dtype, width, eps):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(width)
    x = dev(rng.normal(3.0, 5.0, size=(23, width)), torch.float32)       # a large mean: one-pass variance would fail
    gain, shift = dev(rng.uniform(0.5, 1.5, width), torch.float32), dev(rng.normal(0, 0.1, width), torch.float32)
    out = torch.empty(23, width, device="cuda", dtype=dtype)
    ops.layernorm(out, x, gain, shift, eps)
    expected = plain.layer_norm(f64(x), f64(gain), f64(shift), eps)
    np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(dtype, 4))
    rows = [22, 0, 7, 7]
    some = torch.empty(4, width, device="cuda", dtype=dtype)
    ops.layernorm(some, x, gain, shift, eps, dev(rows, torch.int32))
    np.testing.assert_allclose(f64(some), expected[rows], rtol=0, atol=tol(dtype, 4))


# every size with a plain store; the other epilogues at the smaller sizes
LINEAR_PLAIN_CASES = [(m, n, k, e) for m, n, k in [(1, 50, 96), (7, 1000, 160), (65, 129, 33), (130, 768, 3072), (2, 50257, 64)]
                      for e in ("store", "gelu_tanh", "gelu_erf", "add") if e == "store" or n <= 2000]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m, n, k, epilogue", LINEAR_PLAIN_CASES)
def test_linear_plain(dtype, m, n, k, epilogue):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m * n + k)
    a, w = dev(rng.normal(size=(m, k)), dtype), dev(rng.normal(size=(n, k)) / math.sqrt(k), dtype)
    bias = dev(rng.normal(size=n), torch.float32)
    acc = f64(a) @ f64(w).T + f64(bias)
    if epilogue == "add":
        out = dev(rng.normal(size=(m, n)), torch.float32)
        expected = f64(out) + acc
        ops.linear_plain(out, a, w, bias, "add")
    else:
        out = torch.full((m, n), float("nan"), device="cuda", dtype=dtype)
        ops.linear_plain(out, a, w, bias, epilogue)
        expected = {"store": acc, "gelu_tanh": plain.gelu_tanh(acc), "gelu_erf": plain.gelu_erf(acc)}[epilogue]
    out_tol = tol(torch.float32 if epilogue == "add" else dtype, 4)
    np.testing.assert_allclose(f64(out), expected, rtol=0, atol=out_tol)
    # a strided input (a column slice) and no bias
    wide = dev(rng.normal(size=(m, k + 24)), dtype)
    out2 = torch.empty(m, n, device="cuda", dtype=dtype)
    ops.linear_plain(out2, wide[:, 8:8 + k], w, None, "store")
    np.testing.assert_allclose(f64(out2), f64(wide)[:, 8:8 + k] @ f64(w).T, rtol=0, atol=tol(dtype, 4))


def paged_case(rng, lengths, n_new, n_heads, n_kv_heads, head, page, dtype, extra_pages=5):
    """Requests with ``lengths[i]`` cached tokens each, of which the last ``n_new[i]`` are this
    step's; pages handed out in a shuffled order.  Returns device tensors and the dense K, V."""
    width = n_kv_heads * head
    max_blocks = max(-(-l // page) for l in lengths) + 1
    n_pages = sum(-(-l // page) for l in lengths) + extra_pages
    order = rng.permutation(n_pages)
    table = np.full((len(lengths), max_blocks), -1, dtype=np.int32)
    k_pages = np.full((n_pages, page, width), np.nan)
    v_pages = np.full((n_pages, page, width), np.nan)
    dense, positions, items = [], [], []
    used = 0
    for i, (length, new) in enumerate(zip(lengths, n_new)):
        k, v = rng.normal(size=(length, width)), rng.normal(size=(length, width))
        dense.append((k, v))
        for b in range(-(-length // page)):
            table[i, b] = order[used]
            used += 1
        for p in range(length):
            k_pages[table[i, p // page], p % page] = k[p]
            v_pages[table[i, p // page], p % page] = v[p]
        positions.extend(range(length - new, length))
        items.extend([i] * new)
    return (dev(np.nan_to_num(k_pages, nan=1e4), dtype), dev(np.nan_to_num(v_pages, nan=1e4), dtype),
            dev(table), dev(np.array(positions, dtype=np.int32)), dev(np.array(items, dtype=np.int32)), dense)


def attention_expected(q, dense, positions, items, n_heads, n_kv_heads, head, scale, window):
    out = np.zeros_like(q)
    for t, (p, i) in enumerate(zip(positions, items)):
        k, v = dense[i]
        lo = max(0, p - window + 1) if window else 0
        for h in range(n_heads):
            g = h // (n_heads // n_kv_heads)
            s = (k[lo:p + 1, g * head:(g + 1) * head] @ q[t, h * head:(h + 1) * head]) * scale
            w = np.exp(s - s.max())
            out[t, h * head:(h + 1) * head] = (w / w.sum()) @ v[lo:p + 1, g * head:(g + 1) * head]
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_heads, n_kv_heads, head, page, window", [
    (3, 3, 16, 16, 0), (2, 2, 48, 8, 0), (6, 2, 64, 16, 0), (5, 1, 80, 4, 0), (1, 1, 256, 16, 0),
    (4, 2, 32, 8, 21), (2, 2, 64, 16, 16), (25, 25, 64, 16, 0)])
def test_attention_plain_over_pages(dtype, n_heads, n_kv_heads, head, page, window):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(n_heads * head + page)
    lengths, n_new = [37, 1, 300, 64, 17], [37, 1, 1, 9, 2]      # a whole prompt, first token, decode, portions
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, lengths, n_new, n_heads, n_kv_heads, head,
                                                                  page, dtype)
    dense = [(f64(dev(k, dtype)), f64(dev(v, dtype))) for k, v in dense]
    q = dev(rng.normal(size=(len(f64(positions)), n_heads * head)), dtype)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(head)
    ops.attention_plain(out, q, k_pages, v_pages, table, positions, items, n_heads, n_kv_heads, head, page, scale,
                        window)
    expected = attention_expected(f64(q), dense, f64(positions).astype(int), f64(items).astype(int), n_heads,
                                  n_kv_heads, head, scale, window)
    np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(dtype, 2))


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_finds_one_far_key_and_respects_the_windows_edge(dtype):
    """One key among hundreds is made to stand out (query and key scaled), on a page of its
    own far from the query; its value must come through.  With a window that ends one short
    of it, it must vanish."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(5)
    head, page, length = 64, 16, 500
    far = 3 * page + 5                                  # position 53: fourth page
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, [length], [1], 1, 1, head, page, dtype)
    k, v = dense[0]
    q = rng.normal(size=(1, head))
    k[far] = q[0] * 4.0 / math.sqrt(head)               # score (q.k)/sqrt(D) about 4 |q|^2 / D ... far above the rest
    k[far] *= 8.0
    v[far] = 100.0 + np.arange(head)
    block, offset = int(f64(table)[0, far // page]), far % page
    k_pages[block, offset] = dev(k[far], dtype)
    v_pages[block, offset] = dev(v[far], dtype)
    qd = dev(q, dtype)
    out = torch.empty_like(qd)
    scale = 1.0 / math.sqrt(head)
    ops.attention_plain(out, qd, k_pages, v_pages, table, positions, items, 1, 1, head, page, scale, 0)
    np.testing.assert_allclose(f64(out)[0], f64(dev(v[far], dtype)), rtol=2e-2, atol=0.5)
    window = length - 1 - far                           # keys far+1 .. length-1: the far key is just outside
    ops.attention_plain(out, qd, k_pages, v_pages, table, positions, items, 1, 1, head, page, scale, window)
    assert float(out.float().abs().max()) < 10.0
    ops.attention_plain(out, qd, k_pages, v_pages, table, positions, items, 1, 1, head, page, scale, window + 1)
    np.testing.assert_allclose(f64(out)[0], f64(dev(v[far], dtype)), rtol=2e-2, atol=0.5)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kv_store_writes_only_its_own_slots(dtype):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(9)
    page, width, n_pages = 8, 96, 12
    k_pages = torch.full((n_pages, page, width), 7.0, device="cuda", dtype=dtype)
    v_pages = torch.full((n_pages, page, width), 7.0, device="cuda", dtype=dtype)
    table = dev(np.array([[5, 2, -1], [9, 0, 11]], dtype=np.int32))
    positions = dev(np.array([6, 7, 8, 9, 17], dtype=np.int32))          # crosses a page edge
    items = dev(np.array([0, 0, 0, 0, 1], dtype=np.int32))
    src = dev(rng.normal(size=(5, 3 * width)), dtype)                    # keys and values as column slices
    ops.kv_store(k_pages, v_pages, src[:, width:2 * width], src[:, 2 * width:], positions, items, table, page)
    expect_k = torch.full_like(k_pages, 7.0)
    expect_v = torch.full_like(v_pages, 7.0)
    for row, (pg, off) in enumerate([(5, 6), (5, 7), (2, 0), (2, 1), (11, 1)]):
        expect_k[pg, off] = src[row, width:2 * width]
        expect_v[pg, off] = src[row, 2 * width:]
    assert torch.equal(k_pages, expect_k) and torch.equal(v_pages, expect_v)


def test_sampling_greedy_rules():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(3)
    logits = rng.normal(size=(6, 50257)).astype(np.float32)
    logits[1, 777] = logits[1, 40000] = 9.0           # a tie: the first index wins
    logits[2, 50256] = 11.0                           # the last column
    logits[3, 123] = np.nan                           # a NaN beats numbers, the first NaN wins
    logits[3, 4567] = np.nan
    logits[4, 0] = 12.0
    logits[5] = -np.inf
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.sample_rows(out, dev(logits))
    assert out.tolist() == [plain.argmax_first(row) for row in logits]
    assert out.tolist()[1:] == [777, 50256, 123, 0, 0]


@pytest.mark.parametrize("vocab", [1000, 50257])
def test_sampling_temperature_and_nucleus_match_the_plain_sampler(vocab):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(vocab)
    rows = 24
    logits = (rng.normal(size=(rows, vocab)) * 2.0).astype(np.float32)
    temperature = np.array([0.8, 1.0, 0.3, 1.7] * 6, dtype=np.float32)
    top_p = np.array([1.0] * 8 + [0.95] * 8 + [0.5] * 4 + [0.05] * 4, dtype=np.float32)
    seeds = rng.integers(0, 2 ** 63, rows)
    counters = rng.integers(0, 1000, rows).astype(np.int32)
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample_rows(out, dev(logits), dev(temperature), dev(top_p), dev(seeds.astype(np.int64)), dev(counters))
    got = out.tolist()
    near_ties = 0
    for r in range(rows):
        choice, margin = plain.sample(logits[r], float(temperature[r]), float(top_p[r]), int(seeds[r]),
                                      int(counters[r]), return_margin=True)
        if got[r] != choice:
            assert margin < 1e-3, f"row {r}: engine chose {got[r]}, plain {choice} with margin {margin}"
            near_ties += 1
    assert near_ties <= 1
    again = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops.sample_rows(again, dev(logits), dev(temperature), dev(top_p), dev(seeds.astype(np.int64)), dev(counters + 1))
    assert again.tolist() != got                      # another counter, another draw
    # the frequencies of many draws follow the softmax
    few = np.array([[0.0, 1.0, 2.0, -1.0, 0.5]], dtype=np.float32).repeat(4000, axis=0)
    out = torch.empty(4000, dtype=torch.int32, device="cuda")
    ops.sample_rows(out, dev(few), dev(np.ones(4000, dtype=np.float32)), None,
                    dev(np.full(4000, 99, dtype=np.int64)), dev(np.arange(4000, dtype=np.int32)))
    freq = np.bincount(out.cpu().numpy(), minlength=5) / 4000.0
    p = np.exp(few[0]) / np.exp(few[0]).sum()
    assert np.abs(freq - p).max() < 0.03


# ---- kernels for steps of few tokens --------------------------------------------------------

# every row count and size with a plain store; the other epilogues at fewer of them
SKINNY_CASES = [(m, n, k, e) for m in (1, 2, 3, 5, 8, 13, 16, 37, 64)
                for n, k in [(768, 768), (100, 96), (1000, 160), (2304, 768), (777, 3072), (50257, 64)]
                for e in ("store", "gelu_tanh", "gelu_erf", "add")
                if e == "store" or (n <= 3000 and m in (1, 5, 16, 37))]


@pytest.mark.parametrize("m, n, k, epilogue", SKINNY_CASES)
def test_skinny_linear(m, n, k, epilogue):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m * 7 + n + k)
    a, w = dev(rng.normal(size=(m, k + 8)), torch.bfloat16)[:, :k], dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.normal(size=n), torch.float32)
    acc = f64(a) @ f64(w).T + f64(bias)
    if epilogue == "add":
        out = dev(rng.normal(size=(m, n)), torch.float32)
        expected = f64(out) + acc
        ops.skinny_linear(out, a, w, bias, "add")
        np.testing.assert_allclose(f64(out), expected, rtol=0, atol=1e-4)
        return
    expected = {"store": acc, "gelu_tanh": plain.gelu_tanh(acc), "gelu_erf": plain.gelu_erf(acc)}[epilogue]
    out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.skinny_linear(out, a, w, bias, epilogue)
    np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(torch.bfloat16, 4))
    wide = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
    ops.skinny_linear(wide, a, w, None, "store")                       # fp32 output (logits), no bias
    np.testing.assert_allclose(f64(wide), f64(a) @ f64(w).T, rtol=0, atol=1e-4)


@pytest.mark.parametrize("m", [1, 6, 16, 33])
@pytest.mark.parametrize("k, eps", [(96, 1e-6), (768, 1e-5), (1600, 1e-3)])
def test_skinny_linear_with_the_norm_on_the_way_in(m, k, eps):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m + k)
    n = 200
    x = dev(rng.normal(2.0, 3.0, size=(m + 9, k)), torch.float32)
    gain, shift = dev(rng.uniform(0.5, 1.5, k), torch.float32), dev(rng.normal(0, 0.1, k), torch.float32)
    w, bias = dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16), dev(rng.normal(size=n), torch.float32)
    rows = rng.integers(0, m + 9, m)
    normed = plain.round_to_bfloat16(plain.layer_norm(f64(x), f64(gain), f64(shift), eps))
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    ops.skinny_linear(out, x, w, bias, "store", norm=(gain, shift, eps, dev(rows.astype(np.int32))))
    np.testing.assert_allclose(f64(out), normed[rows] @ f64(w).T + f64(bias), rtol=0, atol=tol(torch.bfloat16, 4))
    ops.skinny_linear(out, x[:m], w, bias, "store", norm=(gain, shift, eps, None))
    np.testing.assert_allclose(f64(out), normed[:m] @ f64(w).T + f64(bias), rtol=0, atol=tol(torch.bfloat16, 4))


def test_skinny_linear_scatters_keys_and_values_into_pages():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(4)
    heads, kv_heads, head, page, k = 4, 2, 16, 8, 96
    q_width, kv_width = heads * head, kv_heads * head
    a = dev(rng.normal(size=(5, k)), torch.bfloat16)
    w = dev(rng.normal(size=(q_width + 2 * kv_width, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.normal(size=q_width + 2 * kv_width), torch.float32)
    k_pages = torch.full((12, page, kv_width), 7.0, device="cuda", dtype=torch.bfloat16)
    v_pages = torch.full_like(k_pages, 7.0)
    table = dev(np.array([[5, 2, -1], [9, 0, 11]], dtype=np.int32))
    positions, items = dev(np.array([6, 7, 8, 9, 17], dtype=np.int32)), dev(np.array([0, 0, 0, 0, 1], dtype=np.int32))
    q = torch.empty(5, q_width, device="cuda", dtype=torch.bfloat16)
    ops.skinny_linear(q, a, w, bias, "store", scatter=(k_pages, v_pages, positions, items, table, page, q_width, kv_width))
    full = torch.empty(5, q_width + 2 * kv_width, device="cuda", dtype=torch.bfloat16)
    ops.linear_plain(full, a, w, bias, "store")
    np.testing.assert_allclose(f64(q), f64(full[:, :q_width]), rtol=0, atol=tol(torch.bfloat16))
    expect_k, expect_v = torch.full_like(k_pages, 7.0), torch.full_like(v_pages, 7.0)
    for row, (pg, off) in enumerate([(5, 6), (5, 7), (2, 0), (2, 1), (11, 1)]):
        expect_k[pg, off] = full[row, q_width:q_width + kv_width]
        expect_v[pg, off] = full[row, q_width + kv_width:]
    np.testing.assert_allclose(f64(k_pages), f64(expect_k), rtol=0, atol=tol(torch.bfloat16))
    np.testing.assert_allclose(f64(v_pages), f64(expect_v), rtol=0, atol=tol(torch.bfloat16))


def split_scratch(tokens, heads, max_chunks, head):
    return (torch.full((tokens * heads * max_chunks * head,), float("nan"), device="cuda"),
            torch.full((tokens * heads * max_chunks * 2,), float("nan"), device="cuda"),
            torch.zeros(tokens * heads, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("n_heads, n_kv_heads, head, page, window", [
    (3, 3, 16, 16, 0), (6, 2, 64, 16, 0), (5, 1, 32, 4, 0), (1, 1, 256, 16, 0), (2, 2, 128, 8, 0),
    (4, 2, 32, 8, 21), (2, 2, 64, 16, 16), (25, 25, 64, 16, 0)])
@pytest.mark.parametrize("chunk", [64, 128, 256])
def test_split_attention_over_pages(n_heads, n_kv_heads, head, page, window, chunk):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(n_heads * head + page + chunk)
    lengths, n_new = [37, 1, 300, 64, 17, 129], [37, 1, 1, 9, 2, 1]
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, lengths, n_new, n_heads, n_kv_heads, head,
                                                                  page, torch.bfloat16)
    dense = [(f64(dev(k, torch.bfloat16)), f64(dev(v, torch.bfloat16))) for k, v in dense]
    n = len(f64(positions))
    q = dev(rng.normal(size=(n, n_heads * head)), torch.bfloat16)
    out = torch.full_like(q, float("nan"))
    scale = 1.0 / math.sqrt(head)
    max_chunks = -(-(table.shape[1] * page) // chunk)
    acc, ml, counters = split_scratch(n, n_heads, max_chunks, head)
    expected = attention_expected(f64(q), dense, f64(positions).astype(int), f64(items).astype(int), n_heads,
                                  n_kv_heads, head, scale, window)
    for _ in range(2):                                  # twice on the same scratch: the counters return to zero
        ops.split_attention(out, q, k_pages, v_pages, table, positions, items, n_heads, n_kv_heads, head, page,
                            scale, window, chunk, max_chunks, acc, ml, counters)
        np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(torch.bfloat16, 2))
        assert int(counters.abs().sum()) == 0
        out.fill_(float("nan"))


@pytest.mark.parametrize("n_heads, n_kv_heads, head, page, window", [
    (6, 2, 64, 16, 0), (12, 12, 64, 64, 0), (8, 1, 64, 8, 0), (2, 2, 128, 8, 0), (4, 1, 128, 32, 0),
    (2, 2, 64, 16, 16), (6, 3, 64, 4, 150), (25, 25, 64, 16, 0)])
@pytest.mark.parametrize("chunk", [64, 128, 512])
def test_group_attention_over_pages(n_heads, n_kv_heads, head, page, window, chunk):
    """The mma.sync variant of split_attention: groups of 1 to 8 query heads per key/value
    head, lengths that end inside a tile of 16 keys, twice on the same scratch."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(n_heads * head + page + chunk)
    lengths, n_new = [37, 1, 300, 64, 17, 129, 700], [37, 1, 1, 9, 2, 1, 3]
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, lengths, n_new, n_heads, n_kv_heads, head,
                                                                  page, torch.bfloat16)
    dense = [(f64(dev(k, torch.bfloat16)), f64(dev(v, torch.bfloat16))) for k, v in dense]
    n = len(f64(positions))
    q = dev(rng.normal(size=(n, n_heads * head)), torch.bfloat16)
    out = torch.full_like(q, float("nan"))
    scale = 1.0 / math.sqrt(head)
    max_chunks = -(-(table.shape[1] * page) // chunk)
    acc, ml, counters = split_scratch(n, n_heads, max_chunks, head)
    assert ops.group_attention_takes(q, n_heads, n_kv_heads, head)
    expected = attention_expected(f64(q), dense, f64(positions).astype(int), f64(items).astype(int), n_heads,
                                  n_kv_heads, head, scale, window)
    for _ in range(2):
        ops.group_attention(out, q, k_pages, v_pages, table, positions, items, n_heads, n_kv_heads, head, page,
                            scale, window, chunk, max_chunks, acc, ml, counters)
        np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(torch.bfloat16, 2))
        assert int(counters.abs().sum()) == 0
        out.fill_(float("nan"))


def test_group_attention_finds_one_far_key_and_respects_the_windows_edge():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(5)
    head, page, length, chunk = 64, 16, 500, 64
    far = 3 * page + 5
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, [length], [1], 1, 1, head, page, torch.bfloat16)
    k, v = dense[0]
    q = rng.normal(size=(1, head))
    k[far] = q[0] * 4.0
    v[far] = 100.0 + np.arange(head)
    block, offset = int(f64(table)[0, far // page]), far % page
    k_pages[block, offset] = dev(k[far], torch.bfloat16)
    v_pages[block, offset] = dev(v[far], torch.bfloat16)
    qd = dev(q, torch.bfloat16)
    out = torch.empty_like(qd)
    scale = 1.0 / math.sqrt(head)
    max_chunks = -(-(table.shape[1] * page) // chunk)
    scratch = split_scratch(1, 1, max_chunks, head)
    run = lambda window: ops.group_attention(out, qd, k_pages, v_pages, table, positions, items, 1, 1, head, page,
                                             scale, window, chunk, max_chunks, *scratch)
    run(0)
    np.testing.assert_allclose(f64(out)[0], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)
    run(length - 1 - far)
    assert float(out.float().abs().max()) < 10.0
    run(length - far)
    np.testing.assert_allclose(f64(out)[0], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)


def test_split_attention_finds_one_far_key_and_respects_the_windows_edge():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(5)
    head, page, length, chunk = 64, 16, 500, 64
    far = 3 * page + 5
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, [length], [1], 1, 1, head, page, torch.bfloat16)
    k, v = dense[0]
    q = rng.normal(size=(1, head))
    k[far] = q[0] * 4.0
    v[far] = 100.0 + np.arange(head)
    block, offset = int(f64(table)[0, far // page]), far % page
    k_pages[block, offset] = dev(k[far], torch.bfloat16)
    v_pages[block, offset] = dev(v[far], torch.bfloat16)
    qd = dev(q, torch.bfloat16)
    out = torch.empty_like(qd)
    scale = 1.0 / math.sqrt(head)
    max_chunks = -(-(table.shape[1] * page) // chunk)
    scratch = split_scratch(1, 1, max_chunks, head)
    run = lambda window: ops.split_attention(out, qd, k_pages, v_pages, table, positions, items, 1, 1, head, page,
                                             scale, window, chunk, max_chunks, *scratch)
    run(0)
    np.testing.assert_allclose(f64(out)[0], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)
    run(length - 1 - far)
    assert float(out.float().abs().max()) < 10.0
    run(length - far)
    np.testing.assert_allclose(f64(out)[0], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)


# ---- tensor-core matrix product --------------------------------------------------------------

# every size with a plain store; the other epilogues at six of them
GEMM_CASES = [(m, n, k, e) for m, n, k in [
    (128, 128, 64), (128, 128, 256), (256, 384, 768), (300, 1000, 160), (2048, 768, 768), (1, 256, 64),
    (8, 2304, 768), (17, 777, 96), (40, 768, 3072), (64, 1000, 160), (65, 136, 72), (5, 50257, 64),
    (1024, 3072, 768), (513, 768, 3072)]
    for e in ("store", "gelu_tanh", "gelu_erf", "add", "logits")
    if e == "store" or (m, n, k) in [(128, 128, 256), (300, 1000, 160), (17, 777, 96), (64, 1000, 160),
                                     (513, 768, 3072), (5, 50257, 64)]]


@pytest.mark.parametrize("m, n, k, epilogue", GEMM_CASES)
def test_gemm_tcgen05(m, n, k, epilogue):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m + n + k)
    a, w = dev(rng.normal(size=(m, k)), torch.bfloat16), dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.normal(size=n), torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = f64(a) @ f64(w).T + f64(bias)
    if epilogue == "add":
        out = dev(rng.normal(size=(m, n)), torch.float32)
        expected = f64(out) + acc
        ops.gemm_bf16(out, a, w, bias, "add", status)
        atol = 2e-4
    elif epilogue == "logits":
        out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
        ops.gemm_bf16(out, a, w, None, "store", status)
        expected, atol = f64(a) @ f64(w).T, 2e-4
    else:
        out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
        ops.gemm_bf16(out, a, w, bias, epilogue, status)
        expected = {"store": acc, "gelu_tanh": plain.gelu_tanh(acc), "gelu_erf": plain.gelu_erf(acc)}[epilogue]
        atol = tol(torch.bfloat16, 4)
    assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
    np.testing.assert_allclose(f64(out), expected, rtol=0, atol=atol)


@pytest.mark.parametrize("width", [64, 96, 128, 192, 256, 1064, 1096, 1128, 1192, 1256, 2064, 2096, 2128,
                                   7002, 7003, 7004, 7102, 7103, 7104])
@pytest.mark.parametrize("m, n, k, epilogue", [(300, 1000, 160, "gelu_tanh"), (513, 768, 3072, "add"), (17, 777, 96, "store"),
                                               (2048, 2304, 768, "store"), (4000, 1100, 72, "add"), (129, 50257, 64, "logits"),
                                               (2100, 3072, 256, "gelu_erf")])
def test_gemm_tcgen05_every_tile_width(m, n, k, epilogue, width):
    """The persistent kernel at each of its tile widths, on single CTAs (128 tokens a tile) and
    on pairs of CTAs (1000 + width: 256 tokens a tile, each CTA loading half of the tile's
    block of W), with two issuing threads and two accumulators a tile (2000 + width), and with
    tiles of 256 or 128 features shared along K by clusters of 2 to 4 CTAs (7000 / 7100 + CTAs;
    with one or two blocks of K some CTAs of a cluster have none): tiles that are partly empty in rows and in columns, a pair whose second CTA
    has no rows at all, one tile for some CTAs and a dozen for others (so that both accumulators
    and every phase of the ring are in use), every epilogue; bitwise the same result twice."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m + n + k + width)
    a, w = dev(rng.normal(size=(m, k)), torch.bfloat16), dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.normal(size=n), torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = f64(a) @ f64(w).T
    runs = []
    for _ in range(2):
        if epilogue == "add":
            start = dev(np.random.default_rng(3).normal(size=(m, n)), torch.float32)
            out = start.clone()
            ops.gemm_bf16_tile(out, a, w, bias, "add", status, width)
            expected, atol = f64(start) + acc + f64(bias), 2e-4
        elif epilogue == "logits":
            out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
            ops.gemm_bf16_tile(out, a, w, None, "store", status, width)
            expected, atol = acc, 2e-4
        else:
            out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
            ops.gemm_bf16_tile(out, a, w, bias, epilogue, status, width)
            full = acc + f64(bias)
            expected = {"store": full, "gelu_tanh": plain.gelu_tanh(full), "gelu_erf": plain.gelu_erf(full)}[epilogue]
            atol = tol(torch.bfloat16, 4)
        assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
        np.testing.assert_allclose(f64(out), expected, rtol=0, atol=atol)
        runs.append(f64(out))
    np.testing.assert_array_equal(runs[0], runs[1])


def test_gemm_tcgen05_strided_input_and_twin():
    """A column slice as input (the row stride differs from K), against the plain twin."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(77)
    m, n, k = 200, 520, 192
    wide = dev(rng.normal(size=(m, 3 * k)), torch.bfloat16)
    w = dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = wide[:, k:2 * k]
    assert ops.gemm_takes(a, w) and not ops.gemm_takes(wide[:, 4:4 + k], w)
    fast, slow = torch.empty(m, n, device="cuda", dtype=torch.bfloat16), torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    ops.gemm_bf16(fast, a, w, None, "store", status)
    ops.linear_plain(slow, a, w, None, "store")
    assert int(status.item()) == 0
    np.testing.assert_allclose(f64(fast), f64(slow), rtol=0, atol=tol(torch.bfloat16, 2))


# ---- tensor-core attention for prompt portions -----------------------------------------------

@pytest.mark.parametrize("n_heads, n_kv_heads, head, page, window", [
    (2, 2, 64, 16, 0), (3, 1, 64, 8, 0), (2, 2, 128, 16, 0), (4, 2, 64, 32, 0), (1, 1, 64, 128, 0),
    (2, 1, 128, 64, 0), (2, 2, 64, 16, 100), (2, 2, 64, 8, 128), (2, 2, 128, 16, 300), (12, 12, 64, 16, 0)])
def test_attention_prefill_over_pages(n_heads, n_kv_heads, head, page, window):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(n_heads * head + page + window)
    # whole prompts (one not a multiple of the tile), a portion after 300 cached tokens, single tokens
    lengths, n_new = [300, 500, 1, 128, 641, 77, 260], [300, 200, 1, 128, 129, 1, 4]
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, lengths, n_new, n_heads, n_kv_heads, head,
                                                                  page, torch.bfloat16)
    kv_shape = (k_pages.shape[0], page, n_kv_heads, head)
    dense = [(f64(dev(k, torch.bfloat16)), f64(dev(v, torch.bfloat16))) for k, v in dense]
    n = len(f64(positions))
    q = dev(rng.normal(size=(n, n_heads * head)), torch.bfloat16)
    out = torch.full_like(q, float("nan"))
    offsets = np.concatenate([[0], np.cumsum(n_new)[:-1]]).tolist()
    starts = [l - m for l, m in zip(lengths, n_new)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(head)
    expected = attention_expected(f64(q), dense, f64(positions).astype(int), f64(items).astype(int), n_heads,
                                  n_kv_heads, head, scale, window)
    work = torch.zeros(2, dtype=torch.int32, device="cuda")
    # every tile by one CTA, then the long tiles in parts (twice: the counters must be back at zero)
    whole, n_split, most = ops.attention_tiles(offsets, n_new, starts, split=False)
    assert n_split == 0 and most == 1
    ops.attention_prefill(out, q, k_pages.view(kv_shape), v_pages.view(kv_shape), table,
                          dev(np.array(whole, dtype=np.int32)), len(whole), n_heads, n_kv_heads, head, page, scale,
                          window, status, work)
    np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(torch.bfloat16, 2))
    parts, n_split, most = ops.attention_tiles(offsets, n_new, starts, split=True)
    assert n_split == 2 and most == 2 and len(parts) == len(whole) + 2          # the tiles that end past key 512
    scratch = (torch.full((n_split * n_heads * 8 * 128 * (head + 4),), float("nan"), device="cuda"),
               torch.zeros(n_split * n_heads, dtype=torch.int32, device="cuda"))
    for _ in range(2):
        out.fill_(float("nan"))
        ops.attention_prefill(out, q, k_pages.view(kv_shape), v_pages.view(kv_shape), table,
                              dev(np.array(parts, dtype=np.int32)), len(parts), n_heads, n_kv_heads, head, page, scale,
                              window, status, work, scratch, n_split, 8)
        np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(torch.bfloat16, 2))
    assert int(status.item()) == 0 and int(scratch[1].abs().sum().item()) == 0 and int(work.abs().sum().item()) == 0
    assert [r[7] for r in parts] == sorted((r[7] for r in parts), reverse=True)     # the longest units first


def test_attention_prefill_finds_one_far_key_and_respects_the_windows_edge():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(6)
    head, page, length, new = 64, 16, 700, 150
    far = 3 * page + 5
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, [length], [new], 1, 1, head, page, torch.bfloat16)
    k, v = dense[0]
    q = rng.normal(size=(new, head))
    k[far] = q[-1] * 4.0                                  # stands out for the last query
    v[far] = 100.0 + np.arange(head)
    block, offset = int(f64(table)[0, far // page]), far % page
    k_pages[block, offset] = dev(k[far], torch.bfloat16)
    v_pages[block, offset] = dev(v[far], torch.bfloat16)
    kv_shape = (k_pages.shape[0], page, 1, head)
    qd = dev(q, torch.bfloat16)
    out = torch.empty_like(qd)
    records, n_split, most = ops.attention_tiles([0], [new], [length - new])      # two tiles: split by default
    assert n_split == 2 and most == 2 and len(records) == 4
    tiles = dev(np.array(records, dtype=np.int32))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scratch = (torch.empty(n_split * 8 * 128 * (head + 4), device="cuda"), torch.zeros(n_split, dtype=torch.int32, device="cuda"))
    work = torch.zeros(2, dtype=torch.int32, device="cuda")
    run = lambda window: ops.attention_prefill(out, qd, k_pages.view(kv_shape), v_pages.view(kv_shape), table, tiles,
                                               4, 1, 1, head, page, 1.0 / math.sqrt(head), window, status, work,
                                               scratch, n_split, 8)
    run(0)
    np.testing.assert_allclose(f64(out)[-1], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)
    run(length - 1 - far)
    assert float(out[-1].float().abs().max()) < 10.0
    run(length - far)
    np.testing.assert_allclose(f64(out)[-1], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)
    assert int(status.item()) == 0


@pytest.mark.parametrize("n_heads, n_kv_heads, page, window", [
    (2, 2, 16, 0), (3, 1, 8, 0), (4, 2, 32, 0), (1, 1, 128, 0), (2, 1, 64, 0), (2, 2, 16, 100), (2, 2, 8, 128),
    (2, 2, 64, 300), (12, 12, 64, 0)])
def test_attention_prefill_two_tiles_over_pages(n_heads, n_kv_heads, page, window):
    """Two tiles of queries per CTA, one thread per query row: units of 256 tokens that are
    full, that have a ragged second tile or none, that start deep in a cached context and whose
    first tile ends a block of keys before the second; twice, so that the work counter is back
    at zero; against the plain attention over the same pages."""
    from mini_llm_b200.kernels import ops
    head = 64
    rng = np.random.default_rng(n_heads * head + page + window + 1)
    lengths, n_new = [300, 520, 1, 128, 900, 77, 260, 1000], [300, 257, 1, 128, 385, 1, 4, 256]
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, lengths, n_new, n_heads, n_kv_heads, head,
                                                                  page, torch.bfloat16)
    kv_shape = (k_pages.shape[0], page, n_kv_heads, head)
    dense = [(f64(dev(k, torch.bfloat16)), f64(dev(v, torch.bfloat16))) for k, v in dense]
    n = len(f64(positions))
    q = dev(rng.normal(size=(n, n_heads * head)), torch.bfloat16)
    offsets = np.concatenate([[0], np.cumsum(n_new)[:-1]]).tolist()
    starts = [l - m for l, m in zip(lengths, n_new)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(head)
    expected = attention_expected(f64(q), dense, f64(positions).astype(int), f64(items).astype(int), n_heads,
                                  n_kv_heads, head, scale, window)
    work = torch.zeros(2, dtype=torch.int32, device="cuda")
    # every unit by one CTA (a GPU of few SMs), then the long units in parts (as many SMs as it takes)
    for n_sms in (1, 10 ** 6):
        units, n_split, most = ops.attention_units(offsets, n_new, starts, n_heads, n_sms)
        whole = [u for u in units if u[4] == 0]
        assert sum(u[2] for u in whole) == n and max(u[2] for u in whole) == 256
        assert [u[7] for u in units] == sorted((u[7] for u in units), reverse=True)     # the longest records first
        if n_sms == 1:
            assert (n_split, most) == (0, 1) and max(u[7] for u in units) == 8
        else:
            assert n_split >= 4 and most == 4 and max(u[7] for u in units) == 2
        scratch = None if n_split == 0 else (
            torch.full((n_split * n_heads * most * 256 * (head + 4),), float("nan"), device="cuda"),
            torch.zeros(2 * n_split * n_heads, dtype=torch.int32, device="cuda"))
        for _ in range(2):
            out = torch.full_like(q, float("nan"))
            ops.attention_prefill_two_tiles(out, q, k_pages.view(kv_shape), v_pages.view(kv_shape), table,
                                            dev(np.array(units, dtype=np.int32)), len(units), n_heads, n_kv_heads, head,
                                            page, scale, window, status, work, scratch, n_split, most)
            np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(torch.bfloat16, 2))
        assert int(status.item()) == 0 and int(work.abs().sum().item()) == 0
        assert scratch is None or int(scratch[1].abs().sum().item()) == 0


def test_attention_prefill_two_tiles_finds_one_far_key_and_respects_the_windows_edge():
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(8)
    head, page, length, new = 64, 16, 700, 250
    far = 3 * page + 5
    k_pages, v_pages, table, positions, items, dense = paged_case(rng, [length], [new], 1, 1, head, page, torch.bfloat16)
    k, v = dense[0]
    q = rng.normal(size=(new, head))
    k[far] = q[-1] * 4.0                                  # stands out for the last query (a row of the second tile)
    v[far] = 100.0 + np.arange(head)
    block, offset = int(f64(table)[0, far // page]), far % page
    k_pages[block, offset] = dev(k[far], torch.bfloat16)
    v_pages[block, offset] = dev(v[far], torch.bfloat16)
    kv_shape = (k_pages.shape[0], page, 1, head)
    qd = dev(q, torch.bfloat16)
    out = torch.empty_like(qd)
    units, n_split, most = ops.attention_units([0], [new], [length - new])
    assert len(units) == 3 and (n_split, most) == (1, 3)                # six blocks of keys: three parts of two
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    work = torch.zeros(2, dtype=torch.int32, device="cuda")
    scratch = (torch.empty(3 * 256 * (head + 4), device="cuda"), torch.zeros(2, dtype=torch.int32, device="cuda"))
    run = lambda window: ops.attention_prefill_two_tiles(out, qd, k_pages.view(kv_shape), v_pages.view(kv_shape), table,
                                                         dev(np.array(units, dtype=np.int32)), 3, 1, 1, head, page,
                                                         1.0 / math.sqrt(head), window, status, work, scratch, 1, 3)
    run(0)
    np.testing.assert_allclose(f64(out)[-1], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)
    run(length - 1 - far)
    assert float(out[-1].float().abs().max()) < 10.0
    run(length - far)
    np.testing.assert_allclose(f64(out)[-1], f64(dev(v[far], torch.bfloat16)), rtol=2e-2, atol=0.5)
    assert int(status.item()) == 0


@pytest.mark.parametrize("vocab", [1000, 50257])
def test_sliced_sampling_draws_what_the_one_block_kernel_draws(vocab):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(vocab + 1)
    rows = 20
    logits = (rng.normal(size=(rows, vocab)) * 2.0).astype(np.float32)
    logits[3, 17] = logits[3, vocab - 1] = 30.0                      # a tie across slices: the first index wins
    logits[4, vocab // 2] = np.nan
    temperature = dev(np.array([0.0, 0.8, 1.0, 0.0, 0.0] * 4, dtype=np.float32))
    top_p = dev(np.array([1.0] * 10 + [0.9] * 10, dtype=np.float32))
    seeds, counters = dev(rng.integers(0, 2 ** 63, rows).astype(np.int64)), dev(rng.integers(0, 99, rows).astype(np.int32))
    one, many = torch.empty(rows, dtype=torch.int32, device="cuda"), torch.full((rows,), -7, dtype=torch.int32, device="cuda")
    ops.sample_rows(one, dev(logits), temperature, top_p, seeds, counters)
    scratch = (torch.empty(rows * 32, device="cuda"), torch.empty(rows * 32, dtype=torch.int32, device="cuda"),
               torch.zeros(rows, dtype=torch.int32, device="cuda"))
    for _ in range(2):
        ops.sample_rows_sliced(many, dev(logits), temperature, top_p, seeds, counters, scratch, True)
        assert many.tolist() == one.tolist()
        assert int(scratch[2].sum()) == 0
    assert one.tolist()[3] == 17 and one.tolist()[4] == vocab // 2


@pytest.mark.parametrize("width, eps", [(80, 1e-5), (768, 1e-6), (1600, 1e-3), (4100, 1e-5)])
def test_layernorm_warp(width, eps):
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(width)
    x = dev(rng.normal(3.0, 5.0, size=(37, width)), torch.float32)
    gain, shift = dev(rng.uniform(0.5, 1.5, width), torch.float32), dev(rng.normal(0, 0.1, width), torch.float32)
    out = torch.full((37, width), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.layernorm_warp(out, x, gain, shift, eps)
    expected = plain.layer_norm(f64(x), f64(gain), f64(shift), eps)
    np.testing.assert_allclose(f64(out), expected, rtol=0, atol=tol(torch.bfloat16, 4))
    rows = [36, 0, 7, 7, 20]
    some = torch.empty(5, width, device="cuda", dtype=torch.bfloat16)
    ops.layernorm_warp(some, x, gain, shift, eps, dev(rows, torch.int32))
    np.testing.assert_allclose(f64(some), expected[rows], rtol=0, atol=tol(torch.bfloat16, 4))
    twin = torch.empty_like(out)
    ops.layernorm(twin, x, gain, shift, eps)
    np.testing.assert_allclose(f64(out), f64(twin), rtol=0, atol=tol(torch.bfloat16, 2))


@pytest.mark.parametrize("m, n, k, epilogue", [(64, 768, 3072, "add"), (17, 700, 1536, "add"), (40, 300, 2048, "store"),
                                               (30, 512, 1536, "gelu_tanh"), (25, 130, 4096, "logits"),
                                               (64, 768, 768, "add"), (9, 1000, 256, "store")])
def test_gemm_tcgen05_shared_along_k(m, n, k, epilogue):
    """Few tokens and few tiles: a cluster of CTAs shares each tile along K and adds the partial
    sums through shared memory in a fixed order.  Right, and bit-equal between runs."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m * n + k)
    a, w = dev(rng.normal(size=(m, k)), torch.bfloat16), dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.normal(size=n), torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = f64(a) @ f64(w).T + f64(bias)
    runs = []
    for _ in range(3):
        if epilogue == "add":
            start = dev(np.random.default_rng(5).normal(size=(m, n)), torch.float32)
            out = start.clone()
            ops.gemm_bf16(out, a, w, bias, "add", status)
            expected, atol = f64(start) + acc, 3e-4
        elif epilogue == "logits":
            out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.float32)
            ops.gemm_bf16(out, a, w, None, "store", status)
            expected, atol = f64(a) @ f64(w).T, 3e-4
        else:
            out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
            ops.gemm_bf16(out, a, w, bias, epilogue, status)
            expected = {"store": acc, "gelu_tanh": plain.gelu_tanh(acc)}[epilogue]
            atol = tol(torch.bfloat16, 4)
        np.testing.assert_allclose(f64(out), expected, rtol=0, atol=atol)
        runs.append(f64(out))
    assert int(status.item()) == 0
    np.testing.assert_array_equal(runs[0], runs[1])
    np.testing.assert_array_equal(runs[0], runs[2])


@pytest.mark.parametrize("m, q_width, kv_width, k, page", [(300, 768, 768, 256, 16), (40, 256, 64, 128, 8), (5000, 512, 256, 64, 16),
                                                           (130, 96, 32, 64, 64), (64, 128, 128, 512, 4),
                                                           (17, 64, 32, 96, 16)])
def test_gemm_tcgen05_scatters_keys_and_values_into_the_pages(m, q_width, kv_width, k, page):
    """The fused query/key/value product: queries to their buffer, keys and values straight to
    the cache slots that positions and block tables name; nothing else in the pages changes."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m + k)
    n = q_width + 2 * kv_width
    a, w = dev(rng.normal(size=(m, k)), torch.bfloat16), dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.normal(size=n), torch.float32)
    # three requests with different starts; pages handed out in a shuffled order
    counts = [m // 2, m // 3, m - m // 2 - m // 3]
    starts = [5, 0, 3 * page + 1]
    max_blocks = max(-(-(s + c) // page) for s, c in zip(starts, counts)) + 1
    n_pages = 3 * max_blocks + 2
    order = rng.permutation(n_pages)
    table = np.full((3, max_blocks), -1, dtype=np.int32)
    for item in range(3):
        table[item] = order[item * max_blocks:(item + 1) * max_blocks]
    positions = np.concatenate([np.arange(s, s + c) for s, c in zip(starts, counts)]).astype(np.int32)
    token_item = np.concatenate([np.full(c, i) for i, c in enumerate(counts)]).astype(np.int32)
    k_pages = torch.full((n_pages, page, kv_width), 7.0, device="cuda", dtype=torch.bfloat16)
    v_pages = torch.full((n_pages, page, kv_width), -7.0, device="cuda", dtype=torch.bfloat16)
    q = torch.full((m, q_width), float("nan"), device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.gemm_bf16_qkv(q, a, w, bias, status, k_pages, v_pages, dev(positions, torch.int32), dev(token_item, torch.int32),
                      dev(table, torch.int32), page, q_width, kv_width)
    assert int(status.item()) == 0
    expected = f64(a) @ f64(w).T + f64(bias)
    atol = tol(torch.bfloat16, 4)
    np.testing.assert_allclose(f64(q), expected[:, :q_width], rtol=0, atol=atol)
    want_k, want_v = np.full((n_pages, page, kv_width), 7.0), np.full((n_pages, page, kv_width), -7.0)
    for t in range(m):
        pg = table[token_item[t], positions[t] // page]
        want_k[pg, positions[t] % page] = expected[t, q_width:q_width + kv_width]
        want_v[pg, positions[t] % page] = expected[t, q_width + kv_width:]
    np.testing.assert_allclose(f64(k_pages), want_k, rtol=0, atol=atol)
    np.testing.assert_allclose(f64(v_pages), want_v, rtol=0, atol=atol)


@pytest.mark.parametrize("code", [5128, 5256, 5064])
@pytest.mark.parametrize("m, n, k, epilogue", [(300, 768, 3072, "add"), (513, 777, 2048, "gelu_tanh"), (100, 1000, 96, "store"),
                                               (129, 3072, 768, "add"), (512, 768, 3072, "add")])
def test_gemm_tcgen05_swapped_operands_with_wide_token_tiles(m, n, k, epilogue, code):
    """The kernel with swapped operands (the weights fill the tile's 128 rows) with tiles of 64,
    128 and 256 tokens (code 5000 + tokens), its tiles shared along K by a cluster where the
    tiles are few: the engine takes it for up to 512 tokens when K is long.  Right, the same
    bits twice, and what the library chooses by itself agrees."""
    from mini_llm_b200.kernels import ops
    rng = np.random.default_rng(m + n + k + code)
    a, w = dev(rng.normal(size=(m, k)), torch.bfloat16), dev(rng.normal(size=(n, k)) / math.sqrt(k), torch.bfloat16)
    bias = dev(rng.normal(size=n), torch.float32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    acc = f64(a) @ f64(w).T + f64(bias)
    start = dev(rng.normal(size=(m, n)), torch.float32)
    runs = []
    for forced in (code, code, None):
        if epilogue == "add":
            out = start.clone()
            expected, atol = f64(start) + acc, 2e-4
        else:
            out = torch.full((m, n), float("nan"), device="cuda", dtype=torch.bfloat16)
            expected, atol = {"store": acc, "gelu_tanh": plain.gelu_tanh(acc)}[epilogue], tol(torch.bfloat16, 4)
        if forced is None:
            ops.gemm_bf16(out, a, w, bias, epilogue, status)
        else:
            ops.gemm_bf16_tile(out, a, w, bias, epilogue, status, forced)
        assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
        np.testing.assert_allclose(f64(out), expected, rtol=0, atol=atol)
        runs.append(out)
    assert torch.equal(runs[0], runs[1])


@pytest.mark.parametrize("width", [2064, 2096, 2128, 96, 256, 7002, 7104])
def test_gemm_tcgen05_long_runs_of_tiles(width):
    """Many tiles per CTA and an odd number of blocks along K, thirty launches in a row: with two
    issuing threads each thread's blocks change between even and odd places of the K range from
    tile to tile, and every launch must give the same, right result (a thread that looked at a
    stage's barrier two phases late would take operands that are not there yet)."""
    from mini_llm_b200.kernels import ops
    m, n, k = 6000, 800, 1088                      # 47 x 7..13 tiles on 148 CTAs, 17 blocks of K
    g = torch.Generator(device="cuda").manual_seed(width)
    a = torch.randn(m, k, device="cuda", generator=g).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n, device="cuda", generator=g)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    expected = a.float().double() @ w.float().double().T + bias.double()
    first = None
    for launch in range(30):
        out = torch.zeros(m, n, device="cuda", dtype=torch.float32)
        ops.gemm_bf16_tile(out, a, w, bias, "add", status, width)
        if first is None:
            first = out
            assert float((out.double() - expected).abs().max()) < 2e-4
        else:
            assert torch.equal(out, first), f"launch {launch} differs from the first"
    assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"


def test_gemm_tcgen05_time_stamps():
    """The persistent kernel can note when its first CTA passed seven points (start, set-up,
    first operands, last product of the first tile, accumulator ready, first epilogue done,
    end): the stamps come in that order and span less than a millisecond.  Two counters
    follow: the blocks of K its first issuing thread took (4 blocks for each of its tiles:
    20 tiles over at most 20 CTAs, so one tile) and how many had not arrived at its first look."""
    from mini_llm_b200.kernels import ops
    a = torch.randn(600, 256, device="cuda").bfloat16()
    w = (torch.randn(512, 256, device="cuda") / 16).bfloat16()
    out = torch.empty(600, 512, device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stamps = torch.zeros(9, dtype=torch.int64, device="cuda")
    ops.gemm_bf16_tile(out, a, w, None, "store", status, 128, stamps)
    torch.cuda.synchronize()
    times, (looked, not_there) = stamps.tolist()[:7], stamps.tolist()[7:]
    assert looked == 4 and 0 <= not_there <= looked
    assert int(status.item()) == 0 and all(b >= a for a, b in zip(times, times[1:])) and 0 < times[6] - times[0] < 1_000_000
    np.testing.assert_allclose(f64(out), f64(a) @ f64(w).T, rtol=0, atol=tol(torch.bfloat16, 4))
