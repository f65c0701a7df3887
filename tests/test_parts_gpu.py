"""Each part alone: built from a ``PartSpec``, given random weights, run on a hand-made step
context, compared with the plain functions.  Sizes differ from the engine tests'."""

import math

import numpy as np
import pytest
import torch

import plain_gpt2 as plain

pytestmark = pytest.mark.gpu


def f64(t):
    return t.detach().double().cpu().numpy()


def tol(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


def make_ctx(dtype, token_ids, positions, items, plain_only=True):
    from mini_llm_b200.engine.context import StepContext, Workspace
    from mini_llm_b200.kernels.dispatch import Kernels
    ctx = StepContext(Kernels(dtype, plain_only=plain_only), Workspace(torch.device("cuda"), 16), dtype,
                      torch.device("cuda"))
    as_dev = lambda a: torch.tensor(a, dtype=torch.int32, device="cuda")
    ctx.token_ids, ctx.positions, ctx.token_item = as_dev(token_ids), as_dev(positions), as_dev(items)
    ctx.n_tokens = len(token_ids)
    ctx.n_items = max(items) + 1
    return ctx


def bind_random(part, dtype, rng):
    """Random weights for a part: returns {name: float64 array in the FILE's layout}."""
    stored, device = {}, {}
    for w in part.weight_specs():
        values = rng.normal(0, 0.3, size=w.shape) if w.role != "vector" else rng.normal(0.5, 0.5, size=w.shape)
        target = torch.float32 if w.role == "vector" else dtype
        t = torch.tensor(values, device="cuda").to(target)
        stored[w.name] = f64(t)
        device[w.name] = (t.t() if w.transpose else t).contiguous()
    part.bind(device, None)
    return stored


MODES = [(torch.float32, True), (torch.bfloat16, True), (torch.bfloat16, False)]      # (dtype, plain kernels only)


@pytest.mark.parametrize("dtype, plain_only", MODES)
def test_norm_feed_forward_embedding_head(dtype, plain_only):
    from mini_llm_b200.parts import PartSpec, build_part
    rng = np.random.default_rng(0)
    width, inner, vocab, n = 112, 304, 333, 9
    ctx = make_ctx(dtype, rng.integers(0, vocab, n).tolist(), list(range(4, 4 + n)), [0] * n, plain_only)

    emb = build_part(PartSpec("token_embedding", "", {"vocab_size": vocab, "width": width}))
    pos = build_part(PartSpec("learned_positions", "", {"max_positions": 40, "width": width}))
    we, wp = bind_random(emb, dtype, rng), bind_random(pos, dtype, rng)
    hidden = emb.forward(ctx, pos).clone()          # the part's buffer is reused by the next call
    expected = plain.embed(f64(ctx.token_ids).astype(int), we["wte.weight"], wp["wpe.weight"], first_position=4)
    np.testing.assert_allclose(f64(hidden), expected, rtol=0, atol=1e-6)
    np.testing.assert_allclose(f64(emb.forward(ctx, None)), we["wte.weight"][f64(ctx.token_ids).astype(int)], atol=1e-6)

    norm = build_part(PartSpec("layer_norm", "h.3.ln_2", {"width": width, "eps": 1e-3}))
    wn = bind_random(norm, dtype, rng)
    x = norm.forward(ctx, hidden)
    expected_x = plain.layer_norm(expected, wn["h.3.ln_2.weight"], wn["h.3.ln_2.bias"], 1e-3)
    assert x.dtype == dtype
    np.testing.assert_allclose(f64(x), expected_x, rtol=0, atol=tol(dtype))

    for activation, fn in (("gelu_tanh", plain.gelu_tanh), ("gelu_erf", plain.gelu_erf)):
        mlp = build_part(PartSpec("dense_mlp", "h.0.mlp", {"width": width, "inner": inner, "activation": activation}))
        wm = bind_random(mlp, dtype, rng)
        residual = hidden.clone()
        mlp.forward(ctx, x, residual)
        xin = f64(x)
        up = fn(plain.linear(xin, wm["h.0.mlp.c_fc.weight"], wm["h.0.mlp.c_fc.bias"]))
        if dtype == torch.bfloat16:
            up = plain.round_to_bfloat16(up)
        want = f64(hidden) + plain.linear(up, wm["h.0.mlp.c_proj.weight"], wm["h.0.mlp.c_proj.bias"])
        np.testing.assert_allclose(f64(residual), want, rtol=0, atol=tol(dtype) * 4)

    head = build_part(PartSpec("linear_head", "", {"vocab_size": vocab, "width": width, "weight_name": "out.weight"}))
    wh = bind_random(head, dtype, rng)
    logits = head.forward(ctx, x[2:5])
    assert logits.dtype == torch.float32 and logits.shape == (3, vocab)
    np.testing.assert_allclose(f64(logits), f64(x[2:5]) @ wh["out.weight"].T, rtol=0, atol=tol(dtype) * 4)
    # the norm handed over unevaluated, with a gather of rows, as the model's last step does
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device="cuda")
    logits = head.forward(ctx, norm.forward(ctx, hidden, rows=rows, tag="final", defer=True))
    want = expected_x[[8, 0, 3]]
    if dtype == torch.bfloat16:
        want = plain.round_to_bfloat16(want)
    np.testing.assert_allclose(f64(logits), want @ wh["out.weight"].T, rtol=0, atol=tol(dtype) * 4)


@pytest.mark.parametrize("dtype, plain_only", MODES)
@pytest.mark.parametrize("n_heads, n_kv_heads, head, window", [(3, 3, 32, None), (4, 2, 16, None), (2, 2, 48, 5),
                                                              (6, 2, 64, None), (8, 1, 64, 9)])
def test_attention_part_with_its_cache(dtype, plain_only, n_heads, n_kv_heads, head, window):
    """Two requests; the first comes in two steps, so the second step reads keys the first
    stored.  Compared with plain attention over the whole sequences."""
    from mini_llm_b200.cache import CacheManager
    from mini_llm_b200.cache.storage import CacheStorage
    from mini_llm_b200.parts import PartSpec, RunEntry, build_part
    rng = np.random.default_rng(1)
    width = 80
    params = {"width": width, "n_heads": n_heads, "n_kv_heads": n_kv_heads, "head_size": head,
              "score_scale": 0.37, "window": window}
    part = build_part(PartSpec("causal_self_attention", "h.0.attn", params))
    w = bind_random(part, dtype, rng)
    manager = CacheManager([part.cache_need()], page_size=4, n_pages=16, max_requests=2, max_tokens_per_request=32)
    storage = CacheStorage(manager, [RunEntry(0)], dtype, torch.device("cuda"), 2)
    view = storage.views[0]
    lengths = {0: 11, 1: 6}
    xs = {s: torch.tensor(rng.normal(size=(n, width)), device="cuda").to(dtype) for s, n in lengths.items()}
    slots = {s: manager.open() for s in lengths}
    got = {s: [] for s in lengths}
    for step in ([(0, 0, 7)], [(0, 7, 4), (1, 0, 6)]):
        rows, positions, items = [], [], []
        for index, (s, start, n) in enumerate(step):
            assert manager.reserve(slots[s], n)
            rows.append(xs[s][start:start + n])
            positions += list(range(start, start + n))
            items += [index] * n
        ctx = make_ctx(dtype, [0] * len(positions), positions, items, plain_only)
        view.block_table = torch.tensor(np.stack([manager.block_table_row(0, slots[s]) for s, _, _ in step]),
                                        device="cuda")
        x = torch.cat(rows)
        residual = torch.zeros(len(positions), width, device="cuda")
        part.forward(ctx, x, residual, view)
        offset = 0
        for s, start, n in step:
            got[s].append(f64(residual[offset:offset + n]))
            manager.commit(slots[s], n)
            offset += n
    q_width, kv_width = n_heads * head, n_kv_heads * head
    for s in lengths:
        qkv = plain.linear(f64(xs[s]), w["h.0.attn.c_attn.weight"], w["h.0.attn.c_attn.bias"])
        if dtype == torch.bfloat16:
            qkv = plain.round_to_bfloat16(qkv)
        mixed = plain.multi_head_attention(qkv[:, :q_width], qkv[:, q_width:q_width + kv_width],
                                           qkv[:, q_width + kv_width:], n_heads, 0.37, n_kv_heads, window)
        if dtype == torch.bfloat16:
            mixed = plain.round_to_bfloat16(mixed)
        want = plain.linear(mixed, w["h.0.attn.c_proj.weight"], w["h.0.attn.c_proj.bias"])
        np.testing.assert_allclose(np.concatenate(got[s]), want, rtol=0, atol=tol(dtype) * 4)


def test_pre_norm_arrangement_is_the_reference_block():
    from mini_llm_b200.cache import CacheManager
    from mini_llm_b200.cache.storage import CacheStorage
    from mini_llm_b200.parts import PartSpec, RunEntry, build_part, get_arrangement
    rng = np.random.default_rng(2)
    width, heads, inner, n = 48, 3, 100, 13
    config = {"n_embd": width, "n_head": heads, "layer_norm_epsilon": 1e-4, "activation_function": "gelu"}
    specs = {
        "norm_1": PartSpec("layer_norm", "h.0.ln_1", {"width": width, "eps": 1e-4}),
        "mixer": PartSpec("causal_self_attention", "h.0.attn", {"width": width, "n_heads": heads, "head_size": 16,
                                                                "score_scale": 0.25}),
        "norm_2": PartSpec("layer_norm", "h.0.ln_2", {"width": width, "eps": 1e-4}),
        "feed_forward": PartSpec("dense_mlp", "h.0.mlp", {"width": width, "inner": inner, "activation": "gelu_erf"}),
    }
    parts = {role: build_part(s) for role, s in specs.items()}
    tensors = {}
    for part in parts.values():
        tensors.update(bind_random(part, torch.float32, rng))
    manager = CacheManager([parts["mixer"].cache_need()], 8, 4, 1, 32)
    storage = CacheStorage(manager, [RunEntry(0)], torch.float32, torch.device("cuda"), 1)
    slot = manager.open()
    manager.reserve(slot, n)
    storage.views[0].block_table = torch.tensor(manager.block_table_row(0, slot)[None], device="cuda")
    ctx = make_ctx(torch.float32, [0] * n, list(range(n)), [0] * n)
    x = rng.normal(size=(n, width))
    hidden = torch.tensor(x, device="cuda", dtype=torch.float32)
    get_arrangement("pre_norm").run(ctx, parts, hidden, storage.views[0])
    np.testing.assert_allclose(f64(hidden), plain.block(f64(torch.tensor(x, dtype=torch.float32)), tensors, config, 0),
                               rtol=0, atol=1e-4)
