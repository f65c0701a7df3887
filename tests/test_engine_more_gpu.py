"""The engine where the benchmark runs it, and from the inside: GPT-2 small's real layer
widths, decode steps of dozens of requests, replayed CUDA graphs of prompt steps, the hooks
that show what the cache and the residual stream hold, poisoned pages, refused and failed
steps, and pins on how many kernels a step launches and which."""

import numpy as np
import pytest

import plain_gpt2 as plain
from engine_helpers import (F32_ATOL, bf16_atol, make_model, plain_logits, random_tokens, run_schedule,
                            schedule_mixed, schedule_portions, schedule_tail_one_by_one, schedule_whole)
from tiny_configs import SMALL_WIDTHS, TINY_A, TINY_D

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder_d(tmp_path_factory):
    # (sharpened as in test_engine_gpu.py, which says why not more)
    return make_model(str(tmp_path_factory.mktemp("more_d")), TINY_D, "varied", 3, sharpen=1.25)


@pytest.fixture(scope="module")
def folder_small(tmp_path_factory):
    # The init this size is stated with (matrices N(0, 0.02), output projections scaled down by
    # sqrt(2 L), seed 0), queries and keys scaled up so that single keys matter.  Gains, shifts
    # and biases that are not 1 and 0 are config D's part: at this width the "varied" recipe
    # makes a badly conditioned model, whose bfloat16 rounding alone (fast or plain kernels
    # alike, measured) reaches the bound that was fixed for these tests.
    return make_model(str(tmp_path_factory.mktemp("small_widths")), SMALL_WIDTHS, "gpt2", 0, sharpen=2.0)


def compare(folder, dtype, got, requests, positions=None):
    for name, tokens in requests.items():
        expected = plain_logits(folder, tokens, bf16_weights=(dtype == "bfloat16"))
        atol = F32_ATOL if dtype == "float32" else bf16_atol(expected)
        rows = range(len(tokens)) if positions is None else positions[name]
        for position in rows:
            assert not np.isnan(got[name][position]).any(), (name, position)
            diff = np.abs(got[name][position] - expected[position]).max()
            assert diff <= atol, f"{dtype} request {name} position {position}: |diff| {diff:.3g} > {atol:.3g}"


# ---- GPT-2 small's real widths -------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_layer_sizes_of_gpt2_small(folder_small, dtype):
    """Width 768, 12 heads of 64, inner size 3072, 50,257 tokens, pages of 64 and of 16: a
    200-token request whole, with its last 32 tokens one by one, and in portions; logits at
    every position against the plain implementation."""
    from mini_llm_b200.engine import Engine
    requests = {"r": random_tokens(77, 200, SMALL_WIDTHS["vocab_size"])}
    for page_size in (64, 16):
        engine = Engine(folder_small, dtype=dtype, page_size=page_size, cache_tokens=1024, max_requests=4)
        for steps in (schedule_whole(requests), schedule_tail_one_by_one(requests),
                      schedule_portions(requests, sizes=(70, 2, 129, 3))):
            got = run_schedule(engine, requests, steps)
            compare(folder_small, dtype, got, requests)
        if dtype == "bfloat16":
            assert engine.fused is not None, engine.fused_reason
            # (the whole-request step of 200 tokens was filled up to 256, the next round shape; a
            # portion longer than a tile goes to the kernel with two tiles per CTA, shorter ones
            # to the kernel with one)
            assert engine.kernels.choices[("attention", 256, 12, 64)] == "attention_two_tiles"
            assert engine.kernels.choices[("attention", 128, 12, 64)] == "attention_tcgen05"
            assert engine.kernels.choices[("qkv", 256, 2304, 768)] == "gemm_tcgen05"
        engine.check_status()
        engine.cache.check()
        del engine


# ---- decode steps of many requests ---------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [64, 16])
def test_decode_steps_of_forty_requests(folder_d, dtype, page_size):
    """Forty live requests, one of them past 600 keys, decoded together for six steps: in
    bfloat16 that is the part-by-part path (more than 16 tokens), its captured graph from the
    third step on, the tensor-core product with swapped operands and split-key attention."""
    from mini_llm_b200.engine import Engine, StepEntry
    vocab, decode_steps = TINY_D["vocab_size"], 6
    rng = np.random.default_rng(40)
    lengths = [int(n) for n in rng.integers(3, 150, 40)]
    lengths[7] = 640
    requests = {f"r{i}": random_tokens(500 + i, n + decode_steps, vocab) for i, n in enumerate(lengths)}
    engine = Engine(folder_d, dtype=dtype, page_size=page_size, cache_tokens=8192, max_requests=40,
                    max_tokens_per_step=4096)
    slots = {name: engine.open_request() for name in requests}
    names = list(requests)
    got = {name: np.full((len(t), vocab), np.nan, dtype=np.float32) for name, t in requests.items()}
    for first in range(0, 40, 10):                                   # the prompts, ten requests a step
        batch = names[first:first + 10]
        logits = engine.step([StepEntry(slots[n], requests[n][:-decode_steps], [len(requests[n]) - decode_steps - 1])
                              for n in batch]).cpu().numpy()
        for row, n in zip(logits, batch):
            got[n][len(requests[n]) - decode_steps - 1] = row
    before = engine.kernels.launches
    for step in range(decode_steps):
        place = {n: len(requests[n]) - decode_steps + step for n in names}
        logits = engine.step([StepEntry(slots[n], [requests[n][place[n]]], [0]) for n in names]).cpu().numpy()
        for row, n in zip(logits, names):
            got[n][place[n]] = row
    engine.check_status()
    positions = {n: range(len(requests[n]) - decode_steps - 1, len(requests[n])) for n in names}
    compare(folder_d, dtype, got, requests, positions)
    if dtype == "bfloat16":
        assert engine.fused is not None and not engine.fused.takes_sizes(40, True)
        assert engine.kernels.choices[("attention", 40, 4, 64)] == "split_attention"
        assert engine.kernels.choices[("qkv", 40, 768, 256)] == "gemm_tcgen05"
        assert any(isinstance(held, tuple) for held in engine._graphs.values()), "no decode step was replayed"
        assert (engine.kernels.launches - before) % decode_steps == 0       # replayed steps count what they hold
    for slot in slots.values():
        engine.close_request(slot)
    engine.cache.check()


@pytest.mark.parametrize("parts", [1, 2, 3, 5, 16])
def test_the_one_kernel_step_with_keys_in_parts(folder_d, parts):
    """In the one-kernel decode step several CTAs may share the keys of a (token, head) pair;
    the one that finishes last merges their states.  With any number of parts (more parts than
    a short request has keys, and more units than CTAs among them) the logits are the plain
    implementation's."""
    from mini_llm_b200.engine import Engine, StepEntry
    vocab = TINY_D["vocab_size"]
    lengths = {"s": 3, "m": 90, "l": 500, "x": 33, "y": 257}
    requests = {n: random_tokens(300 + i, count + 4, vocab) for i, (n, count) in enumerate(lengths.items())}
    engine = Engine(folder_d, dtype="bfloat16", page_size=16, cache_tokens=2048, max_requests=8)
    assert engine.fused is not None, engine.fused_reason
    engine.fused.force_parts = parts
    slots = {n: engine.open_request() for n in requests}
    engine.step([StepEntry(slots[n], t[:-4], []) for n, t in requests.items()])
    got = {n: np.full((len(t), vocab), np.nan, dtype=np.float32) for n, t in requests.items()}
    before = engine.kernels.launches
    for step in range(4):
        logits = engine.step([StepEntry(slots[n], [t[len(t) - 4 + step]], [0]) for n, t in requests.items()]).cpu().numpy()
        for row, (n, t) in zip(logits, requests.items()):
            got[n][len(t) - 4 + step] = row
    assert engine.kernels.launches - before == 4
    engine.check_status()
    compare(folder_d, "bfloat16", got, requests, {n: range(len(t) - 4, len(t)) for n, t in requests.items()})


# ---- captured graphs of prompt steps -------------------------------------------------------------

def test_prompt_steps_replayed_from_a_captured_graph(folder_d):
    """Steps with prompt portions are filled up to round shapes; a round shape runs
    eagerly once, is captured the second time and replayed from then on: eight requests
    of the same length, each whole in a step of its own, then a portion of another length
    beside a decoding request, which falls into the same round shape; every step's logits are
    checked, the replayed ones among them."""
    from mini_llm_b200.engine import Engine, StepEntry
    vocab = TINY_D["vocab_size"]
    engine = Engine(folder_d, dtype="bfloat16", page_size=64, cache_tokens=4096, max_requests=8)
    requests = {f"p{i}": random_tokens(900 + i, 150, vocab) for i in range(8)}
    got = run_schedule(engine, requests, schedule_whole(requests), want_all=False)
    compare(folder_d, "bfloat16", got, requests, {n: [149] for n in requests})
    captured = [held for held in engine._graphs.values() if isinstance(held, tuple)]
    assert len(captured) == 1, "the prompt shape was not captured"
    # a mixed shape: one request decodes while others bring 140 tokens each
    decoding = random_tokens(77, 60, vocab)
    others = {f"q{i}": random_tokens(950 + i, 140, vocab) for i in range(7)}
    slot = engine.open_request()
    engine.step([StepEntry(slot, decoding[:50], [])])
    rows = {}
    for i, (name, tokens) in enumerate(others.items()):
        other = engine.open_request()
        logits = engine.step([StepEntry(slot, [decoding[50 + i]], [0]), StepEntry(other, tokens, [139])]).cpu().numpy()
        rows[name] = logits.copy()
        engine.close_request(other)
    engine.close_request(slot)
    engine.check_status()
    expected_decoding = plain_logits(folder_d, decoding, bf16_weights=True)
    for i, (name, tokens) in enumerate(others.items()):
        expected = plain_logits(folder_d, tokens, bf16_weights=True)
        assert np.abs(rows[name][0] - expected_decoding[50 + i]).max() <= bf16_atol(expected_decoding), (name, "decoding")
        assert np.abs(rows[name][1] - expected[139]).max() <= bf16_atol(expected), (name, "prompt")
    # Both shapes are filled up to the same round shape (192 tokens, 8 entries, 8 wanted rows, 4
    # attention tiles): the mixed steps replayed the graph that the first shape captured.
    captured = [held for held in engine._graphs.values() if isinstance(held, tuple)]
    assert len(captured) == 1 and len(engine._graphs) == 1 and captured[0][1].shape[0] == 8
    engine.cache.check()


# ---- looking inside ------------------------------------------------------------------------------

def test_kernels_launched_as_dependents_give_the_same_logits(folder_d):
    """Kernels are launched so that each may be scheduled, and set itself up, while the one
    before it still runs; it waits for that kernel's end before it touches memory.  With that
    switched off every kernel starts after the last has ended.  Both ways give the same logits
    bit for bit, step by step and from captured graphs: prompts in portions beside decoding
    requests on pages that are used again, and decode steps of forty requests (part by part)."""
    from mini_llm_b200.engine import Engine, StepEntry
    from mini_llm_b200.kernels import ops
    vocab, decode_steps = TINY_D["vocab_size"], 6
    lengths = {"a": 300, "b": 45, "c": 131, "d": 2, "e": 260, "f": 90}
    requests = {n: random_tokens(900 + i, count, vocab) for i, (n, count) in enumerate(lengths.items())}
    prompts = {n: max(1, 2 * len(t) // 3) for n, t in requests.items()}
    many = {f"m{i}": random_tokens(950 + i, 20 + 3 * i + decode_steps, vocab) for i in range(40)}
    results = {}
    try:
        for on in (True, False):
            ops.set_dependent_launch(on)
            engine = Engine(folder_d, dtype="bfloat16", page_size=16, cache_tokens=304 + 272 + 144 + 96, max_requests=4)
            steps = schedule_mixed(requests, prompts, max_live=4, portion_sizes=(66, 2, 140, 5, 31))
            got = run_schedule(engine, requests, steps)
            engine.check_status()
            wide = Engine(folder_d, dtype="bfloat16", page_size=16, cache_tokens=8192, max_requests=40, max_tokens_per_step=4096)
            slots = {name: wide.open_request() for name in many}
            names = list(many)
            for first in range(0, 40, 10):
                wide.step([StepEntry(slots[n], many[n][:-decode_steps], []) for n in names[first:first + 10]])
            rows = []
            for step in range(decode_steps):
                rows.append(wide.step([StepEntry(slots[n], [many[n][len(many[n]) - decode_steps + step]], [0])
                                       for n in names]).cpu().numpy())
            wide.check_status()
            assert wide.step_kinds["replayed"] > 0
            got["forty"] = np.stack(rows)
            results[on] = got
            del engine, wide
    finally:
        ops.set_dependent_launch(True)
    compare(folder_d, "bfloat16", results[True], requests)
    for name in results[True]:
        assert np.array_equal(results[True][name], results[False][name]), name


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_stored_keys_and_values_and_the_residual_stream(folder_d, dtype):
    """What the cache holds for a request that came in portions equals norm + projection of
    the plain implementation, layer by layer (the reference's own check,
    engine/tests/test_gpt2_gpu.c:96-150), and the residual stream after every layer equals
    the plain implementation's."""
    from mini_llm_b200.engine import Engine, StepEntry
    tokens = random_tokens(31, 300, TINY_D["vocab_size"])
    config, tensors = plain.load_model(folder_d, round_matrices_to_bfloat16=(dtype == "bfloat16"))
    records = []
    _, blocks = plain.forward(config, tensors, tokens, return_blocks=True, records=records)
    engine = Engine(folder_d, dtype=dtype, page_size=16, cache_tokens=1024, max_requests=2)
    slot = engine.open_request()
    dumps = []
    for first, count in ((0, 130), (130, 3), (133, 1), (134, 166)):
        engine.step([StepEntry(slot, tokens[first:first + count], [])], dump_hidden=True)
        dumps.append([h.cpu().numpy() for h in engine.hidden_dump])
    tolerance = 1e-4 if dtype == "float32" else 0.03
    for layer in range(config["n_layer"]):
        k, v = engine.read_kv(slot, layer)
        assert k.shape == (300, 4, 64) and v.shape == (300, 4, 64)
        for name, mine in (("k", k), ("v", v)):
            expected = records[layer][name]
            diff = np.abs(mine.float().cpu().numpy().reshape(300, 256) - expected).max()
            assert diff <= tolerance * max(1.0, np.abs(expected).max()), (layer, name, diff)
    part, _ = engine.read_kv(slot, 1, first=129, count=5)
    whole, _ = engine.read_kv(slot, 1)
    assert (part == whole[129:134]).all()
    with pytest.raises(ValueError):
        engine.read_kv(slot, 0, first=299, count=2)
    for entry in range(config["n_layer"] + 1):
        mine = np.concatenate([d[entry] for d in dumps])
        scale = max(1.0, float(np.abs(blocks[entry]).max()))
        assert np.abs(mine - blocks[entry]).max() <= tolerance * scale, entry
    engine.close_request(slot)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_poisoned_pages(folder_d, dtype):
    """With ``debug_poison`` every slot of the cache that holds no live token holds a value
    that ruins whatever reads it.  A mixed schedule on so few pages that they are used again
    still gives the plain implementation's logits: nothing reads past a request's length or
    through a block-table row that is not its own."""
    from mini_llm_b200.engine import Engine
    vocab = TINY_D["vocab_size"]
    lengths = {"a": 300, "b": 45, "c": 131, "d": 2, "e": 260, "f": 90}
    requests = {n: random_tokens(700 + i, count, vocab) for i, (n, count) in enumerate(lengths.items())}
    prompts = {n: max(1, 2 * len(t) // 3) for n, t in requests.items()}
    engine = Engine(folder_d, dtype=dtype, page_size=16, cache_tokens=304 + 272 + 144 + 96, max_requests=4,
                    debug_poison=True)
    pool = engine.storage.keys[0][:, :-1]            # (the page past the pool's last is the fillers', no request's)
    assert (torch_isnan(pool).all() if dtype == "float32" else (pool == 1e30).all())
    for order in (list(requests), list(reversed(list(requests)))):
        ordered = {n: requests[n] for n in order}
        steps = schedule_mixed(ordered, prompts, max_live=4, portion_sizes=(66, 2, 140, 5, 31))
        got = run_schedule(engine, ordered, steps)
        compare(folder_d, dtype, got, ordered)
    assert engine.cache.groups[0].pool.reused > 0 and engine.cache.pages_in_use() == [0]
    # every page went back: all of the pool is poison again
    assert (torch_isnan(pool).all() if dtype == "float32" else (pool == 1e30).all())
    engine.cache.check()


def torch_isnan(tensor):
    import torch
    return torch.isnan(tensor)


# ---- steps that are refused or fail --------------------------------------------------------------

def test_a_step_over_the_token_limit_is_refused_and_a_failed_step_changes_nothing(folder_d):
    from mini_llm_b200.engine import Engine, StepEntry, StepError
    vocab = TINY_D["vocab_size"]
    engine = Engine(folder_d, dtype="float32", page_size=16, cache_tokens=1024, max_requests=4, max_tokens_per_step=96)
    a, b = engine.open_request(), engine.open_request()
    tokens = random_tokens(8, 120, vocab)
    with pytest.raises(StepError, match="more than the 96"):
        engine.step([StepEntry(a, tokens[:60], []), StepEntry(b, tokens[:37], [])])
    engine.step([StepEntry(a, tokens[:60], [])])
    assert engine.cache.pages_in_use() == [4]
    # a kernel launcher that raises in the middle of the step: pages reserved for it go back,
    # the lengths stay, and the same tokens can be run again
    real_forward = engine.model.forward

    def failing_forward(ctx, views):
        raise RuntimeError("injected")

    engine.model.forward = failing_forward
    with pytest.raises(RuntimeError, match="injected"):
        engine.step([StepEntry(a, tokens[60:100], [39]), StepEntry(b, tokens[:33], [])])
    engine.model.forward = real_forward
    assert engine.cached_tokens(a) == 60 and engine.cached_tokens(b) == 0
    assert engine.cache.pages_in_use() == [4]
    engine.cache.check()
    got = engine.step([StepEntry(a, tokens[60:100], [39]), StepEntry(b, tokens[:33], [32])]).cpu().numpy()
    expected = plain_logits(folder_d, tokens)
    assert np.abs(got[0] - expected[99]).max() <= F32_ATOL and np.abs(got[1] - expected[32]).max() <= F32_ATOL
    engine.close_request(a)
    engine.close_request(b)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_place_may_be_wanted_twice(folder_d, dtype):
    from mini_llm_b200.engine import Engine, StepEntry
    tokens = random_tokens(9, 21, TINY_D["vocab_size"])
    engine = Engine(folder_d, dtype=dtype, page_size=16, cache_tokens=256, max_requests=2)
    slot = engine.open_request()
    engine.step([StepEntry(slot, tokens[:19], [])])
    got = engine.step([StepEntry(slot, tokens[19:20], [0, 0, 0])]).cpu().numpy()        # more wanted rows than tokens
    more = engine.step([StepEntry(slot, tokens[20:], [0, 0])]).cpu().numpy()
    expected = plain_logits(folder_d, tokens, bf16_weights=(dtype == "bfloat16"))
    atol = F32_ATOL if dtype == "float32" else bf16_atol(expected)
    assert got.shape == (3, TINY_D["vocab_size"]) and (got[0] == got[1]).all() and (got[0] == got[2]).all()
    assert np.abs(got[0] - expected[19]).max() <= atol and np.abs(more[1] - expected[20]).max() <= atol
    engine.close_request(slot)


def test_a_barrier_wait_that_runs_out_is_reported_and_the_next_step_is_right(folder_d):
    """The one-kernel decode step bounds every wait at its grid barrier.  Here one CTA stays
    away from the first barrier (a test switch of the kernel) and the limit is 2 ms: the
    kernel returns with a status code, ``sampled_tokens`` raises instead of handing out
    tokens, the engine puts its counters back, and the following steps equal the part-by-part
    path's."""
    from mini_llm_b200.engine import Engine, SamplingParams, StepEntry
    from mini_llm_b200.kernels.lib import KernelError
    vocab = TINY_D["vocab_size"]
    fused = Engine(folder_d, dtype="bfloat16", page_size=16, cache_tokens=2048, max_requests=8)
    parts = Engine(folder_d, dtype="bfloat16", page_size=16, cache_tokens=2048, max_requests=8, fused_decode=False)
    assert fused.fused is not None, fused.fused_reason
    prompts = [random_tokens(60 + i, n, vocab) for i, n in enumerate((70, 3, 130))]
    greedy = [SamplingParams(0.0, 1.0, 0, 0)] * 3

    def start(engine):
        slots = [engine.open_request() for _ in prompts]
        engine.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
        return slots

    slots = start(fused)
    fused.step([StepEntry(s, [5 + i], [0]) for i, s in enumerate(slots)], greedy)
    assert len(fused.sampled_tokens()) == 3
    fused.fused.barrier_limit_ns, fused.fused.skip_arrival = 2_000_000, True
    fused.step([StepEntry(s, [9 + i], [0]) for i, s in enumerate(slots)], greedy)
    with pytest.raises(KernelError, match="bounded wait"):
        fused.sampled_tokens()
    fused.fused.barrier_limit_ns, fused.fused.skip_arrival = 0, False
    for s in slots:                                    # what a scheduler does with the requests of a failed step
        fused.close_request(s)
    fused.cache.check()
    slots, reference = start(fused), start(parts)
    for step in range(4):
        feed = [11 + 3 * step + i for i in range(3)]
        a = fused.step([StepEntry(s, [t], [0]) for s, t in zip(slots, feed)], greedy).cpu().numpy()
        b = parts.step([StepEntry(s, [t], [0]) for s, t in zip(reference, feed)], greedy).cpu().numpy()
        np.testing.assert_allclose(a, b, rtol=0, atol=bf16_atol(b))
        assert len(fused.sampled_tokens()) == 3
    assert fused.fused is not None
    fused.check_status()


# ---- how many kernels, and which -----------------------------------------------------------------

def test_launch_counts_and_kernel_choices(folder_d):
    """Pins of the kind the reference keeps on its launch counter
    (engine/tests/test_gpt2_gpu_batch.c:170-194: 88 launches whatever the batch): a decode
    step of up to 16 requests is ONE launch, sampling included; a prompt step is 7 per layer
    + 2; a decode step of more requests is 7 per layer + 3; and which kernel each product
    and each attention went to."""
    from mini_llm_b200.engine import Engine, SamplingParams, StepEntry
    vocab, layers = TINY_D["vocab_size"], TINY_D["n_layer"]
    engine = Engine(folder_d, dtype="bfloat16", page_size=64, cache_tokens=8192, max_requests=24, cuda_graphs=False)
    kernels = engine.kernels
    slots = [engine.open_request() for _ in range(20)]
    before = kernels.launches
    engine.step([StepEntry(slots[0], random_tokens(1, 300, vocab), [299])])
    # embed; per layer norm, qkv, attention, proj, norm, fc, down; the head with the final norm on its way in
    assert kernels.launches - before == 7 * layers + 2
    assert kernels.choices[("qkv", 300, 768, 256)] == "gemm_tcgen05"
    assert kernels.choices[("attention", 300, 4, 64)] == "attention_two_tiles"        # one long portion: units of 256 tokens
    assert kernels.choices[("linear", 300, 1024, 256)] == "gemm_tcgen05"
    assert kernels.choices[("linear", 1, 1031, 256)] == "skinny_linear"     # the head on the one wanted row
    engine.step([StepEntry(s, random_tokens(2 + i, 10 + i, vocab), []) for i, s in enumerate(slots[1:], 1)])
    assert kernels.choices[("attention", 380, 4, 64)] == "attention_tcgen05"          # nineteen short portions: tiles
    for count in (1, 8, 16):
        before = kernels.launches
        engine.step([StepEntry(s, [7], [0]) for s in slots[:count]], [SamplingParams(0.0, 1.0, 0, 0)] * count)
        assert kernels.launches - before == 1, count            # the whole step, sampling included
    before = kernels.launches
    engine.step([StepEntry(s, [8], [0]) for s in slots])
    # 20 rows: the norms run on their own (2 per layer + 1), then qkv, attention, proj, fc, down, embed, head
    assert kernels.launches - before == 7 * layers + 3
    assert kernels.choices[("attention", 20, 4, 64)] == "split_attention"
    assert kernels.choices[("qkv", 20, 768, 256)] == "gemm_tcgen05"
    # the 32-bit path never leaves the plain kernels
    plain_engine = Engine(folder_d, dtype="float32", page_size=64, cache_tokens=1024, max_requests=2)
    slot = plain_engine.open_request()
    plain_engine.step([StepEntry(slot, random_tokens(1, 200, vocab), [199])])
    plain_engine.step([StepEntry(slot, [3], [0])])
    assert set(plain_engine.kernels.choices.values()) == {"linear_plain", "attention_plain"}
    assert plain_engine.fused is None and "bfloat16" in plain_engine.fused_reason
    engine.check_status()


def test_tiny_a_from_the_stated_seed(tmp_path):
    """The first tiny configuration exactly as the target states it: weights of the "gpt2"
    recipe from seed 0 (matrices N(0, 0.02), output projections N(0, 0.02 / sqrt(2 L)), biases
    0, gains 1, shifts 0), prompts of 5, 17 and 33 tokens, 8 greedy tokens each, pages of 16:
    logits at every position in 32-bit, and the greedy tokens."""
    from mini_llm_b200.engine import Engine
    from mini_llm_b200.generate import generate
    folder = make_model(str(tmp_path / "a0"), TINY_A, "gpt2", 0)
    prompts = [random_tokens(i, n, 512) for i, n in enumerate((5, 17, 33))]
    got = generate(folder, prompts, max_new_tokens=8, temperature=0.0, dtype="float32", page_size=16)
    config, tensors = plain.load_model(folder)
    for prompt, tokens in zip(prompts, got):
        expected, margins = plain.generate(config, tensors, prompt, 8)
        for i, (mine, theirs) in enumerate(zip(tokens, expected)):
            if mine != theirs:
                assert margins[i] < 1e-4, (prompt, tokens, expected)     # the unsharpened model's logits lie close
                break
    engine = Engine(folder, dtype="float32", page_size=16, cache_tokens=256, max_requests=4)
    requests = {f"p{i}": p + t for i, (p, t) in enumerate(zip(prompts, got))}
    for steps in (schedule_whole(requests), schedule_tail_one_by_one(requests, tail=8)):
        out = run_schedule(engine, requests, steps)
        compare(folder, "float32", out, requests)
