"""The engine against the plain implementation, in 32-bit and in bfloat16, under every way
of cutting the same requests into steps."""

import json
import os
import subprocess
import sys
import zlib

import numpy as np
import pytest

from engine_helpers import (F32_ATOL, bf16_atol, make_model, plain_logits, random_tokens, run_schedule,
                            schedule_mixed, schedule_portions, schedule_tail_one_by_one, schedule_whole)
from tiny_configs import RECIPES, SMALL_WIDTHS, TINY_A, TINY_B, TINY_C, TINY_D

pytestmark = pytest.mark.gpu

CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "D16": TINY_D}
# D runs with pages of 64 tokens (the engine's default and the benchmark's) and again with pages of 16
PAGE_SIZES = {"A": 16, "B": 8, "C": 16, "D": 64, "D16": 16}
# factor on the query and key weights that brings the scores' spread to about 1 (see
# engine_helpers.sharpen_attention); it depends on the recipe's weight scale and the width
# (D: at 1.5 the bfloat16 path's worst error over the schedules below lies at 0.95 to 1.02 of
# the bound for every seed of the weights, from the rounding of activations alone, so that the
# order of a sum decides whether a test passes; at 1.25 it lies at 0.7)
SHARPEN = {"A": 6.0, "B": 2.0, "C": 2.0, "D": 1.25}
# request lengths per configuration (within n_positions); prompts for the mixed schedule
LENGTHS = {"A": {"a": 5, "b": 17, "c": 33, "d": 70, "e": 128},
           "B": {"a": 1, "b": 9, "c": 24, "d": 40, "e": 64, "f": 57},
           "C": {"a": 300, "b": 45, "c": 131, "d": 2, "e": 640},
           "D": {"a": 700, "b": 45, "c": 131, "d": 2, "e": 260}}
LENGTHS["D16"] = LENGTHS["D"]
ALL_KEYS = ["A", "B", "C", "D", "D16"]


@pytest.fixture(scope="session")
def folders(tmp_path_factory):
    out = {}
    for key, raw in CONFIGS.items():
        if key == "D16":
            continue
        recipe, seed = RECIPES[key]
        out[key] = make_model(str(tmp_path_factory.mktemp(f"tiny_{key}")), raw, recipe, seed, sharpen=SHARPEN[key])
    out["D16"] = out["D"]
    return out


def requests_of(key):
    vocab = CONFIGS[key]["vocab_size"]
    key = "D" if key == "D16" else key
    return {name: random_tokens(zlib.crc32(f"{key}/{name}".encode()) % 1000 + i, n, vocab)
            for i, (name, n) in enumerate(LENGTHS[key].items())}


_engines = {}


def engine_of(folders, key, dtype, cache_tokens=None, **kw):
    from mini_llm_b200.engine import Engine
    handle = (key, dtype, cache_tokens, tuple(sorted(kw.items())))
    if handle not in _engines:
        _engines[handle] = Engine(folders[key], dtype=dtype, page_size=PAGE_SIZES[key],
                                  cache_tokens=cache_tokens or 4096, max_requests=8, **kw)
    return _engines[handle]


def check(key, folders, dtype, got, requests):
    worst = 0.0
    for name, tokens in requests.items():
        expected = plain_logits(folders[key], tokens, bf16_weights=(dtype == "bfloat16"))
        assert not np.isnan(got[name]).any(), f"request {name}: logits missing"
        atol = F32_ATOL if dtype == "float32" else bf16_atol(expected)
        diff = np.abs(got[name] - expected).max(axis=1)
        first_bad = np.flatnonzero(diff > atol)
        assert first_bad.size == 0, (f"config {key} {dtype} request {name} (len {len(tokens)}): first wrong position "
                                     f"{first_bad[0]}, |diff| {diff[first_bad[0]]:.3g} > {atol:.3g}")
        worst = max(worst, float(diff.max()) / atol)
    return worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ALL_KEYS)
@pytest.mark.parametrize("cut", ["whole", "tail", "portions"])
def test_each_request_alone(folders, key, dtype, cut):
    requests = requests_of(key)
    steps = {"whole": schedule_whole, "tail": schedule_tail_one_by_one, "portions": schedule_portions}[cut](requests)
    engine = engine_of(folders, key, dtype)
    got = run_schedule(engine, requests, steps)
    check(key, folders, dtype, got, requests)
    assert engine.cache.pages_in_use() == [0]
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["D", "D16"])
def test_portions_of_more_than_a_tile(folders, key, dtype):
    """Portions longer than the 64 tokens up to which a step goes to the decode kernels, and
    longer than one tile of 128 queries, beside portions of two and three tokens: the
    tensor-core products and the tensor-core prompt attention start in the middle of a
    request, of a page and of a block of 128 keys."""
    requests = requests_of(key)
    engine = engine_of(folders, key, dtype)
    got = run_schedule(engine, requests, schedule_portions(requests, sizes=(130, 2, 257, 65, 3)))
    check(key, folders, dtype, got, requests)
    if dtype == "bfloat16":
        assert "attention_tcgen05" in engine.kernels.choices.values()
        assert "gemm_tcgen05" in engine.kernels.choices.values()
    engine.cache.check()


# sizes of prompt portions in the mixed schedule: for D some are longer than a tile of 128 queries
MIXED_PORTIONS = {"D": (130, 3, 70, 9, 257), "D16": (66, 2, 200, 5, 129)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ALL_KEYS)
def test_mixed_batches_with_reused_pages(folders, key, dtype):
    requests = requests_of(key)
    longest = sorted(len(t) for t in requests.values())
    # room for the four longest together, rounded up to pages: later requests must reuse pages
    page = PAGE_SIZES[key]
    cache_tokens = sum(-(-n // page) * page for n in longest[-4:])
    prompts = {name: max(1, (2 * len(t)) // 3) for name, t in requests.items()}
    engine = engine_of(folders, key, dtype, cache_tokens=cache_tokens)
    before = engine.cache.groups[0].pool.reused
    # twice over, in two orders: the second pass runs entirely on used pages
    for order in (list(requests), list(reversed(list(requests)))):
        ordered = {n: requests[n] for n in order}
        steps = schedule_mixed(ordered, prompts, max_live=4, portion_sizes=MIXED_PORTIONS.get(key, (7, 3, 2, 9, 5)))
        assert max(len(s) for s in steps) == min(4, len(requests))
        assert any(len({n for _, n in s}) > 1 and min(n for _, n in s) == 1 for s in steps), "no mixed step"
        got = run_schedule(engine, ordered, steps)
        check(key, folders, dtype, got, ordered)
    assert engine.cache.groups[0].pool.reused > before
    assert engine.cache.pages_in_use() == [0]
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(folders, dtype):
    key = "C"
    tokens = random_tokens(11, 400, CONFIGS[key]["vocab_size"])
    requests = {"long": tokens}
    steps = [[("long", 3)]] + [[("long", 1)]] * 397
    got = run_schedule(engine_of(folders, key, dtype), requests, steps)
    check(key, folders, dtype, got, requests)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["A", "B"])
def test_first_tokens_of_a_sequence(folders, key, dtype):
    vocab = CONFIGS[key]["vocab_size"]
    requests = {"one": random_tokens(1, 1, vocab), "two": random_tokens(2, 2, vocab), "three": random_tokens(3, 3, vocab)}
    engine = engine_of(folders, key, dtype)
    check(key, folders, dtype, run_schedule(engine, requests, schedule_whole(requests)), requests)
    check(key, folders, dtype, run_schedule(engine, requests, [[("one", 1), ("two", 1), ("three", 1)],
                                                               [("two", 1), ("three", 1)], [("three", 1)]]), requests)


def test_cuts_agree_with_each_other_closely(folders):
    """Beyond the comparison with the plain implementation: on the 32-bit path, two ways of
    cutting differ by rounding only."""
    key = "B"
    requests = requests_of(key)
    engine = engine_of(folders, key, "float32")
    whole = run_schedule(engine, requests, schedule_whole(requests))
    parts = run_schedule(engine, requests, schedule_portions(requests))
    for name in requests:
        np.testing.assert_allclose(parts[name], whole[name], rtol=0, atol=2e-5)


def test_refused_steps_change_nothing(folders):
    from mini_llm_b200.engine import OutOfPages, StepEntry, StepError
    engine = engine_of(folders, "A", "float32", cache_tokens=64)
    slot = engine.open_request()
    other = engine.open_request()
    for bad in ([StepEntry(slot, [], [])], [StepEntry(slot, [512], [0])], [StepEntry(slot, [-1], [0])],
                [StepEntry(slot, [1, 2], [2])], [StepEntry(slot, [1], []), StepEntry(slot, [2], [])],
                [StepEntry(99, [1], [0])], [StepEntry(slot, [1] * 129, [])], []):
        with pytest.raises(StepError):
            engine.step(bad)
    with pytest.raises(OutOfPages):
        engine.step([StepEntry(slot, [1] * 40, [39]), StepEntry(other, [2] * 40, [39])])
    assert engine.cached_tokens(slot) == 0 and engine.cache.pages_in_use() == [0]
    tokens = random_tokens(5, 40, 512)
    got = engine.step([StepEntry(slot, tokens, [39])]).cpu().numpy()
    np.testing.assert_allclose(got[0], plain_logits(folders["A"], tokens)[-1], rtol=0, atol=F32_ATOL)
    engine.close_request(slot)
    engine.close_request(other)
    engine.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(folders, tmp_path, dtype):
    """bin/trace_run as a user runs it: a subprocess, steps on standard input."""
    key = "B"
    requests = {"p": random_tokens(21, 50, 1000), "q": random_tokens(22, 37, 1000), "r": random_tokens(23, 64, 1000)}
    lines, expected_files = [], {}
    progress = {n: 0 for n in requests}
    plan = [[("p", 20)], [("p", 2), ("q", 30)], [("p", 1), ("q", 1)], [("p", 27), ("q", 6)], [("r", 64)]]
    for step, batch in enumerate(plan):
        entries, places, end = [], [], []
        for name, n in batch:
            start = progress[name]
            want = [n - 1] if step != 3 else list(range(n))
            entries.append({"id": name, "tokens": requests[name][start:start + n], "want": want})
            places.extend((name, start + w) for w in want)
            progress[name] += n
            if progress[name] == len(requests[name]):
                end.append(name)
        lines.append(json.dumps({"step": step, "entries": entries, "end": end}))
        expected_files[step] = places
    lines.insert(3, json.dumps({"step": 77, "entries": [{"id": "p", "tokens": [], "want": []}][:0], "end": []}))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    # 128 tokens: p (50 -> 64) and q (37 -> 64) live together; r (64) afterwards on their pages
    done = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders[key], "--dtype", dtype,
                           "--out", str(out), "--max-tokens", "128", "--page-size", "8"],
                          input="\n".join(lines) + "\n", capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2", "done 77",
                                                                          "done 3", "done 4"]
    for step, places in expected_files.items():
        got = np.fromfile(out / f"{step}.f32", dtype="<f4").reshape(len(places), 1000)
        for row, (name, position) in zip(got, places):
            expected = plain_logits(folders[key], requests[name], bf16_weights=(dtype == "bfloat16"))
            atol = F32_ATOL if dtype == "float32" else bf16_atol(expected)
            assert np.abs(row - expected[position]).max() <= atol, (step, name, position)
    assert not (out / "77.f32").exists()


def test_fused_decode_step_agrees_with_the_part_by_part_path(folders):
    """Steps of up to 16 single tokens of a plain pre-norm stack run as one persistent kernel.
    It must be in use for such a model, give the part-by-part path's logits (bfloat16
    rounding apart), and leave every other step to the generic path."""
    from mini_llm_b200.engine import Engine, SamplingParams, StepEntry
    key = "C"                                            # head size 32: the fused kernel takes it
    vocab = CONFIGS[key]["vocab_size"]
    fused = Engine(folders[key], dtype="bfloat16", page_size=16, cache_tokens=4096, max_requests=8)
    plain = Engine(folders[key], dtype="bfloat16", page_size=16, cache_tokens=4096, max_requests=8, fused_decode=False)
    assert fused.fused is not None and plain.fused is None
    prompts = [random_tokens(40 + i, n, vocab) for i, n in enumerate((70, 3, 130, 17, 33))]
    feed = np.random.default_rng(7).integers(0, vocab, (40, len(prompts)))
    logits = {}
    for name, engine in (("fused", fused), ("plain", plain)):
        slots = [engine.open_request() for _ in prompts]
        engine.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
        rows = []
        for step in range(40):
            out = engine.step([StepEntry(s, [int(feed[step, i])], [0]) for i, s in enumerate(slots)],
                              [SamplingParams(0.7, 1.0, 11 + i, step) for i in range(len(slots))])
            rows.append((out.cpu().numpy().copy(), engine.sampled_tokens()))
        engine.check_status()
        logits[name] = rows
        assert (engine.fused is not None) == (name == "fused")
    launches_fused, launches_plain = fused.kernels.launches, plain.kernels.launches
    assert launches_fused < launches_plain / 3          # one kernel per step instead of dozens
    agree = 0
    for (a, ta), (b, tb) in zip(logits["fused"], logits["plain"]):
        np.testing.assert_allclose(a, b, rtol=0, atol=bf16_atol(b))
        agree += sum(x == y for x, y in zip(ta, tb))
    assert agree >= 0.97 * 40 * len(prompts)             # the same draws, near-ties apart
    # one long request: few (token, head) pairs, so several CTAs share each pair's keys
    long_prompt = random_tokens(77, 600, vocab)
    rows = {}
    for name, engine in (("fused", fused), ("plain", plain)):
        slot = engine.open_request()
        engine.step([StepEntry(slot, long_prompt, [])])
        rows[name] = [engine.step([StepEntry(slot, [int(feed[step, 0])], [0])]).cpu().numpy().copy() for step in range(12)]
        engine.close_request(slot)
    class _One:
        n_tokens, item_starts = 1, [600]
    assert fused.fused.attention_parts(_One) >= 4
    for a, b in zip(rows["fused"], rows["plain"]):
        np.testing.assert_allclose(a, b, rtol=0, atol=bf16_atol(b))
    fused.check_status()
    # a model the fused kernel does not take (head size 48) runs the generic path silently
    other = Engine(folders["B"], dtype="bfloat16", page_size=8, cache_tokens=1024, max_requests=4)
    slot = other.open_request()
    other.step([StepEntry(slot, random_tokens(1, 9, 1000), [8])])
    other.step([StepEntry(slot, [5], [0])])
    assert other.fused is None or not other.fused.takes(other.ctx)


@pytest.mark.parametrize("dtype, key", [("float32", "A"), ("bfloat16", "B"), ("bfloat16", "C")])
def test_previous_names_the_last_sampled_token_on_the_device(folders, dtype, key):
    """A request fed PREVIOUS gets exactly what it gets when the host reads the sampled token
    and feeds it back: through the one-kernel decode step (C), the part-by-part path (A, B),
    with several requests per step and as the first token of a longer entry."""
    from mini_llm_b200.engine import PREVIOUS, SamplingParams, StepEntry, StepError
    engine = engine_of(folders, key, dtype)
    vocab = CONFIGS[key]["vocab_size"]
    prompts = [random_tokens(300 + i, n, vocab) for i, n in enumerate((19, 4, 33))]
    results = {}
    for mode in ("host", "device"):
        slots = [engine.open_request() for _ in prompts]
        with pytest.raises(StepError, match="has sampled no token"):
            engine.step([StepEntry(slots[0], [PREVIOUS], [0])])
        engine.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)],
                    [SamplingParams(0.9, 1.0, 50 + i, 0) for i in range(3)])
        tokens = engine.sampled_tokens()
        rows, drawn = [], [tokens]
        for step in range(1, 6):
            feed = [[PREVIOUS] if mode == "device" else [t] for t in tokens]
            if step == 3:                                  # a longer entry that starts with the sampled token
                feed[1] = feed[1] + [7, 11]
            out = engine.step([StepEntry(s, f, [len(f) - 1]) for s, f in zip(slots, feed)],
                              [SamplingParams(0.9, 1.0, 50 + i, step) for i in range(3)])
            rows.append(out.cpu().numpy().copy())
            tokens = engine.sampled_tokens()
            drawn.append(tokens)
        assert engine.sampled_tokens(ago=1) == drawn[-2]   # the step before stays readable
        for s in slots:
            engine.close_request(s)
        results[mode] = (rows, drawn)
    engine.check_status()
    assert results["host"][1] == results["device"][1]
    for a, b in zip(results["host"][0], results["device"][0]):
        np.testing.assert_array_equal(a, b)
    if key == "C":
        assert engine.fused is not None


def test_fused_decode_step_with_products_that_stream(tmp_path):
    """Sizes at which the one-kernel step's products do not fit their prefetch: a vocabulary of
    40,000 (17 blocks of rows per CTA, each longer than the prefetch) and an inner size of 4096
    (a warp's share of K longer than the prefetch).  Against the part-by-part path."""
    from mini_llm_b200.engine import Engine, SamplingParams, StepEntry
    raw = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 2, "n_embd": 512, "n_head": 8,
           "n_inner": 4096, "vocab_size": 40000, "n_positions": 256, "activation_function": "gelu_new",
           "layer_norm_epsilon": 1e-5, "tie_word_embeddings": True}
    folder = make_model(str(tmp_path / "wide"), raw, "varied", 3)
    fused = Engine(folder, dtype="bfloat16", page_size=16, cache_tokens=2048, max_requests=8)
    plain = Engine(folder, dtype="bfloat16", page_size=16, cache_tokens=2048, max_requests=8, fused_decode=False)
    assert fused.fused is not None
    prompts = [random_tokens(90 + i, n, 40000) for i, n in enumerate((60, 7, 150))]
    feed = np.random.default_rng(9).integers(0, 40000, (6, len(prompts)))
    rows = {}
    for name, engine in (("fused", fused), ("plain", plain)):
        slots = [engine.open_request() for _ in prompts]
        engine.step([StepEntry(s, p, []) for s, p in zip(slots, prompts)])
        rows[name] = []
        for step in range(6):
            out = engine.step([StepEntry(s, [int(feed[step, i])], [0]) for i, s in enumerate(slots)],
                              [SamplingParams(0.0, 1.0, 0, step) for _ in slots])
            rows[name].append((out.cpu().numpy().copy(), engine.sampled_tokens()))
        engine.check_status()
    assert fused.fused is not None and fused.kernels.launches < plain.kernels.launches / 3
    agree = 0
    for (a, ta), (b, tb) in zip(rows["fused"], rows["plain"]):
        np.testing.assert_allclose(a, b, rtol=0, atol=bf16_atol(b))
        agree += sum(x == y for x, y in zip(ta, tb))
    assert agree >= 16                                   # greedy choices agree, near-ties apart
