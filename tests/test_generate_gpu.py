"""Generation through the Python entry point and the command line, against the plain
implementation recomputing the whole sequence for every token."""

import os
import subprocess
import sys

import numpy as np
import pytest

import plain_gpt2 as plain
from engine_helpers import make_model, random_tokens
from tiny_configs import TINY_A, TINY_B

pytestmark = pytest.mark.gpu

# A chosen token may differ from the plain implementation's only where the two best
# candidates are this close (logit units, after temperature and noise).
MARGIN = {"float32": 1e-4, "bfloat16": 3e-2}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {"A": make_model(str(tmp_path_factory.mktemp("gen_a")), TINY_A, "varied", 0, sharpen=2.0),
            "B": make_model(str(tmp_path_factory.mktemp("gen_b")), TINY_B, "varied", 1, sharpen=2.0)}


def follow(folder, dtype, prompt, tokens, temperature=0.0, top_p=1.0, seed=0):
    """Teacher-forced comparison: at every step the plain implementation, given the engine's
    tokens so far, must choose the engine's next token, or be undecided within MARGIN."""
    config, tensors = plain.load_model(folder, round_matrices_to_bfloat16=(dtype == "bfloat16"))
    history = list(prompt)
    undecided = 0
    for step, token in enumerate(tokens):
        logits = plain.forward(config, tensors, history)[-1]
        if temperature > 0:
            choice, margin = plain.sample(logits, temperature, top_p, seed, step, return_margin=True)
        else:
            choice = plain.argmax_first(logits)
            ordered = np.sort(logits)
            margin = float(ordered[-1] - ordered[-2])
        if choice != token:
            assert margin < MARGIN[dtype], f"step {step}: engine {token}, plain {choice}, margin {margin}"
            undecided += 1
        history.append(token)
    return undecided


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation(folders, dtype):
    from mini_llm_b200.generate import generate
    prompts = [random_tokens(i, n, 512) for i, n in enumerate((5, 17, 33))]
    got = generate(folders["A"], prompts, max_new_tokens=8, temperature=0.0, dtype=dtype, page_size=16)
    assert [len(t) for t in got] == [8, 8, 8]
    undecided = sum(follow(folders["A"], dtype, p, t) for p, t in zip(prompts, got))
    assert undecided <= (0 if dtype == "float32" else 2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_temperature_sampling_in_mixed_batches(folders, dtype):
    """Four requests, prompts cut into portions of 7 tokens beside decoding requests, pages
    of 8 tokens, temperature 0.8: each request's tokens are those of the plain sampler with
    the same seed, whatever it was batched with."""
    from mini_llm_b200.generate import LLM
    prompts = [random_tokens(10 + i, n, 1000) for i, n in enumerate((1, 9, 24, 40))]
    seeds = [101, 102, 103, 104]
    llm = LLM(folders["B"], dtype=dtype, page_size=8, max_tokens_per_step=7, max_sessions=4)
    got = llm.generate(prompts, max_new_tokens=12, temperature=0.8, seed=seeds)
    stats = llm.scheduler.stats()
    assert stats["tokens"] == 48 and stats["prefill_tokens"] == 74 and stats["mean_batch_size"] > 1.5
    undecided = sum(follow(folders["B"], dtype, p, t, 0.8, 1.0, s) for p, t, s in zip(prompts, got, seeds))
    assert undecided <= (0 if dtype == "float32" else 3)
    alone = LLM(folders["B"], dtype=dtype, page_size=8).generate([prompts[2]], 12, 0.8, seed=[103])
    assert alone[0] == got[2]                      # the same tokens alone and whole as in the mixed batches
    nucleus = llm.generate(prompts[1:3], max_new_tokens=6, temperature=1.3, top_p=0.6, seed=[7, 8])
    for p, t, s in zip(prompts[1:3], nucleus, [7, 8]):
        follow(folders["B"], dtype, p, t, 1.3, 0.6, s)
    assert llm.engine.cache.pages_in_use() == [0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_preemption_on_the_device_keeps_the_tokens(folders, dtype):
    """So few pages that decoding requests are preempted and recomputed: same tokens."""
    from mini_llm_b200.generate import LLM
    prompts = [random_tokens(20 + i, n, 512) for i, n in enumerate((30, 28, 26))]
    roomy = LLM(folders["A"], dtype=dtype, page_size=16).generate(prompts, max_new_tokens=40)
    tight = LLM(folders["A"], dtype=dtype, page_size=16, cache_tokens=176, max_sessions=3)
    got = tight.generate(prompts, max_new_tokens=40)
    assert tight.scheduler.stats()["preemptions"] >= 1
    assert tight.engine.cache.pages_in_use() == [0]
    tight.engine.cache.check()
    if dtype == "float32":
        assert got == roomy
    else:
        # a recomputed request meets other kernels (a prompt step instead of decode steps) and
        # so other rounding: its tokens are the plain implementation's, near-ties apart
        undecided = sum(follow(folders["A"], dtype, p, t) for p, t in zip(prompts, got))
        undecided += sum(follow(folders["A"], dtype, p, t) for p, t in zip(prompts, roomy))
        assert undecided <= 6


def test_a_bad_prompt_fails_alone(folders):
    """A prompt with an id outside the vocabulary, or a negative one (which the engine would
    read as "the token sampled last"), fails by itself at submission; the requests beside it
    run to their ends."""
    from mini_llm_b200.generate import LLM
    llm = LLM(folders["A"], dtype="float32", page_size=16)
    good = [random_tokens(70 + i, n, 512) for i, n in enumerate((9, 20))]
    requests = llm.generate([good[0], [3, 512, 4], good[1], [5, -1], [-1]], max_new_tokens=6, return_requests=True)
    assert [r.error is None for r in requests] == [True, False, True, False, False]
    assert "512" in requests[1].error and "-1" in requests[3].error
    assert all(len(r.generated) == 6 for r in (requests[0], requests[2]))
    assert follow(folders["A"], "float32", good[0], requests[0].generated) == 0
    assert llm.engine.cache.pages_in_use() == [0] and llm.engine.cache.free_slots == llm.engine.max_requests


def test_stop_context_and_errors(folders):
    from mini_llm_b200.generate import LLM
    llm = LLM(folders["A"], dtype="float32")
    prompt = random_tokens(3, 20, 512)
    free_run = llm.generate([prompt], max_new_tokens=6)[0]
    requests = llm.generate([prompt, random_tokens(4, 120, 512)], max_new_tokens=30, eos_token_id=free_run[3],
                            return_requests=True)
    assert requests[0].generated == free_run[:4] and requests[0].finish_reason == "stop"
    assert requests[1].finish_reason == "context" and len(requests[1].generated) == 8
    with pytest.raises(RuntimeError):
        llm.generate([[1] * 128], max_new_tokens=1)
    with pytest.raises(TypeError):
        LLM(folders["A"], no_such_option=1)


def test_command_line(folders):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    prompt = random_tokens(6, 12, 512)
    done = subprocess.run([sys.executable, "-m", "mini_llm_b200.cli", "--model", folders["A"], "--dtype", "float32",
                           "--max-new-tokens", "5", "--temperature", "0", "--prompt-ids",
                           ",".join(map(str, prompt))], capture_output=True, text=True, cwd=root, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    tokens = [int(t) for t in done.stdout.split()]
    assert len(tokens) == 5 and follow(folders["A"], "float32", prompt, tokens) == 0
    # random-weights mode: a config.json alone
    config_path = os.path.join(folders["A"], "config.json")
    twice = [subprocess.run([sys.executable, "-m", "mini_llm_b200.cli", "--random", config_path, "--weights-seed", "3",
                             "--dtype", "float32", "--max-new-tokens", "4", "--temperature", "0", "--prompt-ids",
                             "1,2,3"], capture_output=True, text=True, cwd=root, timeout=600) for _ in range(2)]
    assert twice[0].returncode == 0, twice[0].stderr[-2000:]
    assert len(twice[0].stdout.split()) == 4 and twice[0].stdout == twice[1].stdout      # the seed fixes the weights
    refused = subprocess.run([sys.executable, "-m", "mini_llm_b200.cli", "--model", folders["A"], "--device", "cpu"],
                             capture_output=True, text=True, cwd=root, timeout=600)
    assert refused.returncode != 0 and "no CPU path" in refused.stderr


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_ahead_of_the_host_changes_no_token(folders, dtype):
    """The scheduler launches a step before it has read the last one's tokens (requests feed
    themselves on the device).  Tokens, endings and the pages given back are those of the
    plain loop: with stop tokens found a step late, prompts in portions and sampling."""
    from mini_llm_b200.generate import LLM
    prompts = [random_tokens(60 + i, n, 1000) for i, n in enumerate((3, 21, 9, 40, 14, 2))]
    seeds = [5, 6, 7, 8, 9, 10]
    runs = {}
    for ahead in (False, True):
        llm = LLM(folders["B"], dtype=dtype, page_size=8, max_tokens_per_step=16, max_sessions=4, run_ahead=ahead)
        first = llm.generate(prompts, max_new_tokens=14, temperature=0.7, top_p=0.9, seed=seeds)
        eos = first[1][5]                                # a token request 1 really draws: it must stop there
        requests = llm.generate(prompts, max_new_tokens=14, temperature=0.7, top_p=0.9, seed=seeds, eos_token_id=eos,
                                return_requests=True)
        greedy = llm.generate(prompts[:3], max_new_tokens=9)
        assert llm.engine.cache.pages_in_use() == [0] and llm.scheduler._flight is None
        runs[ahead] = (first, [(r.generated, r.finish_reason) for r in requests], greedy)
        assert requests[1].finish_reason == "stop" and requests[1].generated == first[1][:first[1].index(eos) + 1]
    if dtype == "float32":
        assert runs[True] == runs[False]
    else:
        # The two modes admit a request a step apart, so a token may meet another batch (and
        # another kernel's rounding) in one than in the other: each mode's tokens are those of
        # the plain sampler, near-ties apart.
        for ahead in (False, True):
            undecided = sum(follow(folders["B"], dtype, p, t, 0.7, 0.9, s) for p, t, s in zip(prompts, runs[ahead][0], seeds))
            undecided += sum(follow(folders["B"], dtype, p, t) for p, t in zip(prompts[:3], runs[ahead][2]))
            assert undecided <= 4



def test_many_requests_through_the_scheduler_in_32_bit(folders):
    """Twenty requests of mixed lengths through four slots, prompts in portions of 16 tokens
    beside decoding requests, sampled: running ahead of the host or not, every request draws
    the same tokens (in 32-bit nothing depends on what a token was batched with), and every page
    and slot comes back."""
    from mini_llm_b200.generate import LLM
    rng = np.random.default_rng(21)
    prompts = [random_tokens(200 + i, int(rng.integers(1, 46)), 1000) for i in range(20)]
    seeds = list(range(300, 320))
    outs = {}
    for ahead in (True, False):
        llm = LLM(folders["B"], dtype="float32", page_size=8, cache_tokens=480, max_tokens_per_step=24,
                  max_prefill_chunk=16, max_sessions=4, run_ahead=ahead)
        requests = llm.generate(prompts, max_new_tokens=18, temperature=0.9, top_p=0.95, seed=seeds, return_requests=True)
        assert all(r.error is None and len(r.generated) == 18 for r in requests)
        stats = llm.scheduler.stats()
        assert stats["tokens"] == 20 * 18 and stats["running"] == 0 and stats["waiting"] == 0
        assert llm.engine.cache.pages_in_use() == [0] and llm.engine.cache.free_slots == 4
        llm.engine.check_status()
        outs[ahead] = [list(r.generated) for r in requests]
    assert outs[True] == outs[False]
    assert follow(folders["B"], "float32", prompts[7], outs[True][7], 0.9, 0.95, seeds[7]) == 0
