"""Shared by the GPU tests: tiny model folders, the plain logits, and schedules that cut the
same requests into steps in different ways."""

import os
import struct
import json

import numpy as np

import plain_gpt2 as plain
from mini_llm_b200.config import config_from_dict
from mini_llm_b200.weights import write_random_model

# Largest allowed |engine - plain| on logits.  32-bit path: the target stated for it.
# bfloat16 path: a bound from its rounding, fixed before any run: every activation between
# kernels is rounded to 8 mantissa bits (relative 2^-9), about five roundings a layer, which
# add up like a random walk; the bound allows 4 % of the logits' standard deviation.
F32_ATOL = 1e-4


def bf16_atol(expected):
    return 0.04 * float(np.std(expected)) + 1e-3


def sharpen_attention(folder, factor):
    """Scale the query and key columns of every fused projection so that scores spread out
    and single keys matter: with the small random weights attention is nearly uniform and a
    lost or misplaced key would barely move the logits."""
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as handle:
        data = handle.read()
    (header_len,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + header_len])
    body = bytearray(data[8 + header_len:])
    for name, info in header.items():
        if not name.endswith("attn.c_attn.weight") or info["dtype"] != "F32":
            continue
        begin, end = info["data_offsets"]
        values = np.frombuffer(bytes(body[begin:end]), dtype="<f4").reshape(info["shape"]).copy()
        width = values.shape[0]
        values[:, :2 * width] *= factor
        body[begin:end] = values.astype("<f4").tobytes()
    with open(path, "wb") as handle:
        handle.write(data[:8 + header_len])
        handle.write(bytes(body))


def make_model(folder, raw_config, recipe, seed, sharpen=None):
    """Write a random model folder (stored in 32-bit)."""
    write_random_model(config_from_dict(raw_config), seed, folder, recipe=recipe, store_dtype="float32")
    if sharpen:
        sharpen_attention(folder, sharpen)
    return folder


_plain_cache = {}


def plain_logits(folder, tokens, bf16_weights=False):
    """Logits [len, vocab] of the plain implementation, float64 arithmetic."""
    key = (folder, tuple(tokens), bf16_weights)
    if key not in _plain_cache:
        config, tensors = plain.load_model(folder, round_matrices_to_bfloat16=bf16_weights)
        _plain_cache[key] = plain.forward(config, tensors, list(tokens))
    return _plain_cache[key]


def random_tokens(seed, length, vocab):
    return np.random.default_rng(seed).integers(0, vocab, length).tolist()


# ---- schedules: lists of steps; a step is a list of (request name, n tokens) -----------------

def schedule_whole(requests):
    return [[(name, len(tokens))] for name, tokens in requests.items()]


def schedule_tail_one_by_one(requests, tail=32):
    steps = []
    for name, tokens in requests.items():
        head = len(tokens) - tail
        if head > 0:
            steps.append([(name, head)])
        steps.extend([[(name, 1)]] * min(tail, len(tokens)))
    return steps


def schedule_portions(requests, sizes=(13, 7, 5, 3, 2, 2, 11, 2, 4)):
    steps = []
    for name, tokens in requests.items():
        left, i = len(tokens), 0
        while left > 0:
            n = min(sizes[i % len(sizes)], left)
            if left - n == 1:            # never leave a single token for a portion: fold it in
                n = left
            steps.append([(name, n)])
            left -= n
            i += 1
    return steps


def schedule_mixed(requests, prompt_lengths, max_live=4, portion_sizes=(7, 3, 2, 9, 5)):
    """Up to ``max_live`` requests at a time; each step every live request brings either its
    next prompt portion or, past its prompt, one token.  Requests start one step apart."""
    names = list(requests)
    progress = {n: 0 for n in names}
    waiting = list(names)
    live = []
    steps = []
    turn = 0
    while waiting or live:
        if waiting and len(live) < max_live:
            live.append(waiting.pop(0))
        step = []
        for name in list(live):
            done, total = progress[name], len(requests[name])
            if done < prompt_lengths[name]:
                n = min(portion_sizes[(turn + len(step)) % len(portion_sizes)], prompt_lengths[name] - done)
            else:
                n = 1
            n = min(n, total - done)
            step.append((name, n))
            progress[name] += n
            if progress[name] == total:
                live.remove(name)
        steps.append(step)
        turn += 1
    return steps


def run_schedule(engine, requests, steps, want_all=True):
    """Drive ``engine.step`` with a schedule.  Returns {name: logits [len, vocab]} (numpy
    float32) and closes each request after its last token."""
    from mini_llm_b200.engine import StepEntry

    progress = {n: 0 for n in requests}
    slots = {}
    vocab = engine.spec.vocab_size
    out = {n: np.full((len(t), vocab), np.nan, dtype=np.float32) for n, t in requests.items()}
    for step in steps:
        entries, places = [], []
        for name, n in step:
            if name not in slots:
                slots[name] = engine.open_request()
                assert slots[name] is not None, "no free slot"
            start = progress[name]
            want = list(range(n)) if want_all else [n - 1]
            entries.append(StepEntry(slots[name], requests[name][start:start + n], want))
            places.extend((name, start + w) for w in want)
            progress[name] += n
        logits = engine.step(entries).cpu().numpy()
        engine.check_status()
        assert logits.shape == (len(places), vocab)
        for row, (name, position) in zip(logits, places):
            out[name][position] = row
        for name, _ in step:
            if progress[name] == len(requests[name]):
                engine.close_request(slots.pop(name))
    return out
