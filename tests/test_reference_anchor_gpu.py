"""The engine's 32-bit path against the reference's own GPU library, at GPT-2 small's full size.

The reference (WillyBruhn/mini_llm) is compiled for GPT-2 small only
(engine/include/gpt2.h:12-19), so this is the one size at which its own code can judge the
engine end to end.  The same seeded random weights go to both: as a model folder to the
engine, and as raw ``transformer.<name>.bin`` files (scripts/dump_weights.py:37-53) to the
reference's ``NativeGPT2`` (pytorch/src/mini_llm/native.py:169-233).  The reference then
prefills a prompt and decodes twelve tokens through its cached session
(native.py:88-166); the engine runs the same tokens cut two ways.  The gate is the
reference's own: logits within 1e-3 of their scale and the same best token
(engine/bench/bench.c:91-113, engine/tests/test_gpt2_gpu.c:220-247).

Skipped when the reference is not installed under ``baseline/_ref`` or its library cannot be
built here.
"""

import os
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REFERENCE = os.path.join(ROOT, "baseline", "_ref")


def reference_engine(weights_folder):
    if not os.path.isdir(os.path.join(REFERENCE, "mini_llm")):
        pytest.skip("the reference is not installed under baseline/_ref")
    sys.path.insert(0, ROOT)
    import bench
    library = os.path.join(REFERENCE, "build", "libmini_llm_gpu.so")
    if not os.path.isfile(library):
        problem = bench.build_reference_library(library)
        if problem:
            pytest.skip(f"the reference's library cannot be built: {problem}")
    sys.path.insert(0, REFERENCE)
    try:
        from mini_llm.native import EngineOptions, NativeGPT2
    except Exception as error:                                   # its dependencies are not all installed here
        pytest.skip(f"the reference's binding does not import: {error}")
    return NativeGPT2(weights_folder, library, backend="gpu",
                      options=EngineOptions(use_kv_cache=True, max_sessions=2, fp16_decode=False))


def test_the_32_bit_path_agrees_with_the_references_gpu_library(tmp_path):
    import bench
    from mini_llm_b200.config import config_from_dict, describe_model
    from mini_llm_b200.engine import Engine, StepEntry
    from mini_llm_b200.weights import random_tensors, write_random_model

    config = dict(bench.GPT2_SMALL)
    vocab = config["vocab_size"]
    typed = config_from_dict(config)
    # "varied": gains, shifts and biases that are not 1 and 0, and attention that is not uniform
    bins = tmp_path / "bins"
    bins.mkdir()
    for name, values in random_tensors(describe_model(typed), 7, "varied").items():
        values.astype("<f4").tofile(str(bins / f"transformer.{name}.bin"))
    folder = write_random_model(typed, 7, str(tmp_path / "model"), recipe="varied", store_dtype="float32")

    rng = np.random.default_rng(5)
    prompt = rng.integers(0, vocab, 21).tolist()
    reference = reference_engine(str(bins))
    session = reference.open_session()
    theirs = [session.prefill(np.asarray(prompt, dtype=np.int32)).copy()]
    tokens = list(prompt)
    for _ in range(12):
        tokens.append(int(np.argmax(theirs[-1])))               # teacher forcing with the reference's own choice
        theirs.append(session.decode(tokens[-1]).copy())
    session.close()
    reference.close()
    theirs = np.stack(theirs)                                    # logits at positions 20 .. 32

    engine = Engine(folder, dtype="float32", page_size=16, cache_tokens=256, max_requests=2)

    def check(mine, what):
        scale = max(1.0, float(np.abs(theirs).max()))
        worst = float(np.abs(mine - theirs).max()) / scale
        assert worst <= 1e-3, f"{what}: scaled difference {worst:.3g}"
        assert (mine.argmax(axis=1) == theirs.argmax(axis=1)).all(), what
        return worst

    # cut 1: the prompt whole, then token by token, as the reference runs it
    slot = engine.open_request()
    rows = [engine.step([StepEntry(slot, prompt, [20])]).cpu().numpy()[0]]
    for token in tokens[21:]:
        rows.append(engine.step([StepEntry(slot, [token], [0])]).cpu().numpy()[0])
    engine.close_request(slot)
    first = check(np.stack(rows), "whole prompt, then one token a step")

    # cut 2: the prompt in portions beside another request that decodes, then both together
    slot, other = engine.open_request(), engine.open_request()
    filler = rng.integers(0, vocab, 40).tolist()
    engine.step([StepEntry(other, filler[:9], [])])
    engine.step([StepEntry(slot, prompt[:8], []), StepEntry(other, filler[9:10], [])])
    engine.step([StepEntry(other, filler[10:11], []), StepEntry(slot, prompt[8:10], [])])
    rows = [engine.step([StepEntry(slot, prompt[10:], [10]), StepEntry(other, filler[11:12], [])]).cpu().numpy()[0]]
    for i, token in enumerate(tokens[21:]):
        out = engine.step([StepEntry(other, filler[12 + i:13 + i], []), StepEntry(slot, [token], [0])])
        rows.append(out.cpu().numpy()[0])
    engine.close_request(slot)
    engine.close_request(other)
    second = check(np.stack(rows), "prompt in portions beside a decoding request")
    engine.check_status()
    print(f"scaled difference to the reference's GPU library: {first:.3g} whole, {second:.3g} in portions")
