"""The plain implementation against the reference's own compiled CPU code.

``tests/golden/reference_tiny.npz`` was made once by ``tests/golden/make_golden.py`` from the
reference's unchanged ``engine/src/*.c``.  The whole model there uses gelu_new and the
1/sqrt(head size) scale, the only block the reference has; the erf gelu, another eps and a
head size of 48 are compared operator by operator.  The score scale by 1/(layer index + 1)
exists nowhere in the reference as an option; since scores are linear in the queries, the
reference's attention fed q/(layer index + 1) pins the mechanism.  That GPT-2's
``scale_attn_by_inverse_layer_idx`` means this rests on the key's stated meaning."""

import json
import os

import numpy as np

import plain_gpt2 as plain

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_tiny.npz"))
CONFIG = json.loads(str(GOLDEN["config"]))
WEIGHTS = {k[2:]: GOLDEN[k].astype(np.float64) for k in GOLDEN.files if k.startswith("w:")}


def test_embedding():
    got = plain.embed(GOLDEN["tokens"], WEIGHTS["wte.weight"], WEIGHTS["wpe.weight"])
    np.testing.assert_allclose(got, GOLDEN["embedded"], rtol=0, atol=1e-6)


def test_blocks_and_logits():
    logits, blocks = plain.forward(CONFIG, WEIGHTS, GOLDEN["tokens"], return_blocks=True)
    np.testing.assert_allclose(blocks[0], GOLDEN["embedded"], rtol=0, atol=1e-6)
    for i, hidden in enumerate(blocks[1:]):
        np.testing.assert_allclose(hidden, GOLDEN[f"block_{i}"], rtol=1e-5, atol=2e-5)
    np.testing.assert_allclose(logits, GOLDEN["logits"], rtol=1e-5, atol=5e-5)
    assert (logits.argmax(-1) == GOLDEN["logits"].argmax(-1)).all()


def test_float32_mode_agrees_too():
    logits = plain.forward(CONFIG, WEIGHTS, GOLDEN["tokens"], dtype=np.float32)
    np.testing.assert_allclose(logits, GOLDEN["logits"], rtol=1e-4, atol=2e-4)


def test_gelu_erf():
    got = plain.gelu_erf(GOLDEN["gelu_erf_in"].astype(np.float64))
    np.testing.assert_allclose(got, GOLDEN["gelu_erf_out"], rtol=1e-6, atol=1e-6)


def test_layer_norm_other_eps():
    got = plain.layer_norm(GOLDEN["ln_in"].astype(np.float64), GOLDEN["ln_gain"], GOLDEN["ln_shift"], 1e-6)
    np.testing.assert_allclose(got, GOLDEN["ln_out"], rtol=1e-5, atol=1e-5)


def test_attention_head_size_48():
    q, k, v = (GOLDEN[n].astype(np.float64) for n in ("att_q", "att_k", "att_v"))
    got = plain.multi_head_attention(q, k, v, 2, 1.0 / np.sqrt(48.0))
    np.testing.assert_allclose(got, GOLDEN["att_out"], rtol=1e-5, atol=1e-5)


def test_score_scale_by_inverse_layer_index():
    """Layer 2 (0-based) of a model with scale_attn_by_inverse_layer_idx: the plain
    implementation's scale 1/sqrt(head) / 3 against the reference's attention fed q / 3."""
    q, k, v = (GOLDEN[n].astype(np.float64) for n in ("att_q", "att_k", "att_v"))
    config = {"n_embd": 96, "n_head": 2, "scale_attn_by_inverse_layer_idx": True}
    assert abs(plain.score_scale(config, 2) - 1.0 / np.sqrt(48.0) / 3.0) < 1e-15
    got = plain.multi_head_attention(q, k, v, 2, plain.score_scale(config, 2))
    np.testing.assert_allclose(got, GOLDEN["att_out_layer_2"], rtol=1e-5, atol=1e-5)
    assert np.abs(got - GOLDEN["att_out"]).max() > 1e-2          # the option changes the result


def test_window_equals_full_when_wide():
    rng = np.random.default_rng(0)
    q, k, v = (rng.normal(size=(9, 16)) for _ in range(3))
    full = plain.attention_head(q, k, v, 0.25)
    np.testing.assert_allclose(plain.attention_head(q, k, v, 0.25, window=9), full)
    narrow = plain.attention_head(q, k, v, 0.25, window=3)
    np.testing.assert_allclose(narrow[:3], full[:3])
    assert not np.allclose(narrow[5], full[5])


def test_sampler_rules():
    assert plain.argmax_first([1.0, 3.0, 3.0]) == 1
    assert plain.argmax_first([1.0, np.nan, 5.0, np.nan]) == 1
    logits = np.array([0.0, 5.0, 4.9, -3.0])
    assert plain.sample(logits, 0.0) == 1
    picks = {plain.sample(logits, 1.0, 1.0, seed=7, counter=c) for c in range(200)}
    assert {1, 2} <= picks
    nucleus = {plain.sample(logits, 1.0, 0.5, seed=7, counter=c) for c in range(200)}
    assert nucleus == {1}                       # p(1) = 0.52 reaches 0.5 alone
    two = {plain.sample(logits, 1.0, 0.9, seed=7, counter=c) for c in range(200)}
    assert two == {1, 2}
