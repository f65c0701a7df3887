"""Generality of the parts framework, shown with toy parts that exist only in this test:

* a mixer with state of its own (a decaying running sum per request, kept in the request's
  slot), a new architecture name and configuration class, registered from here, built from a
  model folder, and stepped in portions, with no change to the framework's files;
* a run order that names a layer twice;
* a layer that reads another layer's cache.

The toy mixer computes with torch operations: it is a test double, not a product kernel."""

import json
import os
from dataclasses import dataclass, field

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from engine_helpers import F32_ATOL, random_tokens, run_schedule, schedule_portions, schedule_whole
from mini_llm_b200.config import ModelConfig, register_architecture
from mini_llm_b200.parts import (FixedState, LayerSpec, Mixer, ModelSpec, PartSpec, RunEntry, WeightSpec,
                                 register_part)
from mini_llm_b200.weights import write_random_model

pytestmark = pytest.mark.gpu


class DecayingSum(Mixer):
    """state_t = decay * state_{t-1} + x_t;  hidden_t += W state_t."""

    def __init__(self, prefix, width, decay):
        super().__init__(prefix)
        self.width, self.decay = int(width), float(decay)

    def weight_specs(self):
        return [WeightSpec(self.full_name("mix.weight"), (self.width, self.width), init="residual_matrix")]

    def cache_need(self):
        return FixedState((self.width,), "float32")

    def forward(self, ctx, x, hidden, cache):
        weight = self.w("mix.weight").float()
        for slot, offset, count in zip(ctx.item_slots, ctx.item_offsets, ctx.item_counts):
            state = cache.state[slot].clone()
            rows = x[offset:offset + count].float()
            states = torch.empty_like(rows)
            for t in range(count):
                state = self.decay * state + rows[t]
                states[t] = state
            hidden[offset:offset + count] += states @ weight.t()
            if cache.writes:
                cache.state[slot] = state


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    n_layer: int = field(default=0, metadata={"kind": int})
    width: int = field(default=0, metadata={"kind": int})
    inner: int = field(default=0, metadata={"kind": int})
    vocab_size: int = field(default=0, metadata={"kind": int})
    decay: float = field(default=0.5, metadata={"kind": float})


def describe_toy(config):
    layers = tuple(LayerSpec("pre_norm", {
        "norm_1": PartSpec("layer_norm", f"l.{i}.n1", {"width": config.width, "eps": 1e-5}),
        "mixer": PartSpec("decaying_sum", f"l.{i}", {"width": config.width, "decay": config.decay / (i + 1)}),
        "norm_2": PartSpec("layer_norm", f"l.{i}.n2", {"width": config.width, "eps": 1e-5}),
        "feed_forward": PartSpec("dense_mlp", f"l.{i}.ff", {"width": config.width, "inner": config.inner,
                                                             "activation": "gelu_tanh"}),
    }) for i in range(config.n_layer))
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab_size, max_positions=None,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab_size, "width": config.width}),
        position=None, layers=layers,
        order=(RunEntry(0), RunEntry(1), RunEntry(0)),          # layer 0 runs twice, each run with its own state
        final_norm=PartSpec("layer_norm", "out_norm", {"width": config.width, "eps": 1e-5}),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab_size, "width": config.width,
                                          "weight_name": "wte.weight"}))


def toy_plain_logits(folder, tokens):
    config, t = plain.load_model(folder)
    hidden = t["wte.weight"][np.asarray(tokens)]
    for layer, decay in ((0, config["decay"]), (1, config["decay"] / 2), (0, config["decay"])):
        p = f"l.{layer}."
        x = plain.layer_norm(hidden, t[p + "n1.weight"], t[p + "n1.bias"], 1e-5)
        state = np.zeros(config["width"])
        states = np.empty_like(x)
        for i in range(len(tokens)):
            state = decay * state + x[i]
            states[i] = state
        hidden = hidden + states @ t[p + "mix.weight"].T
        x = plain.layer_norm(hidden, t[p + "n2.weight"], t[p + "n2.bias"], 1e-5)
        up = plain.gelu_tanh(plain.linear(x, t[p + "ff.c_fc.weight"], t[p + "ff.c_fc.bias"]))
        hidden = hidden + plain.linear(up, t[p + "ff.c_proj.weight"], t[p + "ff.c_proj.bias"])
    return plain.layer_norm(hidden, t["out_norm.weight"], t["out_norm.bias"], 1e-5) @ t["wte.weight"].T


def test_a_mixer_with_state_of_its_own_registers_builds_and_steps(tmp_path):
    from mini_llm_b200.engine import Engine
    register_part("decaying_sum", DecayingSum)
    register_architecture("ToyDecayLM", ToyConfig, describe_toy)
    config = ToyConfig(architecture="ToyDecayLM", n_layer=2, width=48, inner=72, vocab_size=201, decay=0.8)
    folder = write_random_model(config, 4, str(tmp_path / "toy"), recipe="varied")
    assert json.load(open(os.path.join(folder, "config.json")))["architectures"] == ["ToyDecayLM"]
    engine = Engine(folder, dtype="float32", max_requests=3)
    assert [g.paged for g in engine.cache.groups] == [False]
    assert engine.storage.states[0].shape == (3, 3, 48)        # three run entries, three slots
    requests = {"u": random_tokens(1, 23, 201), "v": random_tokens(2, 9, 201), "w": random_tokens(3, 40, 201)}
    for steps in (schedule_whole(requests), schedule_portions(requests, sizes=(5, 2, 3, 7)),
                  [[("u", 10), ("v", 4)], [("u", 1), ("v", 1), ("w", 13)], [("u", 12), ("v", 4), ("w", 27)]]):
        got = run_schedule(engine, requests, steps)       # slots are reused: their state must restart at zero
        for name, tokens in requests.items():
            np.testing.assert_allclose(got[name], toy_plain_logits(folder, tokens), rtol=0, atol=F32_ATOL)


@dataclass(frozen=True)
class SharedCacheConfig(ModelConfig):
    width: int = field(default=0, metadata={"kind": int})
    n_head: int = field(default=0, metadata={"kind": int})
    inner: int = field(default=0, metadata={"kind": int})
    vocab_size: int = field(default=0, metadata={"kind": int})
    n_positions: int = field(default=0, metadata={"kind": int})


def describe_shared(config):
    head = config.width // config.n_head
    def layer(i):
        return LayerSpec("pre_norm", {
            "norm_1": PartSpec("layer_norm", f"h.{i}.ln_1", {"width": config.width, "eps": 1e-5}),
            "mixer": PartSpec("causal_self_attention", f"h.{i}.attn", {"width": config.width, "n_heads": config.n_head,
                                                                       "head_size": head, "score_scale": head ** -0.5}),
            "norm_2": PartSpec("layer_norm", f"h.{i}.ln_2", {"width": config.width, "eps": 1e-5}),
            "feed_forward": PartSpec("dense_mlp", f"h.{i}.mlp", {"width": config.width, "inner": config.inner,
                                                                  "activation": "gelu_tanh"})})
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab_size, max_positions=config.n_positions,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab_size, "width": config.width}),
        position=PartSpec("learned_positions", "", {"max_positions": config.n_positions, "width": config.width}),
        layers=(layer(0), layer(1)),
        order=(RunEntry(0), RunEntry(1, cache_of=0)),           # layer 1 attends over layer 0's keys and values
        final_norm=PartSpec("layer_norm", "ln_f", {"width": config.width, "eps": 1e-5}),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab_size, "width": config.width,
                                          "weight_name": "wte.weight"}))


def shared_plain_logits(folder, tokens):
    config, t = plain.load_model(folder)
    width, heads = config["width"], config["n_head"]
    scale = (width // heads) ** -0.5
    hidden = plain.embed(tokens, t["wte.weight"], t["wpe.weight"])
    kept = None
    for i in range(2):
        p = f"h.{i}."
        x = plain.layer_norm(hidden, t[p + "ln_1.weight"], t[p + "ln_1.bias"], 1e-5)
        qkv = plain.linear(x, t[p + "attn.c_attn.weight"], t[p + "attn.c_attn.bias"])
        q, k, v = qkv[:, :width], qkv[:, width:2 * width], qkv[:, 2 * width:]
        if i == 0:
            kept = (k, v)
        mixed = plain.multi_head_attention(q, kept[0], kept[1], heads, scale)
        hidden = hidden + plain.linear(mixed, t[p + "attn.c_proj.weight"], t[p + "attn.c_proj.bias"])
        x = plain.layer_norm(hidden, t[p + "ln_2.weight"], t[p + "ln_2.bias"], 1e-5)
        up = plain.gelu_tanh(plain.linear(x, t[p + "mlp.c_fc.weight"], t[p + "mlp.c_fc.bias"]))
        hidden = hidden + plain.linear(up, t[p + "mlp.c_proj.weight"], t[p + "mlp.c_proj.bias"])
    return plain.layer_norm(hidden, t["ln_f.weight"], t["ln_f.bias"], 1e-5) @ t["wte.weight"].T


def test_a_layer_reads_another_layers_cache(tmp_path):
    from mini_llm_b200.engine import Engine
    register_architecture("ToySharedCacheLM", SharedCacheConfig, describe_shared)
    config = SharedCacheConfig(architecture="ToySharedCacheLM", width=64, n_head=2, inner=96, vocab_size=150,
                               n_positions=64)
    folder = write_random_model(config, 8, str(tmp_path / "shared"), recipe="varied")
    engine = Engine(folder, dtype="float32", page_size=8, max_requests=2)
    assert len(engine.cache.groups) == 1 and engine.cache.groups[0].entries == [0]      # one cache for two layers
    assert engine.storage.keys[0].shape[0] == 1
    requests = {"s": random_tokens(5, 50, 150), "t": random_tokens(6, 21, 150)}
    for steps in (schedule_whole(requests), schedule_portions(requests)):
        got = run_schedule(engine, requests, steps)
        for name, tokens in requests.items():
            np.testing.assert_allclose(got[name], shared_plain_logits(folder, tokens), rtol=0, atol=F32_ATOL)
