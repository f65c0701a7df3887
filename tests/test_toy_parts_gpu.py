"""Generality of the parts framework, shown with toy parts that exist only in this test:

* a mixer with state of its own (a decaying running sum per request, kept in the request's
  slot), a new architecture name and configuration class, registered from here, built from a
  model folder, and stepped in portions, with no change to the framework's files;
* a run order that names a layer twice;
* a layer that reads another layer's cache;
* layers with and without a window in one model (two cache groups), a feed-forward with
  routing, and a position encoding that rotates queries and keys inside the attention part.

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
from mini_llm_b200.parts import (FeedForward, FixedState, LayerSpec, Mixer, ModelSpec, PartSpec, PositionEncoding,
                                 RunEntry, WeightSpec, register_part)
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


def test_a_model_the_one_kernel_step_does_not_take_says_why_and_builds_no_tile_list(tmp_path):
    """The toy stack in bfloat16: its decode steps run part by part, the engine says which
    part stands in the way, and a step makes no work list of attention tiles, since no part
    of the model reads one."""
    from mini_llm_b200.engine import Engine, StepEntry
    register_part("decaying_sum", DecayingSum)
    register_architecture("ToyDecayLM", ToyConfig, describe_toy)
    config = ToyConfig(architecture="ToyDecayLM", n_layer=2, width=64, inner=96, vocab_size=201, decay=0.8)
    folder = write_random_model(config, 4, str(tmp_path / "toy16"), recipe="varied")
    engine = Engine(folder, dtype="bfloat16", max_requests=3)
    assert engine.fused is None and "decaying_sum" in engine.fused_reason and "mixer" in engine.fused_reason
    assert not engine.model.wants_attention_tiles
    slot = engine.open_request()
    tokens = random_tokens(1, 90, 201)
    logits = engine.step([StepEntry(slot, tokens, [89])]).cpu().numpy()
    assert engine.ctx.att_tiles is None and engine.ctx.n_att_tiles == 0
    expected = toy_plain_logits(folder, tokens)
    assert np.abs(logits[0] - expected[89]).max() <= 0.04 * expected.std() + 1e-3 + 0.02   # torch's bf16 products in the toy
    engine.close_request(slot)


# ---- a window, a routed feed-forward and a rotation: toy architectures over the product kernels ----

@dataclass(frozen=True)
class ToyMixConfig(ModelConfig):
    width: int = field(default=0, metadata={"kind": int})
    n_head: int = field(default=0, metadata={"kind": int})
    inner: int = field(default=0, metadata={"kind": int})
    vocab_size: int = field(default=0, metadata={"kind": int})
    n_positions: int = field(default=0, metadata={"kind": int})
    window: int = field(default=0, metadata={"kind": int})
    n_experts: int = field(default=0, metadata={"kind": int})
    rotary_base: float = field(default=0.0, metadata={"kind": float})


class RoutedMlp(FeedForward):
    """A feed-forward with routing: the router's logits (32-bit) choose one expert per token;
    hidden += W_down[e] gelu(W_up[e] x).  Torch operations: a test double, not a product kernel."""

    def __init__(self, prefix, width, inner, n_experts):
        super().__init__(prefix)
        self.width, self.inner, self.n_experts = int(width), int(inner), int(n_experts)

    def weight_specs(self):
        specs = [WeightSpec(self.full_name("router.weight"), (self.n_experts, self.width), keep_32bit=True)]
        for e in range(self.n_experts):
            specs.append(WeightSpec(self.full_name(f"experts.{e}.up.weight"), (self.inner, self.width)))
            specs.append(WeightSpec(self.full_name(f"experts.{e}.down.weight"), (self.width, self.inner),
                                    init="residual_matrix"))
        return specs

    def forward(self, ctx, x, hidden):
        x = x.float()
        choice = (x @ self.w("router.weight").float().t()).argmax(dim=1)
        for e in range(self.n_experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                up = torch.nn.functional.gelu(x[rows] @ self.w(f"experts.{e}.up.weight").float().t(), approximate="tanh")
                hidden[rows] += up @ self.w(f"experts.{e}.down.weight").float().t()


class ToyRotation(PositionEncoding):
    """Rotates pairs (i, i + D/2) of every head of q and k by position * base^(-2i/D); the
    angles are 32-bit.  It has no weights and is given to the attention part as ``position``."""

    def __init__(self, prefix, base):
        super().__init__(prefix)
        self.base = float(base)

    def rotate(self, ctx, q, k, n_heads, n_kv_heads, head_size):
        half = head_size // 2
        inv = self.base ** (-torch.arange(half, device=q.device, dtype=torch.float32) / half)
        angle = ctx.positions[:q.shape[0]].float()[:, None] * inv[None, :]
        cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
        for tensor, heads in ((q, n_heads), (k, n_kv_heads)):
            view = tensor.unflatten(1, (heads, head_size))        # a view: q and k are column ranges of one buffer
            lo, hi = view[..., :half].float(), view[..., half:].float()
            new_lo, new_hi = lo * cos - hi * sin, hi * cos + lo * sin      # both before either is written
            view[..., :half] = new_lo.to(tensor.dtype)
            view[..., half:] = new_hi.to(tensor.dtype)


def describe_mix(config):
    head = config.width // config.n_head
    position = PartSpec("toy_rotation", "", {"base": config.rotary_base}) if config.rotary_base > 0 else None

    def layer(i):
        mixer = {"width": config.width, "n_heads": config.n_head, "head_size": head, "score_scale": head ** -0.5}
        if config.window > 0 and i % 2 == 0:                 # layers with a window and layers without, in turn
            mixer["window"] = config.window
        if position is not None:
            mixer["position"] = position
        if config.n_experts > 0 and i % 2 == 1:
            ff = PartSpec("routed_mlp", f"h.{i}.moe", {"width": config.width, "inner": config.inner,
                                                       "n_experts": config.n_experts})
        else:
            ff = PartSpec("dense_mlp", f"h.{i}.mlp", {"width": config.width, "inner": config.inner,
                                                      "activation": "gelu_tanh"})
        return LayerSpec("pre_norm", {
            "norm_1": PartSpec("layer_norm", f"h.{i}.ln_1", {"width": config.width, "eps": 1e-5}),
            "mixer": PartSpec("causal_self_attention", f"h.{i}.attn", mixer),
            "norm_2": PartSpec("layer_norm", f"h.{i}.ln_2", {"width": config.width, "eps": 1e-5}),
            "feed_forward": ff})
    learned = config.rotary_base <= 0
    return ModelSpec(
        hidden_size=config.width, vocab_size=config.vocab_size, max_positions=config.n_positions,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab_size, "width": config.width}),
        position=PartSpec("learned_positions", "", {"max_positions": config.n_positions, "width": config.width})
        if learned else None,
        layers=(layer(0), layer(1)), order=(RunEntry(0), RunEntry(1)),
        final_norm=PartSpec("layer_norm", "ln_f", {"width": config.width, "eps": 1e-5}),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab_size, "width": config.width,
                                          "weight_name": "wte.weight"}))


def mix_plain_logits(folder, tokens, bf16=False):
    config, t = plain.load_model(folder, round_matrices_to_bfloat16=bf16)
    width, heads = config["width"], config["n_head"]
    head = width // heads
    n = len(tokens)
    rotary = config.get("rotary_base", 0.0) > 0
    hidden = t["wte.weight"][np.asarray(tokens)] + (0 if rotary else t["wpe.weight"][np.arange(n)])
    for i in range(2):
        p = f"h.{i}."
        x = plain.layer_norm(hidden, t[p + "ln_1.weight"], t[p + "ln_1.bias"], 1e-5)
        qkv = plain.linear(x, t[p + "attn.c_attn.weight"], t[p + "attn.c_attn.bias"])
        q, k, v = qkv[:, :width].copy(), qkv[:, width:2 * width].copy(), qkv[:, 2 * width:]
        if rotary:
            half = head // 2
            inv = config["rotary_base"] ** (-np.arange(half) / half)
            angle = np.arange(n)[:, None] * inv[None, :]
            for m in (q, k):
                for h in range(heads):
                    lo, hi = m[:, h * head:h * head + half].copy(), m[:, h * head + half:(h + 1) * head].copy()
                    m[:, h * head:h * head + half] = lo * np.cos(angle) - hi * np.sin(angle)
                    m[:, h * head + half:(h + 1) * head] = hi * np.cos(angle) + lo * np.sin(angle)
        window = config["window"] if config.get("window", 0) > 0 and i % 2 == 0 else None
        mixed = plain.multi_head_attention(q, k, v, heads, head ** -0.5, window=window)
        hidden = hidden + plain.linear(mixed, t[p + "attn.c_proj.weight"], t[p + "attn.c_proj.bias"])
        x = plain.layer_norm(hidden, t[p + "ln_2.weight"], t[p + "ln_2.bias"], 1e-5)
        if config.get("n_experts", 0) > 0 and i % 2 == 1:
            choice = (x @ t[p + "moe.router.weight"].T).argmax(axis=1)
            out = np.zeros_like(hidden)
            for e in range(config["n_experts"]):
                rows = np.flatnonzero(choice == e)
                up = plain.gelu_tanh(x[rows] @ t[p + f"moe.experts.{e}.up.weight"].T)
                out[rows] = up @ t[p + f"moe.experts.{e}.down.weight"].T
            hidden = hidden + out
        else:
            up = plain.gelu_tanh(plain.linear(x, t[p + "mlp.c_fc.weight"], t[p + "mlp.c_fc.bias"]))
            hidden = hidden + plain.linear(up, t[p + "mlp.c_proj.weight"], t[p + "mlp.c_proj.bias"])
    return plain.layer_norm(hidden, t["ln_f.weight"], t["ln_f.bias"], 1e-5) @ t["wte.weight"].T


def register_mix():
    register_part("routed_mlp", RoutedMlp)
    register_part("toy_rotation", ToyRotation)
    register_architecture("ToyMixLM", ToyMixConfig, describe_mix)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_window_through_the_engine(tmp_path, dtype):
    """One layer sees the last 20 keys only, the other all of them: two cache groups with
    pools of their own.  Portions that start and end on either side of the window's edge and
    of a page's, decoding across both, and so few pages that the pages the window has passed
    are given back in the middle of a request and used again by another."""
    from mini_llm_b200.engine import Engine
    from engine_helpers import sharpen_attention
    register_mix()
    config = ToyMixConfig(architecture="ToyMixLM", width=128, n_head=2, inner=192, vocab_size=211, n_positions=160,
                          window=20)
    folder = write_random_model(config, 6, str(tmp_path / "window"), recipe="varied", store_dtype="float32")
    sharpen_attention(folder, 1.5)
    # the windowed group: at most 4 pages of 8 per request (20 keys + a portion's reach); both small
    engine = Engine(folder, dtype=dtype, page_size=8, n_pages=44, max_requests=4)
    assert [g.need.window for g in engine.cache.groups] == [20, None]
    if dtype == "bfloat16":
        assert engine.fused is None and "group" in engine.fused_reason      # two cache groups: the part-by-part path
    requests = {"w1": random_tokens(1, 150, 211), "w2": random_tokens(2, 47, 211), "w3": random_tokens(3, 96, 211),
                "w4": random_tokens(4, 21, 211)}
    tolerance = (lambda e: F32_ATOL) if dtype == "float32" else (lambda e: 0.04 * float(np.std(e)) + 1e-3)
    before = engine.cache.freed_by_window
    for steps in (schedule_whole(requests), schedule_portions(requests, sizes=(13, 7, 5, 3, 2, 2, 11, 2, 4)),
                  schedule_portions(requests, sizes=(70, 2, 19, 21, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1)),
                  [[("w1", 100), ("w2", 3)], [("w1", 1), ("w2", 40), ("w3", 90)], [("w1", 49), ("w2", 4), ("w3", 6), ("w4", 21)]]):
        got = run_schedule(engine, requests, steps)
        for name, tokens in requests.items():
            expected = mix_plain_logits(folder, tokens, bf16=(dtype == "bfloat16"))
            diff = np.abs(got[name] - expected).max(axis=1)
            bad = np.flatnonzero(diff > tolerance(expected))
            assert bad.size == 0, (name, int(bad[0]), float(diff[bad[0]]))
        engine.cache.check()
    assert engine.cache.freed_by_window > before and engine.cache.groups[0].pool.reused > 0
    assert engine.cache.pages_in_use() == [0, 0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_feed_forward_with_routing_and_a_rotation_of_queries_and_keys(tmp_path, dtype):
    """A layer whose feed-forward routes every token to one of three experts, and a position
    encoding that rotates queries and keys inside the attention part instead of adding a
    table to the embedding: both are parts of this test, registered from here, and run
    between the framework's own norm, product and attention kernels."""
    from mini_llm_b200.engine import Engine
    register_mix()
    config = ToyMixConfig(architecture="ToyMixLM", width=128, n_head=2, inner=160, vocab_size=173, n_positions=128,
                          n_experts=3, rotary_base=100.0)
    folder = write_random_model(config, 9, str(tmp_path / "routed"), recipe="varied", store_dtype="float32")
    engine = Engine(folder, dtype=dtype, page_size=16, cache_tokens=512, max_requests=3)
    assert engine.model.position is None
    requests = {"x": random_tokens(11, 100, 173), "y": random_tokens(12, 30, 173), "z": random_tokens(13, 3, 173)}
    for steps in (schedule_whole(requests), schedule_portions(requests, sizes=(66, 2, 9, 1, 1, 5)),
                  [[("x", 70), ("y", 29)], [("x", 1), ("y", 1), ("z", 3)], [("x", 29)]]):
        got = run_schedule(engine, requests, steps)
        for name, tokens in requests.items():
            expected = mix_plain_logits(folder, tokens, bf16=(dtype == "bfloat16"))
            if dtype == "float32":
                np.testing.assert_allclose(got[name], expected, rtol=0, atol=2e-4)     # the toy's torch sums
            else:
                # a token whose two best experts lie within rounding may take the other one:
                # most positions agree within the bfloat16 bound
                close = np.abs(got[name] - expected).max(axis=1) <= 0.04 * float(np.std(expected)) + 1e-3 + 0.02
                assert close.mean() >= 0.9, (name, close.mean())
