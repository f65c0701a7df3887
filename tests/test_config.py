import json

import pytest

from mini_llm_b200.config import (ConfigError, Gpt2Config, config_from_dict, config_from_folder, describe_model,
                                  known_architectures)
from tiny_configs import TINY_A, TINY_B


def test_reads_the_architectures_own_keys():
    c = config_from_dict(TINY_B)
    assert isinstance(c, Gpt2Config)
    assert (c.n_layer, c.n_embd, c.n_head, c.n_inner, c.vocab_size, c.n_positions) == (3, 96, 2, 160, 1000, 64)
    assert c.layer_norm_epsilon == 1e-6 and c.activation == "gelu_erf" and c.scale_attn_by_inverse_layer_idx
    assert c.head_size == 48 and c.architecture == "GPT2LMHeadModel"


def test_defaults_aliases_and_null():
    raw = {"model_type": "gpt2", "n_layer": 1, "n_embd": 32, "n_head": 2, "vocab_size": 50, "n_ctx": 16,
           "n_inner": None, "eos_token_id": 7, "unknown_key": [1, 2]}
    c = config_from_dict(raw)
    assert c.n_inner == 128 and c.n_positions == 16 and c.activation == "gelu_tanh" and c.eos_token_id == 7
    assert c.scale_attn_weights and not c.scale_attn_by_inverse_layer_idx and c.tie_word_embeddings
    again = config_from_dict(json.loads(json.dumps(c.to_dict())))
    assert again == c


@pytest.mark.parametrize("change, word", [
    ({"n_embd": 65}, "n_embd"), ({"n_head": 0}, "n_head"), ({"activation_function": "swish"}, "activation_function"),
    ({"n_layer": "two"}, "n_layer"), ({"layer_norm_epsilon": 0}, "layer_norm_epsilon"),
    ({"vocab_size": None}, "vocab_size"), ({"scale_attn_by_inverse_layer_idx": 1}, "scale_attn_by_inverse_layer_idx"),
    ({"eos_token_id": 512}, "eos_token_id"),
])
def test_errors_name_the_key(change, word):
    with pytest.raises(ConfigError) as error:
        config_from_dict({**TINY_A, **change})
    assert word in str(error.value)


def test_unknown_architecture_lists_known():
    with pytest.raises(ConfigError) as error:
        config_from_dict({**TINY_A, "architectures": ["SomethingElse"]})
    assert "SomethingElse" in str(error.value) and "GPT2LMHeadModel" in str(error.value)
    assert "GPT2LMHeadModel" in known_architectures()
    with pytest.raises(ConfigError):
        config_from_dict({"n_layer": 1})


def test_folder(tmp_path):
    with pytest.raises(ConfigError):
        config_from_folder(str(tmp_path))
    (tmp_path / "config.json").write_text("{not json")
    with pytest.raises(ConfigError):
        config_from_folder(str(tmp_path))
    (tmp_path / "config.json").write_text(json.dumps(TINY_A))
    assert config_from_folder(str(tmp_path)).n_embd == 64


def test_description_is_data():
    spec = describe_model(config_from_dict(TINY_B))
    assert len(spec.layers) == 3 and [e.layer for e in spec.order] == [0, 1, 2]
    scales = [layer.parts["mixer"].params["score_scale"] for layer in spec.layers]
    assert scales == pytest.approx([48 ** -0.5 / (i + 1) for i in range(3)])
    assert spec.layers[0].parts["feed_forward"].params == {"width": 96, "inner": 160, "activation": "gelu_erf"}
    assert spec.head.params["weight_name"] == "wte.weight"
    untied = describe_model(config_from_dict({**TINY_B, "tie_word_embeddings": False}))
    assert untied.head.params["weight_name"] == "lm_head.weight"
    flat = describe_model(config_from_dict({**TINY_A, "scale_attn_weights": False}))
    assert flat.layers[1].parts["mixer"].params["score_scale"] == 1.0
