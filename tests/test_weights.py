import json
import os

import numpy as np
import pytest
import torch

import plain_gpt2 as plain
from mini_llm_b200.config import config_from_dict, describe_model
from mini_llm_b200.engine.model import Model
from mini_llm_b200.weights import (SafetensorsFile, WeightsError, collect_specs, load_weights, random_tensors,
                                   write_random_model, write_safetensors)
from mini_llm_b200.weights.safetensors_io import float32_to_bfloat16_bits
from tiny_configs import TINY_A, TINY_B


def _folder(tmp_path, raw=TINY_A, **kw):
    return write_random_model(config_from_dict(raw), 3, str(tmp_path / "m"), **kw)


def _specs(raw=TINY_A):
    spec = describe_model(config_from_dict(raw))
    return spec, collect_specs(Model(spec).parts())


def test_random_model_folder_roundtrip(tmp_path):
    folder = _folder(tmp_path, TINY_B, recipe="varied")
    assert sorted(os.listdir(folder)) == ["config.json", "model.safetensors"]
    spec, specs = _specs(TINY_B)
    tensors = load_weights(folder, specs, torch.float32, "cpu", spec.file_prefixes, spec.ignored_weights)
    assert set(tensors) == set(specs) and len(specs) == 2 + 3 * 12 + 2
    config, plain_tensors = plain.load_model(folder)
    assert config["n_inner"] == 160
    # [in, out] in the file, [out, in] on the device; vectors unchanged
    np.testing.assert_array_equal(tensors["h.1.attn.c_attn.weight"].numpy().T, plain_tensors["h.1.attn.c_attn.weight"])
    assert tensors["h.1.attn.c_attn.weight"].shape == (3 * 96, 96) and tensors["h.1.attn.c_attn.weight"].is_contiguous()
    np.testing.assert_array_equal(tensors["ln_f.bias"].numpy(), plain_tensors["ln_f.bias"])
    assert float(np.abs(plain_tensors["ln_f.bias"]).max()) > 0       # "varied" leaves nothing trivial


def test_same_seed_same_weights_other_seed_other(tmp_path):
    spec = describe_model(config_from_dict(TINY_A))
    a, b, c = random_tensors(spec, 5), random_tensors(spec, 5), random_tensors(spec, 6)
    assert all(np.array_equal(a[k], b[k]) for k in a)
    assert not np.array_equal(a["wte.weight"], c["wte.weight"])
    assert np.all(a["h.0.ln_1.weight"] == 1) and np.all(a["h.0.attn.c_attn.bias"] == 0)
    assert a["h.0.attn.c_proj.weight"].std() < 0.7 * a["h.0.attn.c_attn.weight"].std()


def test_dtypes_kept(tmp_path):
    folder = _folder(tmp_path, store_dtype="bfloat16")
    file = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    assert file.tensors["wte.weight"].dtype == "BF16" and file.tensors["ln_f.weight"].dtype == "F32"
    spec, specs = _specs()
    bf = load_weights(folder, specs, torch.bfloat16, "cpu", spec.file_prefixes, spec.ignored_weights)
    assert bf["wte.weight"].dtype == torch.bfloat16 and bf["h.0.mlp.c_fc.weight"].dtype == torch.bfloat16
    assert bf["ln_f.weight"].dtype == torch.float32 and bf["h.0.mlp.c_fc.bias"].dtype == torch.float32
    wide = load_weights(folder, specs, torch.float32, "cpu", spec.file_prefixes, spec.ignored_weights)
    assert wide["wte.weight"].dtype == torch.float32
    np.testing.assert_array_equal(wide["wte.weight"].numpy(), bf["wte.weight"].float().numpy())
    _, plain_tensors = plain.load_model(folder)
    np.testing.assert_array_equal(wide["wte.weight"].numpy(), plain_tensors["wte.weight"].astype(np.float32))


def test_bfloat16_rounding_matches_torch():
    x = np.random.default_rng(0).normal(size=4096).astype(np.float32)
    ours = float32_to_bfloat16_bits(x)
    theirs = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    np.testing.assert_array_equal(ours, theirs)
    np.testing.assert_array_equal(plain.round_to_bfloat16(x), torch.from_numpy(x).to(torch.bfloat16).float().numpy())


def test_prefixed_names_and_ignored_buffers(tmp_path):
    folder = _folder(tmp_path, file_prefix="transformer.")
    spec, specs = _specs()
    path = os.path.join(folder, "model.safetensors")
    stored = {n: np.asarray(t.bits) for n, t in SafetensorsFile(path).tensors.items()}
    stored["transformer.h.0.attn.bias"] = np.ones((1, 1, 4, 4), dtype=np.float32)
    stored["transformer.h.1.attn.masked_bias"] = np.float32(-1e4)
    stored["lm_head.weight"] = stored["transformer.wte.weight"]
    write_safetensors(path, stored)
    tensors = load_weights(folder, specs, torch.float32, "cpu", spec.file_prefixes, spec.ignored_weights)
    assert set(tensors) == set(specs)


def test_one_error_lists_everything(tmp_path):
    folder = _folder(tmp_path)
    spec, specs = _specs()
    path = os.path.join(folder, "model.safetensors")
    stored = {n: np.asarray(t.bits) for n, t in SafetensorsFile(path).tensors.items()}
    del stored["h.1.ln_2.bias"], stored["wpe.weight"]
    stored["h.0.attn.c_attn.weight"] = stored["h.0.attn.c_attn.weight"].T.copy()
    stored["h.7.mlp.c_fc.weight"] = np.zeros((2, 2), dtype=np.float32)
    stored["extra.scale"] = np.zeros(3, dtype=np.float32)
    stored["ln_f.weight"] = np.zeros(64, dtype=np.int32)
    stored["transformer.ln_f.bias"] = stored["ln_f.bias"]
    write_safetensors(path, stored)
    with pytest.raises(WeightsError) as error:
        load_weights(folder, specs, torch.float32, "cpu", spec.file_prefixes, spec.ignored_weights)
    e = error.value
    assert e.missing == ["h.1.ln_2.bias", "wpe.weight"]
    assert e.unexpected == ["extra.scale", "h.7.mlp.c_fc.weight"]
    assert e.wrong_shape == [("h.0.attn.c_attn.weight", (192, 64), (64, 192))]
    assert e.wrong_dtype == [("ln_f.weight", "I32", "F32, BF16 or F16")]
    assert e.duplicates and e.duplicates[0][0] == "ln_f.bias"
    text = str(e)
    for word in ("missing", "unexpected", "wrong shapes", "h.1.ln_2.bias", "extra.scale", "[192, 64]", "[64, 192]"):
        assert word in text


def test_untied_head_needs_its_tensor(tmp_path):
    raw = {**TINY_A, "tie_word_embeddings": False}
    folder = _folder(tmp_path, raw)
    spec, specs = _specs(raw)
    assert "lm_head.weight" in specs
    tensors = load_weights(folder, specs, torch.float32, "cpu", spec.file_prefixes, spec.ignored_weights)
    assert tensors["lm_head.weight"].shape == (512, 64)
    tied_spec, tied_specs = _specs(TINY_A)
    load_weights(folder, tied_specs, torch.float32, "cpu", tied_spec.file_prefixes, tied_spec.ignored_weights)
    tied_folder = write_random_model(config_from_dict(TINY_A), 3, str(tmp_path / "tied"))
    with pytest.raises(WeightsError) as error:
        load_weights(tied_folder, specs, torch.float32, "cpu", spec.file_prefixes, spec.ignored_weights)
    assert error.value.missing == ["lm_head.weight"]


def test_broken_files(tmp_path):
    folder = _folder(tmp_path)
    spec, specs = _specs()
    path = os.path.join(folder, "model.safetensors")
    data = open(path, "rb").read()
    open(path, "wb").write(data[:len(data) // 2])
    with pytest.raises(WeightsError) as error:
        load_weights(folder, specs, torch.float32, "cpu")
    assert "truncated" in str(error.value)
    open(path, "wb").write(b"\x05\x00\x00\x00\x00\x00\x00\x00{bad}")
    with pytest.raises(WeightsError):
        load_weights(folder, specs, torch.float32, "cpu")
    os.remove(path)
    with pytest.raises(WeightsError) as error:
        load_weights(folder, specs, torch.float32, "cpu")
    assert "cannot open" in str(error.value)
