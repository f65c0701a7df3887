"""Random-weights mode: fill every tensor a model declares from a seed and
write a model folder (``config.json`` + ``model.safetensors``).

The reference has no random model (its tests fill kernel inputs with
``rand()``, engine/tests/test_gpu_helpers.h:11-19); benchmarks and tests here
need whole models without downloaded weights.  Each tensor draws from its own
generator, keyed by the seed and the tensor's name, so a tensor's values do
not depend on which other tensors exist.

Recipes (by the ``init`` hint of each ``WeightSpec``):
  "gpt2"    matrices and tables N(0, 0.02); matrices that write into the
            residual stream N(0, 0.02 / sqrt(2 * layers)); biases 0; gains 1;
            shifts 0.
  "varied"  matrices and tables N(0, 0.05); biases N(0, 0.02); gains
            U(0.5, 1.5); shifts N(0, 0.1): nothing is trivially 0 or 1, so a
            forgotten bias or gain shows in the logits.
"""

from __future__ import annotations

import json
import math
import os
import zlib

import numpy as np

from ..config.registry import describe_model
from ..parts.base import build_part
from .loader import WEIGHTS_FILE, collect_specs
from .safetensors_io import write_safetensors

RECIPES = ("gpt2", "varied")


def model_parts(spec):
    """Every part of a model description, built (without weights)."""
    parts = [build_part(spec.embedding)]
    if spec.position is not None:
        parts.append(build_part(spec.position))
    for layer in spec.layers:
        parts.extend(build_part(p) for p in layer.parts.values())
    parts.append(build_part(spec.final_norm))
    parts.append(build_part(spec.head))
    return parts


def random_tensors(spec, seed: int, recipe: str = "gpt2") -> dict:
    """``{name: float32 numpy array}`` for every tensor the model declares."""
    if recipe not in RECIPES:
        raise ValueError(f"unknown init recipe '{recipe}' (known: {', '.join(RECIPES)})")
    n_layers = max(1, len(spec.layers))
    tensors = {}
    for name, w in collect_specs(model_parts(spec)).items():
        if w.optional and w.fallback is not None:
            continue
        rng = np.random.default_rng([int(seed) & 0xFFFFFFFF, zlib.crc32(name.encode("utf-8"))])
        shape = tuple(w.shape)
        if w.role == "int_table":
            tensors[name] = rng.integers(0, 2, size=shape, dtype=np.int32)
        elif recipe == "gpt2":
            if w.init in ("matrix", "table"):
                values = rng.normal(0.0, 0.02, size=shape)
            elif w.init == "residual_matrix":
                values = rng.normal(0.0, 0.02 / math.sqrt(2.0 * n_layers), size=shape)
            elif w.init == "gain":
                values = np.ones(shape)
            else:
                values = np.zeros(shape)
            tensors[name] = values.astype(np.float32)
        else:
            if w.init in ("matrix", "table", "residual_matrix"):
                values = rng.normal(0.0, 0.05, size=shape)
            elif w.init == "gain":
                values = rng.uniform(0.5, 1.5, size=shape)
            elif w.init == "shift":
                values = rng.normal(0.0, 0.1, size=shape)
            else:
                values = rng.normal(0.0, 0.02, size=shape)
            tensors[name] = values.astype(np.float32)
    return tensors


def write_random_model(config, seed: int, folder: str, recipe: str = "gpt2", store_dtype: str = "float32",
                       file_prefix: str = "") -> str:
    """Write ``folder/config.json`` and ``folder/model.safetensors``; returns ``folder``.

    store_dtype: "float32" or "bfloat16" (matrices and tables; vectors are
    always stored in 32-bit).  ``file_prefix`` is put before every tensor name
    (e.g. "transformer.").
    """
    if store_dtype not in ("float32", "bfloat16"):
        raise ValueError("store_dtype must be 'float32' or 'bfloat16'")
    spec = describe_model(config)
    tensors = random_tensors(spec, seed, recipe)
    specs = collect_specs(model_parts(spec))
    tags = {}
    named = {}
    for name, values in tensors.items():
        tags[file_prefix + name] = "BF16" if store_dtype == "bfloat16" and specs[name].role != "vector" else "F32"
        named[file_prefix + name] = values
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(config.to_dict(), handle, indent=2)
    write_safetensors(os.path.join(folder, WEIGHTS_FILE), named, tags,
                      metadata={"format": "pt", "seed": seed, "recipe": recipe})
    return folder
