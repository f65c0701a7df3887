"""Loading a model's tensors from ``model.safetensors`` by name.

What the parts declare (``WeightSpec``) is matched against what the file
holds.  Every disagreement is collected and reported in ONE error: tensors
that are missing, tensors the model does not know, wrong shapes, wrong
element types, and names that collide once a file-level prefix is dropped.
The reference reports per file (engine/src/tensor_loading.c:6-52 and the
layer index in engine/src/gpt2.c:145-149); it has no notion of an unexpected
tensor.

Element types on the device:
* matrix-product operands and tables: the engine's type (bfloat16 or float32),
  except a spec with ``keep_32bit`` whose stored tensor is 32-bit: that one
  stays 32-bit;
* vectors (norm gains and shifts, biases): float32 (a bfloat16 value widens
  exactly), since they enter 32-bit arithmetic only;
* integer tables: int32.
Matrices stored [in, out] are transposed once, on the device, to [out, in]
with ``in`` contiguous, the one layout every matrix kernel reads.
"""

from __future__ import annotations

import os
import re
import warnings

import numpy as np
import torch

from ..parts.spec import WeightSpec
from .safetensors_io import SafetensorsError, SafetensorsFile

WEIGHTS_FILE = "model.safetensors"


class WeightsError(ValueError):
    """The weights file and the model disagree.  The lists are also attributes."""

    def __init__(self, path, missing=(), unexpected=(), wrong_shape=(), wrong_dtype=(), duplicates=(), other=()):
        self.path = path
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)      # (name, stored shape, expected shape)
        self.wrong_dtype = list(wrong_dtype)      # (name, stored tag, expected kind)
        self.duplicates = list(duplicates)        # (name, [file names])
        self.other = list(other)
        lines = [f"weights in '{path}' do not fit the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shapes ({len(self.wrong_shape)}): " + "; ".join(
                f"{n}: stored {list(got)}, expected {list(want)}" for n, got, want in self.wrong_shape))
        if self.wrong_dtype:
            lines.append(f"  wrong element types ({len(self.wrong_dtype)}): " + "; ".join(
                f"{n}: stored {got}, expected {want}" for n, got, want in self.wrong_dtype))
        if self.duplicates:
            lines.append(f"  names that collide ({len(self.duplicates)}): " + "; ".join(
                f"{n} <- {', '.join(files)}" for n, files in self.duplicates))
        lines.extend(f"  {text}" for text in self.other)
        super().__init__("\n".join(lines))


def collect_specs(parts) -> dict[str, WeightSpec]:
    """All weight specs of ``parts`` by name.  Two parts may name the same
    tensor (a tied head) if they agree on its shape."""
    specs: dict[str, WeightSpec] = {}
    for part in parts:
        for spec in part.weight_specs():
            known = specs.get(spec.name)
            if known is None:
                specs[spec.name] = spec
            elif tuple(known.shape) != tuple(spec.shape) or known.transpose != spec.transpose:
                raise ValueError(f"two parts declare tensor '{spec.name}' differently: "
                                 f"{known.shape} and {spec.shape}")
    return specs


def _bits_to_torch(stored) -> torch.Tensor:
    """A CPU tensor over the mapped bytes (no copy)."""
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")          # the mapped file is read-only; it is only read
        tensor = torch.from_numpy(np.asarray(stored.bits))
    return tensor.view(torch.bfloat16) if stored.dtype == "BF16" else tensor


def device_dtype(spec: WeightSpec, stored_tag: str, engine_dtype: torch.dtype) -> torch.dtype:
    if spec.role == "int_table":
        return torch.int32
    if spec.role == "vector":
        return torch.float32
    if spec.keep_32bit and stored_tag == "F32":
        return torch.float32
    return engine_dtype


def match_names(file_names, specs: dict, prefixes=("",), ignored=()):
    """Map spec names to file names.  Returns (mapping, unexpected, duplicates)."""
    patterns = [re.compile(p) for p in ignored]
    ordered = sorted((p for p in prefixes if p), key=len, reverse=True)
    claimed: dict[str, list[str]] = {}
    unexpected = []
    for file_name in file_names:
        bare = file_name
        for prefix in ordered:
            if file_name.startswith(prefix):
                bare = file_name[len(prefix):]
                break
        if bare in specs:
            claimed.setdefault(bare, []).append(file_name)
        elif file_name in specs:
            claimed.setdefault(file_name, []).append(file_name)
        elif any(p.fullmatch(bare) or p.fullmatch(file_name) for p in patterns):
            continue
        else:
            unexpected.append(file_name)
    duplicates = [(name, files) for name, files in claimed.items() if len(files) > 1]
    mapping = {name: files[0] for name, files in claimed.items()}
    return mapping, unexpected, duplicates


def load_weights(model_dir: str, specs: dict, engine_dtype: torch.dtype, device, prefixes=("",), ignored=()):
    """Read, check and upload.  Returns ``{spec name: device tensor}``."""
    path = os.path.join(model_dir, WEIGHTS_FILE)
    try:
        file = SafetensorsFile(path)
    except SafetensorsError as error:
        raise WeightsError(path, other=[str(error)]) from None
    mapping, unexpected, duplicates = match_names(file.names(), specs, prefixes, ignored)
    missing, wrong_shape, wrong_dtype = [], [], []
    for name, spec in specs.items():
        if name not in mapping:
            if not spec.optional:
                missing.append(name)
            continue
        stored = file.tensors[mapping[name]]
        if tuple(stored.shape) != tuple(spec.shape):
            wrong_shape.append((name, stored.shape, spec.shape))
        if spec.role == "int_table":
            if stored.dtype not in ("I64", "I32", "I16", "I8", "U8"):
                wrong_dtype.append((name, stored.dtype, "an integer type"))
        elif stored.dtype not in ("F32", "BF16", "F16"):
            wrong_dtype.append((name, stored.dtype, "F32, BF16 or F16"))
    if missing or unexpected or wrong_shape or wrong_dtype or duplicates:
        raise WeightsError(path, sorted(missing), sorted(unexpected), wrong_shape, wrong_dtype, duplicates)

    tensors = {}
    for name, spec in specs.items():
        if name not in mapping:
            continue
        stored = file.tensors[mapping[name]]
        target = device_dtype(spec, stored.dtype, engine_dtype)
        tensor = _bits_to_torch(stored).to(device=device).to(dtype=target)
        if spec.transpose:
            tensor = tensor.t()
        tensors[name] = tensor.contiguous()
    for name, spec in specs.items():
        if name not in tensors and spec.optional and spec.fallback is not None:
            tensors[name] = tensors[spec.fallback]
    return tensors
