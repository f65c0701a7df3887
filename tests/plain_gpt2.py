"""A plain, slow GPT-2 in numpy: whole sequences, no cache, one function per part.

It is the yardstick of the tests and shares no code with ``mini_llm_b200``: it
has its own reader of the weights file, its own formulas and its own sampler.
Each function is written from the formula of the reference's CPU operator it
cites (paths within WillyBruhn/mini_llm).  ``tests/golden/`` holds the outputs
of the reference's own compiled CPU code on a tiny random model, and
``tests/test_plain_against_reference.py`` compares this file with them.

All arithmetic runs in ``dtype`` (float64 by default, so that differences
between an engine and this file are the engine's rounding, not this file's).
"""

from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ---- reading a model folder ------------------------------------------------------------------

def read_safetensors(path):
    """{name: float64/int64 numpy array} of a safetensors file (F32, BF16, F16, I32, I64)."""
    with open(path, "rb") as handle:
        data = handle.read()
    (header_len,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + header_len])
    base = 8 + header_len
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        raw = data[base + begin:base + end]
        tag = info["dtype"]
        if tag == "F32":
            values = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif tag == "F16":
            values = np.frombuffer(raw, dtype="<f2").astype(np.float64)
        elif tag == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            values = bits.view(np.float32).astype(np.float64)
        elif tag == "I32":
            values = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        elif tag == "I64":
            values = np.frombuffer(raw, dtype="<i8").astype(np.int64)
        else:
            raise ValueError(f"{name}: dtype {tag} not handled by the plain reader")
        out[name] = values.reshape(info["shape"])
    return out


def round_to_bfloat16(values):
    """Round to the nearest bfloat16 (ties to even), returned in the input's dtype."""
    as32 = np.asarray(values, dtype=np.float32)
    bits = as32.view(np.uint32)
    rounded = (bits + (0x7FFF + ((bits >> 16) & 1))) & np.uint32(0xFFFF0000)
    return rounded.view(np.float32).astype(np.asarray(values).dtype)


def load_model(folder, round_matrices_to_bfloat16=False):
    """(config dict, {name without 'transformer.' prefix: array})."""
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    tensors = {}
    for name, values in read_safetensors(os.path.join(folder, "model.safetensors")).items():
        if name.startswith("transformer."):
            name = name[len("transformer."):]
        if round_matrices_to_bfloat16 and values.ndim == 2:
            values = round_to_bfloat16(values)
        tensors[name] = values
    return config, tensors


# ---- the parts -------------------------------------------------------------------------------

def embed(token_ids, wte, wpe, first_position=0):
    """hidden[t] = wte[id_t] + wpe[first_position + t]   (engine/src/embedding.c:9-15;
    offset for cached tokens: engine/src/embedding.cu:21-26)."""
    token_ids = np.asarray(token_ids)
    positions = first_position + np.arange(len(token_ids))
    return wte[token_ids] + wpe[positions]


def layer_norm(x, gain, shift, eps):
    """mean; biased variance of the centred values; (x - mean) * (1 / sqrt(var + eps)) * gain
    + shift   (engine/src/layernorm.c:12-33)."""
    mean = x.sum(axis=-1, keepdims=True) / x.shape[-1]
    centred = x - mean
    variance = (centred * centred).sum(axis=-1, keepdims=True) / x.shape[-1]
    inverse = 1.0 / np.sqrt(variance + eps)
    return centred * inverse * gain + shift


def linear(x, weight_in_out, bias):
    """out = x W + b with W stored [in, out]; the bias is added after the full sum
    (engine/src/linear.c:5-19)."""
    return x @ weight_in_out + bias


def gelu_tanh(u):
    """0.5 u (1 + tanh(0.7978845608 (u + 0.044715 u^3)))   (engine/src/gelu.c:11-19,
    engine/include/gelu_math.h:6-11)."""
    return 0.5 * u * (1.0 + np.tanh(0.7978845608 * (u + 0.044715 * u * u * u)))


def gelu_erf(u):
    """0.5 u (1 + erf(u / sqrt(2)))   (engine/src/gelu.c:5-9)."""
    erf = np.vectorize(math.erf, otypes=[np.float64])
    return (0.5 * u * (1.0 + erf(np.asarray(u, dtype=np.float64) / math.sqrt(2.0)))).astype(u.dtype)


ACTIVATIONS = {"gelu_new": gelu_tanh, "gelu_pytorch_tanh": gelu_tanh, "gelu_fast": gelu_tanh, "gelu": gelu_erf}


def causal_softmax(scores):
    """Row i keeps columns 0..i: subtract the row maximum over those, exponentiate, divide by
    the sum; the other columns are 0   (engine/src/softmax.c:29-55)."""
    n = scores.shape[-1]
    keep = np.tril(np.ones((scores.shape[-2], n), dtype=bool), k=n - scores.shape[-2])
    masked = np.where(keep, scores, -np.inf)
    top = masked.max(axis=-1, keepdims=True)
    weights = np.where(keep, np.exp(masked - top), 0.0)
    return weights / weights.sum(axis=-1, keepdims=True)


def attention_head(q, k, v, scale, window=None):
    """scores = (q k^T) * scale, causal softmax, weights @ v   (engine/src/attention.c:24-49;
    the reference's scale is 1/sqrt(head size), engine/src/attention.c:33).  ``window``: a
    query at position i sees only keys i-window+1..i (no counterpart in the reference)."""
    scores = (q @ k.T) * scale
    if window is not None:
        n = scores.shape[0]
        i, j = np.meshgrid(np.arange(n), np.arange(n), indexing="ij")
        scores = np.where(j > i - window, scores, -np.inf)
    return causal_softmax(scores) @ v


def multi_head_attention(q, k, v, n_heads, scale, n_kv_heads=None, window=None):
    """Head h is columns h*D..h*D+D-1 of q, k, v and of the output
    (engine/src/attention.c:78-97)."""
    n_kv_heads = n_kv_heads or n_heads
    head = q.shape[1] // n_heads
    out = np.empty_like(q)
    for h in range(n_heads):
        g = h // (n_heads // n_kv_heads)
        out[:, h * head:(h + 1) * head] = attention_head(q[:, h * head:(h + 1) * head], k[:, g * head:(g + 1) * head],
                                                         v[:, g * head:(g + 1) * head], scale, window)
    return out


def score_scale(config, layer_index):
    """1/sqrt(head size) as in the reference (engine/src/attention.c:33) when
    ``scale_attn_weights`` (default true); times 1/(layer index + 1) when
    ``scale_attn_by_inverse_layer_idx`` (the reference has no such option: this is the meaning
    of GPT-2's configuration key)."""
    scale = 1.0
    if config.get("scale_attn_weights", True):
        scale /= math.sqrt(config["n_embd"] // config["n_head"])
    if config.get("scale_attn_by_inverse_layer_idx", False):
        scale /= layer_index + 1
    return scale


def block(x, tensors, config, layer_index, record=None):
    """r = x + proj(attention(ln_1(x))); out = r + mlp(ln_2(r))
    (engine/src/transformer_block.c:49-71).  ``record``: a dict that receives the layer's
    keys and values (what a cache would hold: engine/tests/test_gpt2_gpu.c:96-150 compares
    the stored rows with the CPU's norm + linear)."""
    p = f"h.{layer_index}."
    eps = config.get("layer_norm_epsilon", 1e-5)
    width = config["n_embd"]
    ln1 = layer_norm(x, tensors[p + "ln_1.weight"], tensors[p + "ln_1.bias"], eps)
    qkv = linear(ln1, tensors[p + "attn.c_attn.weight"], tensors[p + "attn.c_attn.bias"])
    # The fused matrix holds q, k, v as three column blocks (engine/src/gpt2.c:79-90).
    q, k, v = qkv[:, :width], qkv[:, width:2 * width], qkv[:, 2 * width:]
    if record is not None:
        record["k"], record["v"] = k, v
    mixed = multi_head_attention(q, k, v, config["n_head"], score_scale(config, layer_index))
    r = x + linear(mixed, tensors[p + "attn.c_proj.weight"], tensors[p + "attn.c_proj.bias"])
    ln2 = layer_norm(r, tensors[p + "ln_2.weight"], tensors[p + "ln_2.bias"], eps)
    up = linear(ln2, tensors[p + "mlp.c_fc.weight"], tensors[p + "mlp.c_fc.bias"])
    act = ACTIVATIONS[config.get("activation_function", "gelu_new")](up)
    return r + linear(act, tensors[p + "mlp.c_proj.weight"], tensors[p + "mlp.c_proj.bias"])


def forward(config, tensors, token_ids, dtype=np.float64, return_blocks=False, records=None):
    """Logits [len, vocab] of a whole sequence: embed, every block, final norm, then the dot
    with every row of the token table, no bias   (engine/src/gpt2.c:198-256).  With
    ``return_blocks`` also the residual stream after the embedding and after every block;
    ``records``: a list that receives one dict of keys and values per layer."""
    t = {k: (v.astype(dtype) if v.dtype.kind == "f" else v) for k, v in tensors.items()}
    hidden = embed(token_ids, t["wte.weight"], t["wpe.weight"])
    blocks = [hidden]
    for layer in range(config["n_layer"]):
        record = {} if records is not None else None
        hidden = block(hidden, t, config, layer, record)
        blocks.append(hidden)
        if records is not None:
            records.append(record)
    normed = layer_norm(hidden, t["ln_f.weight"], t["ln_f.bias"], config.get("layer_norm_epsilon", 1e-5))
    head = t["wte.weight"] if config.get("tie_word_embeddings", True) else t["lm_head.weight"]
    logits = normed @ head.T
    return (logits, blocks) if return_blocks else logits


# ---- sampling --------------------------------------------------------------------------------

def argmax_first(values):
    """First index of the maximum; a NaN beats every number and the first NaN wins
    (engine/include/argmax.h:10-13, engine/src/argmax.cu:8-18)."""
    values = np.asarray(values)
    nans = np.flatnonzero(np.isnan(values))
    if nans.size:
        return int(nans[0])
    return int(np.argmax(values))


_M64 = (1 << 64) - 1


def _mix64(z):
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def uniform_of(seed, counter, index):
    """The engine's stated draw: a 24-bit uniform in (0, 1) from a hash of (seed, counter,
    index).  Sampling has no counterpart in the reference's engine (greedy only); its command
    line samples through another library (scripts/complete.py:116-123)."""
    h = _mix64(_mix64((seed ^ (counter << 32)) & _M64) ^ index)
    return ((h >> 40) + 0.5) / 16777216.0


def sample(logits, temperature, top_p=1.0, seed=0, counter=0, return_margin=False):
    """Greedy for temperature <= 0 (scripts/complete.py:116-123); else Gumbel-max over the
    nucleus: the smallest set of most probable tokens whose probability reaches top_p (ties at
    its edge included), argmax of logit/T - log(-log(u))."""
    logits = np.asarray(logits, dtype=np.float64)
    if not temperature > 0:
        choice = argmax_first(logits)
        return (choice, np.inf) if return_margin else choice
    scaled = logits / np.float64(np.float32(temperature))
    keep = np.ones(len(logits), dtype=bool)
    if top_p < 1.0:
        p = np.exp(scaled - scaled.max())
        p /= p.sum()
        order = np.argsort(-p, kind="stable")
        cumulative = np.cumsum(p[order])
        k = int(np.searchsorted(cumulative, np.float64(np.float32(top_p)), side="left"))
        k = min(k, len(p) - 1)
        keep = p >= p[order[k]]
    u = np.array([uniform_of(seed, counter, v) for v in range(len(logits))])
    scores = np.where(keep, scaled - np.log(-np.log(u)), -np.inf)
    choice = int(np.argmax(scores))
    if return_margin:
        rest = np.delete(scores, choice)
        return choice, float(scores[choice] - rest.max()) if rest.size else np.inf
    return choice


def generate(config, tensors, prompt, n_new, temperature=0.0, top_p=1.0, seed=0, dtype=np.float64):
    """Whole-sequence recomputation for every new token; returns (tokens, margins)."""
    tokens = list(prompt)
    out, margins = [], []
    for step in range(n_new):
        logits = forward(config, tensors, tokens, dtype=dtype)[-1]
        if temperature > 0:
            choice, margin = sample(logits, temperature, top_p, seed, step, return_margin=True)
        else:
            choice = argmax_first(logits)
            ordered = np.sort(logits)
            margin = float(ordered[-1] - ordered[-2])
        out.append(choice)
        margins.append(margin)
        tokens.append(choice)
    return out, margins
