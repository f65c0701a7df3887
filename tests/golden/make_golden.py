#!/usr/bin/env python3
"""Makes ``reference_tiny.npz``: outputs of the reference's OWN compiled CPU code on a tiny
random GPT-2, for ``tests/test_plain_against_reference.py``.

    python tests/golden/make_golden.py /path/to/mini_llm

It compiles the reference's ``engine/src/*.c`` (unchanged, read from the given checkout) with
gcc into a shared library in a temporary folder and calls, through ctypes:
``embed_tokens`` (engine/src/embedding.c), ``transformer_block_forward``
(engine/src/transformer_block.c:11-93) once per layer with the fused ``c_attn`` matrix split
into q, k, v the reference's way (engine/src/gpt2.c:79-90), ``layernorm``
(engine/src/layernorm.c) for the final norm, ``gelu`` (the erf form, engine/src/gelu.c:5-9), and
``multi_head_attention`` (engine/src/attention.c:78-97) at head size 48, once as it is and once
with the queries divided by 3 (the score scale of a third layer under
``scale_attn_by_inverse_layer_idx``).
``gpt2_forward`` itself is compiled for GPT-2 small's sizes only (engine/include/gpt2.h:12-19),
so its last lines, the dot of the normed rows with the token table
(engine/src/gpt2.c:245-256), are restated here in float32.

The file holds the tiny model's config, its float32 weights (HF names, ``c_attn`` fused,
[in, out] layout), the token ids and the reference's outputs.
"""

import ctypes
import glob
import os
import subprocess
import sys
import tempfile

import numpy as np

CONFIG = {"architectures": ["GPT2LMHeadModel"], "model_type": "gpt2", "n_layer": 2, "n_embd": 32, "n_head": 2,
          "n_inner": 80, "vocab_size": 96, "n_positions": 24, "layer_norm_epsilon": 1e-5,
          "activation_function": "gelu_new"}
TOKENS = 19
F = ctypes.POINTER(ctypes.c_float)


class BlockWeights(ctypes.Structure):
    # engine/include/transformer_block.h:12-29
    _fields_ = [(n, F) for n in ("ln1_gamma", "ln1_beta", "query_weights", "query_bias", "key_weights", "key_bias",
                                 "value_weights", "value_bias", "attention_weights", "attention_bias", "ln2_gamma",
                                 "ln2_beta", "mlp_up_weights", "mlp_up_bias", "mlp_down_weights", "mlp_down_bias")]


def ptr(a):
    return a.ctypes.data_as(F)


def main(reference):
    build = tempfile.mkdtemp(prefix="mini_llm_ref_")
    lib_path = os.path.join(build, "libref_cpu.so")
    sources = sorted(glob.glob(os.path.join(reference, "engine", "src", "*.c")))
    subprocess.run(["gcc", "-O2", "-std=c11", "-shared", "-fPIC", "-I", os.path.join(reference, "engine", "include"),
                    "-o", lib_path, *sources, "-lm"], check=True)
    lib = ctypes.CDLL(lib_path)

    rng = np.random.default_rng(20240229)
    c = CONFIG
    E, I, V, P, L = c["n_embd"], c["n_inner"], c["vocab_size"], c["n_positions"], c["n_layer"]
    w = {"wte.weight": rng.normal(0, 0.3, (V, E)), "wpe.weight": rng.normal(0, 0.1, (P, E)),
         "ln_f.weight": rng.uniform(0.5, 1.5, E), "ln_f.bias": rng.normal(0, 0.1, E)}
    for i in range(L):
        p = f"h.{i}."
        w[p + "ln_1.weight"] = rng.uniform(0.5, 1.5, E)
        w[p + "ln_1.bias"] = rng.normal(0, 0.1, E)
        w[p + "attn.c_attn.weight"] = rng.normal(0, 0.15, (E, 3 * E))
        w[p + "attn.c_attn.bias"] = rng.normal(0, 0.05, 3 * E)
        w[p + "attn.c_proj.weight"] = rng.normal(0, 0.15, (E, E))
        w[p + "attn.c_proj.bias"] = rng.normal(0, 0.05, E)
        w[p + "ln_2.weight"] = rng.uniform(0.5, 1.5, E)
        w[p + "ln_2.bias"] = rng.normal(0, 0.1, E)
        w[p + "mlp.c_fc.weight"] = rng.normal(0, 0.15, (E, I))
        w[p + "mlp.c_fc.bias"] = rng.normal(0, 0.05, I)
        w[p + "mlp.c_proj.weight"] = rng.normal(0, 0.15, (I, E))
        w[p + "mlp.c_proj.bias"] = rng.normal(0, 0.05, E)
    w = {k: np.ascontiguousarray(v, dtype=np.float32) for k, v in w.items()}
    tokens = rng.integers(0, V, TOKENS).astype(np.int32)

    hidden = np.zeros((TOKENS, E), dtype=np.float32)
    lib.embed_tokens.argtypes = [F, ctypes.POINTER(ctypes.c_int), F, F, ctypes.c_size_t, ctypes.c_size_t]
    lib.embed_tokens(ptr(hidden), tokens.ctypes.data_as(ctypes.POINTER(ctypes.c_int)), ptr(w["wte.weight"]),
                     ptr(w["wpe.weight"]), ctypes.c_size_t(TOKENS), ctypes.c_size_t(E))
    out = {"embedded": hidden.copy()}
    lib.transformer_block_forward.argtypes = [F, F, ctypes.POINTER(BlockWeights), ctypes.c_size_t, ctypes.c_size_t,
                                              ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float]
    for i in range(L):
        p = f"h.{i}."
        fused, bias = w[p + "attn.c_attn.weight"], w[p + "attn.c_attn.bias"]
        keep = [np.ascontiguousarray(fused[:, j * E:(j + 1) * E]) for j in range(3)]
        keep += [np.ascontiguousarray(bias[j * E:(j + 1) * E]) for j in range(3)]
        bw = BlockWeights(ptr(w[p + "ln_1.weight"]), ptr(w[p + "ln_1.bias"]), ptr(keep[0]), ptr(keep[3]),
                          ptr(keep[1]), ptr(keep[4]), ptr(keep[2]), ptr(keep[5]), ptr(w[p + "attn.c_proj.weight"]),
                          ptr(w[p + "attn.c_proj.bias"]), ptr(w[p + "ln_2.weight"]), ptr(w[p + "ln_2.bias"]),
                          ptr(w[p + "mlp.c_fc.weight"]), ptr(w[p + "mlp.c_fc.bias"]), ptr(w[p + "mlp.c_proj.weight"]),
                          ptr(w[p + "mlp.c_proj.bias"]))
        nxt = np.zeros_like(hidden)
        lib.transformer_block_forward(ptr(hidden), ptr(nxt), ctypes.byref(bw), TOKENS, E, c["n_head"], I,
                                      ctypes.c_float(c["layer_norm_epsilon"]))
        hidden = nxt
        out[f"block_{i}"] = hidden.copy()
    lib.layernorm.argtypes = [F, F, F, F, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_float]
    normed = np.zeros_like(hidden)
    lib.layernorm(ptr(normed), ptr(hidden), ptr(w["ln_f.weight"]), ptr(w["ln_f.bias"]), TOKENS, E,
                  ctypes.c_float(c["layer_norm_epsilon"]))
    out["final_norm"] = normed
    out["logits"] = (normed @ w["wte.weight"].T).astype(np.float32)     # engine/src/gpt2.c:245-256, restated

    # single operators with the options the whole model above does not use
    x = rng.normal(0, 2.0, 257).astype(np.float32)
    erf_out = np.zeros_like(x)
    lib.gelu.argtypes = [F, F, ctypes.c_size_t]
    lib.gelu(ptr(erf_out), ptr(x.copy()), x.size)
    out["gelu_erf_in"], out["gelu_erf_out"] = x, erf_out
    rows = rng.normal(1.0, 3.0, (5, 48)).astype(np.float32)
    g, b = rng.uniform(0.5, 1.5, 48).astype(np.float32), rng.normal(0, 0.1, 48).astype(np.float32)
    ln_out = np.zeros_like(rows)
    lib.layernorm(ptr(ln_out), ptr(rows), ptr(g), ptr(b), 5, 48, ctypes.c_float(1e-6))
    out.update(ln_in=rows, ln_gain=g, ln_shift=b, ln_out=ln_out)
    q, k, v = (rng.normal(0, 1.0, (11, 96)).astype(np.float32) for _ in range(3))
    att = np.zeros_like(q)
    lib.multi_head_attention.argtypes = [F, F, F, F, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t]
    lib.multi_head_attention(ptr(q), ptr(k), ptr(v), ptr(att), 11, 2, 48)
    out.update(att_q=q, att_k=k, att_v=v, att_out=att)
    # GPT-2's option scale_attn_by_inverse_layer_idx multiplies the scores of layer l (0-based)
    # by 1/(l + 1).  The reference has no such option, but the scores are linear in the
    # queries, so its own attention fed q/(l + 1) computes exactly that (here l = 2).
    q_third = np.ascontiguousarray(q / np.float32(3.0))
    att_third = np.zeros_like(q)
    lib.multi_head_attention(ptr(q_third), ptr(k), ptr(v), ptr(att_third), 11, 2, 48)
    out.update(att_out_layer_2=att_third)

    here = os.path.dirname(os.path.abspath(__file__))
    np.savez_compressed(os.path.join(here, "reference_tiny.npz"), tokens=tokens,
                        config=np.array(__import__("json").dumps(CONFIG)),
                        **{"w:" + k: v for k, v in w.items()}, **out)
    print("wrote", os.path.join(here, "reference_tiny.npz"))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py /path/to/mini_llm")
    main(sys.argv[1])
