"""GPT-2 (``GPT2LMHeadModel``) as a model description.

The dense pre-norm decoder the reference runs (engine/src/gpt2_gpu.cu:220-265,
engine/src/transformer_block.c:49-71): learned absolute positions, one fused
q/k/v projection per layer stored [in, out], a gelu feed-forward, a final
norm, and a head tied to the token table.  Tensor names are those of the
reference's weight export (engine/src/gpt2.c:45-108,131-137), with or without
the ``transformer.`` prefix.
"""

from __future__ import annotations

import math

from ..config.gpt2 import Gpt2Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def describe(config: Gpt2Config) -> ModelSpec:
    width, heads, head_size = config.n_embd, config.n_head, config.head_size
    layers = []
    for index in range(config.n_layer):
        # Scores are scaled by 1/sqrt(head size) (engine/src/attention.c:33) when
        # scale_attn_weights is set, and also by 1/(layer index + 1) when
        # scale_attn_by_inverse_layer_idx is.
        scale = 1.0
        if config.scale_attn_weights:
            scale /= math.sqrt(head_size)
        if config.scale_attn_by_inverse_layer_idx:
            scale /= float(index + 1)
        prefix = f"h.{index}"
        layers.append(LayerSpec("pre_norm", {
            "norm_1": PartSpec("layer_norm", f"{prefix}.ln_1", {"width": width, "eps": config.layer_norm_epsilon}),
            "mixer": PartSpec("causal_self_attention", f"{prefix}.attn",
                              {"width": width, "n_heads": heads, "head_size": head_size, "score_scale": scale}),
            "norm_2": PartSpec("layer_norm", f"{prefix}.ln_2", {"width": width, "eps": config.layer_norm_epsilon}),
            "feed_forward": PartSpec("dense_mlp", f"{prefix}.mlp",
                                     {"width": width, "inner": config.n_inner, "activation": config.activation}),
        }))
    tied = config.tie_word_embeddings
    ignored = [r"h\.\d+\.attn\.bias", r"h\.\d+\.attn\.masked_bias"]
    if tied:
        ignored.append(r"lm_head\.weight")
    return ModelSpec(
        hidden_size=width,
        vocab_size=config.vocab_size,
        max_positions=config.n_positions,
        embedding=PartSpec("token_embedding", "", {"vocab_size": config.vocab_size, "width": width}),
        position=PartSpec("learned_positions", "", {"max_positions": config.n_positions, "width": width}),
        layers=tuple(layers),
        order=tuple(RunEntry(i) for i in range(config.n_layer)),
        final_norm=PartSpec("layer_norm", "ln_f", {"width": width, "eps": config.layer_norm_epsilon}),
        head=PartSpec("linear_head", "", {"vocab_size": config.vocab_size, "width": width,
                                          "weight_name": "wte.weight" if tied else "lm_head.weight"}),
        file_prefixes=("", "transformer."),
        ignored_weights=tuple(ignored),
        eos_token_id=config.eos_token_id if config.eos_token_id >= 0 else None,
    )


register_architecture("GPT2LMHeadModel", Gpt2Config, describe, aliases=("model_type:gpt2",))
