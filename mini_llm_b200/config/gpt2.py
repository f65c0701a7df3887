"""Configuration of the GPT-2 architecture (``GPT2LMHeadModel``).

The reference engine fixes these sizes at compile time
(engine/include/gpt2.h:12-19) and hard-codes the norm's epsilon
(engine/src/gpt2_gpu.cu:15); here every one of them is read from the keys of
the architecture's own ``config.json``.  Sizes have no default: a model folder
must state them.
"""

from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ModelConfig

# Names of the activation functions a GPT-2 config.json may give, mapped to
# the two formulas the feed-forward kernels implement.
ACTIVATIONS = {
    "gelu_new": "gelu_tanh",
    "gelu_pytorch_tanh": "gelu_tanh",
    "gelu_fast": "gelu_tanh",
    "gelu": "gelu_erf",
}

_REQUIRED = ("n_layer", "n_embd", "n_head", "vocab_size", "n_positions")


@dataclass(frozen=True)
class Gpt2Config(ModelConfig):
    n_layer: int = field(default=0, metadata={"kind": int})
    n_embd: int = field(default=0, metadata={"kind": int})
    n_head: int = field(default=0, metadata={"kind": int})
    n_inner: int = field(default=0, metadata={"kind": int})          # 0 / null: 4 * n_embd
    vocab_size: int = field(default=0, metadata={"kind": int})
    n_positions: int = field(default=0, metadata={"kind": int})
    layer_norm_epsilon: float = field(default=1e-5, metadata={"kind": float})
    activation_function: str = field(default="gelu_new", metadata={"kind": str})
    scale_attn_weights: bool = field(default=True, metadata={"kind": bool})
    scale_attn_by_inverse_layer_idx: bool = field(default=False, metadata={"kind": bool})
    tie_word_embeddings: bool = field(default=True, metadata={"kind": bool})
    eos_token_id: int = field(default=-1, metadata={"kind": int})    # -1: none
    bos_token_id: int = field(default=-1, metadata={"kind": int})

    ALIASES = {"n_ctx": "n_positions", "num_hidden_layers": "n_layer",
               "hidden_size": "n_embd", "num_attention_heads": "n_head",
               "max_position_embeddings": "n_positions"}

    def __post_init__(self):
        for key in _REQUIRED:
            if getattr(self, key) <= 0:
                raise ConfigError(f"config key '{key}' is required and must be positive, got {getattr(self, key)}")
        if self.n_inner < 0:
            raise ConfigError(f"config key 'n_inner' must not be negative, got {self.n_inner}")
        if self.n_inner == 0:
            object.__setattr__(self, "n_inner", 4 * self.n_embd)
        if self.n_embd % self.n_head != 0:
            raise ConfigError(
                f"config key 'n_embd' ({self.n_embd}) is not a multiple of 'n_head' ({self.n_head})")
        if not self.layer_norm_epsilon > 0.0:
            raise ConfigError(f"config key 'layer_norm_epsilon' must be positive, got {self.layer_norm_epsilon}")
        if self.activation_function not in ACTIVATIONS:
            known = ", ".join(sorted(ACTIVATIONS))
            raise ConfigError(
                f"config key 'activation_function': unknown activation '{self.activation_function}' (known: {known})")
        for key in ("eos_token_id", "bos_token_id"):
            if getattr(self, key) >= self.vocab_size:
                raise ConfigError(f"config key '{key}' ({getattr(self, key)}) is outside the vocabulary ({self.vocab_size})")

    @property
    def head_size(self) -> int:
        return self.n_embd // self.n_head

    @property
    def activation(self) -> str:
        return ACTIVATIONS[self.activation_function]

    def to_dict(self) -> dict:
        out = super().to_dict()
        out["model_type"] = "gpt2"
        for key in ("eos_token_id", "bos_token_id"):
            if out[key] < 0:
                out[key] = None
        return out
