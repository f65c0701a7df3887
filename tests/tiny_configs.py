"""The tests' own small configurations of the architecture.  A and B differ in every size and
option: head count and head size, width, inner size (B's is not 4x), vocabulary (B's is no
multiple of 8), positions, layers, the norms' eps, the activation, and the score scale rule."""

TINY_A = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 64, "n_head": 4, "n_inner": 256, "vocab_size": 512, "n_positions": 128,
    "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5,
    "scale_attn_by_inverse_layer_idx": False, "tie_word_embeddings": True,
}

TINY_B = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 3, "n_embd": 96, "n_head": 2, "n_inner": 160, "vocab_size": 1000, "n_positions": 64,
    "activation_function": "gelu", "layer_norm_epsilon": 1e-6,
    "scale_attn_by_inverse_layer_idx": True, "tie_word_embeddings": True,
}

# Larger than the two above where a test needs hundreds of keys: 5 heads of 32, a width and
# a vocabulary that are no power of two.
TINY_C = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 160, "n_head": 5, "n_inner": 416, "vocab_size": 777, "n_positions": 640,
    "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5,
    "scale_attn_by_inverse_layer_idx": False, "tie_word_embeddings": True,
}

# Head size 64, the head size of every published GPT-2 size, so that the kernels the
# benchmark runs (tensor-core prompt attention, the one-kernel decode step at head size 64,
# split-key decode attention) meet every way of cutting the work; a vocabulary that is odd;
# requests of up to 700 tokens (six blocks of 128 keys, eleven pages of 64).
TINY_D = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 256, "n_head": 4, "n_inner": 1024, "vocab_size": 1031, "n_positions": 704,
    "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5,
    "scale_attn_by_inverse_layer_idx": False, "tie_word_embeddings": True,
}

# The layer sizes of GPT-2 small (width 768, 12 heads of 64, inner size 3072, vocabulary 50257,
# 1024 positions) with two layers instead of twelve: what one layer computes is what every
# layer computes, and the plain implementation stays within seconds.
SMALL_WIDTHS = {
    "architectures": ["GPT2LMHeadModel"], "model_type": "gpt2",
    "n_layer": 2, "n_embd": 768, "n_head": 12, "n_inner": 3072, "vocab_size": 50257, "n_positions": 1024,
    "activation_function": "gelu_new", "layer_norm_epsilon": 1e-5,
    "scale_attn_by_inverse_layer_idx": False, "tie_word_embeddings": True,
}

RECIPES = {"A": ("gpt2", 0), "B": ("varied", 1), "C": ("varied", 2), "D": ("varied", 3)}
