"""The description of a model as data: parts, layers, and the run order.

An architecture's ``describe(config)`` returns a ``ModelSpec``.  Everything
that builds, loads or runs a model reads this description; none of it knows
an architecture by name.  The reference fixes one sequence of function calls
per block (engine/src/transformer_block.cu:139-203); here the block is a
record of parts chosen per layer, and the order in which layers run is a list.
"""

from __future__ import annotations

from dataclasses import dataclass, field


@dataclass(frozen=True)
class WeightSpec:
    """One tensor a part needs from the weights file.

    name       name in the file (without any file-level prefix)
    shape      shape as stored in the file
    role       "matrix" (a matrix-product operand), "table" (rows gathered by
               index, may also be a product operand), "vector" (gain, shift,
               bias: kept in 32-bit), "int_table" (kept as int32)
    transpose  the file stores [in, out]; the device copy is [out, in]
    init       how random-weights mode fills it: "matrix", "residual_matrix",
               "table", "bias", "gain", "shift"
    optional   may be absent from the file (``fallback`` names the tensor used instead)
    keep_32bit a float tensor stored in 32-bit stays 32-bit in every mode
    """

    name: str
    shape: tuple
    role: str = "matrix"
    transpose: bool = False
    init: str = "matrix"
    optional: bool = False
    fallback: str | None = None
    keep_32bit: bool = False


@dataclass(frozen=True)
class PartSpec:
    """A part: its registered kind, its weight-name prefix and its parameters."""

    kind: str
    prefix: str = ""
    params: dict = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, self.prefix, tuple(sorted((k, repr(v)) for k, v in self.params.items()))))


@dataclass(frozen=True)
class LayerSpec:
    """One layer: an arrangement (how its parts are wired) and its parts by role."""

    arrangement: str
    parts: dict          # role -> PartSpec, roles are defined by the arrangement

    def __hash__(self):
        return hash((self.arrangement, tuple(sorted(self.parts.items(), key=lambda kv: kv[0]))))


@dataclass(frozen=True)
class RunEntry:
    """One entry of the run order.

    layer     index into ``ModelSpec.layers``; a layer may be named more than once
    cache_of  None: this entry has a cache of its own.  k: it reads the cache
              that run entry k (an earlier one) writes, and writes none.
    """

    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int | None          # None: no architectural limit on positions
    embedding: PartSpec
    position: PartSpec | None          # position encoding applied to the embedded tokens, if any
    layers: tuple                      # of LayerSpec
    order: tuple                       # of RunEntry
    final_norm: PartSpec
    head: PartSpec
    file_prefixes: tuple = ("",)       # prefixes a weights file may put before every name
    ignored_weights: tuple = ()        # regular expressions of file names that are no parameters
    eos_token_id: int | None = None

    def __post_init__(self):
        for index, entry in enumerate(self.order):
            if not 0 <= entry.layer < len(self.layers):
                raise ValueError(f"run entry {index} names layer {entry.layer}, but there are {len(self.layers)} layers")
            if entry.cache_of is not None:
                if not 0 <= entry.cache_of < index:
                    raise ValueError(f"run entry {index} reads the cache of entry {entry.cache_of}, which is not an earlier entry")
                if self.order[entry.cache_of].cache_of is not None:
                    raise ValueError(f"run entry {index} reads the cache of entry {entry.cache_of}, which has none of its own")


# ---- what a mixer keeps per request -------------------------------------------------------------

@dataclass(frozen=True)
class PagedKV:
    """Keys and values of every cached token (or of the last ``window`` tokens), in pages."""

    n_kv_heads: int
    head_size: int
    window: int | None = None          # None: all keys


@dataclass(frozen=True)
class FixedState:
    """State of fixed size per request (``shape`` per run entry), in the request's slot."""

    shape: tuple
    dtype: str = "float32"


@dataclass(frozen=True)
class NoCache:
    pass
