"""Interfaces of the parts a layer is put together from, and their registries.

A part is constructed from its weight-name prefix and its own parameters
(sizes, constants), states which tensors it needs (``weight_specs``), receives
them on the device (``bind``) and then runs on a ``StepContext``.  It never
sees a configuration or the model it is in.

Interfaces (``ctx`` is ``engine.context.StepContext``; ``hidden`` is the fp32
residual stream [T, width]; "act" tensors have the engine's element type):

``Norm.forward(ctx, x, rows=None, tag="norm") -> act [R, width]``
    normalise rows of ``x`` (all, or those ``rows`` names).
``Mixer.cache_need() -> PagedKV | FixedState | NoCache``
``Mixer.forward(ctx, x, hidden, cache)``
    add the mixer's output for the normed input ``x`` into ``hidden`` in
    place.  ``cache`` is this run entry's ``cache.views.LayerCache``; when
    ``cache.writes`` is false the entry reads another entry's cache and must
    not store into it.
``FeedForward.forward(ctx, x, hidden)``
    add the feed-forward output for ``x`` into ``hidden`` in place.
``PositionEncoding.add_to_hidden(ctx, hidden)``
    for encodings that act on the embedded tokens; ``additive_table()`` may
    return the table so that the embedding gather fuses the sum.  Encodings
    that act inside a mixer are given to that mixer as a parameter instead.
``Embedding.forward(ctx, position=None) -> hidden``
``Head.forward(ctx, x) -> fp32 logits [R, vocab]``
``Arrangement.run(ctx, parts, hidden, cache)``
    wire one layer's parts (by role) around the residual stream.
"""

from __future__ import annotations

from .spec import NoCache, PartSpec, WeightSpec


class Part:
    """Base of every part.

    ``graph_safe``: the part's ``forward`` launches only kernels on the current stream
    whose arguments (pointers into the context's buffers, sizes that follow from the
    step's shape) are the same for every step of one shape.  Steps of a model whose parts
    all say so may be captured into a CUDA graph; the default is not to."""

    graph_safe = False

    def __init__(self, prefix: str = ""):
        self.prefix = prefix
        self.weights = {}

    def full_name(self, local: str) -> str:
        return f"{self.prefix}.{local}" if self.prefix else local

    def weight_specs(self) -> list[WeightSpec]:
        return []

    def bind(self, tensors: dict, runtime) -> None:
        """Receive the device tensors, keyed by the names of ``weight_specs``."""
        self.weights = tensors
        self.runtime = runtime

    def w(self, local: str):
        return self.weights[self.full_name(local)]


class Norm(Part):
    def forward(self, ctx, x, rows=None, tag="norm"):
        raise NotImplementedError


class Mixer(Part):
    def cache_need(self):
        return NoCache()

    def forward(self, ctx, x, hidden, cache):
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, ctx, x, hidden):
        raise NotImplementedError


class PositionEncoding(Part):
    def add_to_hidden(self, ctx, hidden):
        raise NotImplementedError

    def additive_table(self):
        return None


class Embedding(Part):
    def forward(self, ctx, position=None):
        raise NotImplementedError


class Head(Part):
    def forward(self, ctx, x):
        raise NotImplementedError


class Arrangement:
    """How the parts of one layer are wired; ``roles`` names the parts it needs."""

    roles: tuple = ()

    def run(self, ctx, parts: dict, hidden, cache) -> None:
        raise NotImplementedError

    def mixer_role(self) -> str:
        return "mixer"


_PART_KINDS: dict[str, type] = {}
_ARRANGEMENTS: dict[str, Arrangement] = {}


def register_part(kind: str, cls: type) -> None:
    _PART_KINDS[kind] = cls


def register_arrangement(name: str, arrangement: Arrangement) -> None:
    _ARRANGEMENTS[name] = arrangement


def build_part(spec: PartSpec) -> Part:
    try:
        cls = _PART_KINDS[spec.kind]
    except KeyError:
        raise KeyError(f"unknown part kind '{spec.kind}'; known: {', '.join(sorted(_PART_KINDS))}") from None
    return cls(prefix=spec.prefix, **spec.params)


def get_arrangement(name: str) -> Arrangement:
    try:
        return _ARRANGEMENTS[name]
    except KeyError:
        raise KeyError(f"unknown arrangement '{name}'; known: {', '.join(sorted(_ARRANGEMENTS))}") from None
