"""A model built from its description: parts with their weights, run in order.

Nothing here names an architecture.  ``Model`` builds every part the
description lists, loads the tensors they declare, and runs a step: embed,
the run entries in their order (each with the cache view of its entry), then
the final norm and the head on the rows whose logits are wanted only (the
reference norms and multiplies the last row only,
engine/src/gpt2_gpu.cu:254-263).
"""

from __future__ import annotations

from ..parts.base import build_part, get_arrangement
from ..parts.spec import NoCache
from ..weights.loader import collect_specs, load_weights


class Model:
    def __init__(self, spec):
        self.spec = spec
        self.embedding = build_part(spec.embedding)
        self.position = build_part(spec.position) if spec.position is not None else None
        self.layers = []
        for layer in spec.layers:
            arrangement = get_arrangement(layer.arrangement)
            missing = [role for role in arrangement.roles if role not in layer.parts]
            if missing:
                raise ValueError(f"arrangement '{layer.arrangement}' needs parts {missing}")
            self.layers.append((arrangement, {role: build_part(p) for role, p in layer.parts.items()}))
        self.final_norm = build_part(spec.final_norm)
        self.head = build_part(spec.head)
        # A step may be captured into a CUDA graph only if every part launches nothing but
        # kernels whose arguments stay valid from step to step; parts say so themselves.
        self.graph_safe = all(getattr(part, "graph_safe", False) for part in self.parts())
        # The step makes a work list of attention tiles only if some part says it reads one.
        self.wants_attention_tiles = any(getattr(part, "wants_attention_tiles", False) for part in self.parts())
        # A step of long portions may bring its work list as units of 256 tokens instead, if
        # every part that reads the list can read those too: then this is their number of heads
        # (the step shares long units among so many CTAs that heads x CTAs fill the GPU), else 0.
        heads = {getattr(part, "attention_unit_heads", 0) for part in self.parts() if getattr(part, "wants_attention_tiles", False)}
        self.attention_unit_heads = heads.pop() if len(heads) == 1 else 0

    def parts(self):
        found = [self.embedding]
        if self.position is not None:
            found.append(self.position)
        for _, parts in self.layers:
            found.extend(parts.values())
        found.extend([self.final_norm, self.head])
        return found

    def cache_needs(self):
        """What each run entry keeps per request; None for an entry that reads another's cache."""
        needs = []
        for entry in self.spec.order:
            arrangement, parts = self.layers[entry.layer]
            if entry.cache_of is not None:
                needs.append(None)
                continue
            need = parts[arrangement.mixer_role()].cache_need()
            needs.append(None if isinstance(need, NoCache) else need)
        return needs

    def load(self, model_dir: str, dtype, device, runtime=None):
        specs = collect_specs(self.parts())
        tensors = load_weights(model_dir, specs, dtype, device, self.spec.file_prefixes, self.spec.ignored_weights)
        for part in self.parts():
            part.bind({w.name: tensors[w.name] for w in part.weight_specs() if w.name in tensors}, runtime)
        self.weight_bytes = sum(t.numel() * t.element_size() for t in
                                {t.data_ptr(): t for t in tensors.values()}.values())
        return self

    def forward(self, ctx, cache_views):
        """Run the step's tokens; returns fp32 logits [n_want, vocab] or None."""
        hidden = self.embedding.forward(ctx, self.position)
        dump = getattr(ctx, "dump", None)
        if dump is not None:
            dump.append(hidden.clone())
        for index, entry in enumerate(self.spec.order):
            arrangement, parts = self.layers[entry.layer]
            arrangement.run(ctx, parts, hidden, cache_views[index])
            if dump is not None:
                dump.append(hidden.clone())
        if ctx.n_want == 0:
            return None
        defer = getattr(self.final_norm, "can_defer", False) and getattr(self.head, "accepts_deferred_norm", False)
        rows = self.final_norm.forward(ctx, hidden, rows=ctx.want_rows, tag="final_norm",
                                       **({"defer": True} if defer else {}))
        return self.head.forward(ctx, rows)
