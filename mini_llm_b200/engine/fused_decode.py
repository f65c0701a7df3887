"""A decode step as ONE kernel, when the model is a plain stack of pre-norm layers.

The generic path runs a step part by part, about five kernels a layer.  For steps of few
tokens that is bound by launch gaps, not by memory or arithmetic.  If a model's description
is nothing but ``pre_norm`` layers of ``layer_norm`` / ``causal_self_attention`` /
``layer_norm`` / ``dense_mlp`` around a ``token_embedding`` (with or without
``learned_positions``), a final ``layer_norm`` and a ``linear_head``, the same arithmetic is
compiled into a table of pointers and run by ``csrc/fused_decode.cu``: one persistent kernel
per step.  Any other model, any step with a prompt portion, and any size the kernel does not
take go the generic way; nothing outside this file knows the difference.
"""

from __future__ import annotations

import ctypes

import torch

from ..kernels import ops
from ..kernels.lib import Function, KernelError, load

P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float


class _Layer(ctypes.Structure):
    _fields_ = [("ln1_g", P), ("ln1_b", P), ("w_qkv", P), ("b_qkv", P), ("w_o", P), ("b_o", P), ("ln2_g", P),
                ("ln2_b", P), ("w_fc", P), ("b_fc", P), ("w_proj", P), ("b_proj", P), ("k_pages", P), ("v_pages", P),
                ("score_scale", F), ("eps1", F), ("eps2", F), ("activation", I), ("window", I)]


class _Params(ctypes.Structure):
    _fields_ = [("layers", P), ("n_layers", I), ("E", I), ("H", I), ("Hkv", I), ("D", I), ("I", I), ("V", I), ("T", I),
                ("token_ids", P), ("positions", P), ("token_item", P), ("block_table", P), ("max_blocks", I),
                ("page_size", I), ("want_rows", P), ("n_want", I), ("wte", P), ("wpe", P), ("lnf_g", P), ("lnf_b", P),
                ("eps_f", F), ("w_head", P), ("hidden", P), ("q", P), ("attn", P), ("up", P), ("logits", P),
                ("sample", I),
                ("temperature", P), ("top_p", P), ("seeds", P), ("counters", P), ("out_tokens", P), ("kept", P), ("want_slots", P),
                ("n_kept", I), ("cand_value", P),
                ("cand_index", P), ("cand_done", P), ("barrier", P), ("status", P), ("timeline", P),
                ("att_parts", I), ("att_partial", P), ("att_counters", P),
                ("barrier_limit_ns", ctypes.c_ulonglong), ("skip_arrival", I)]


_step = Function("fused", "mllm_fused_decode_step", [ctypes.POINTER(_Params), P])
MAX_TOKENS = 16
MAX_ATTENTION_PARTS = 16
_KINDS = {"norm_1": "layer_norm", "mixer": "causal_self_attention", "norm_2": "layer_norm", "feed_forward": "dense_mlp"}


def _mismatch(spec) -> str | None:
    """Why the description is not of the fused shape, or None if it is."""
    if spec.embedding.kind != "token_embedding":
        return f"the embedding is a '{spec.embedding.kind}', not a token_embedding"
    if spec.final_norm.kind != "layer_norm":
        return f"the final norm is a '{spec.final_norm.kind}', not a layer_norm"
    if spec.head.kind != "linear_head":
        return f"the head is a '{spec.head.kind}', not a linear_head"
    if spec.position is not None and spec.position.kind != "learned_positions":
        return f"the position encoding is '{spec.position.kind}', not learned_positions"
    for index, layer in enumerate(spec.layers):
        if layer.arrangement != "pre_norm":
            return f"layer {index} is arranged as '{layer.arrangement}', not pre_norm"
        for role, kind in _KINDS.items():
            have = layer.parts[role].kind if role in layer.parts else None
            if have != kind:
                return f"layer {index} has a '{have}' as its {role}, not a {kind}"
        if layer.parts["mixer"].params.get("position") is not None:
            return f"layer {index}'s mixer has a position encoding of its own"
        if set(layer.parts) != set(_KINDS):
            return f"layer {index} has parts beyond {', '.join(_KINDS)}"
    if not spec.order:
        return "no layer runs"
    if any(entry.cache_of is not None for entry in spec.order):
        return "a run entry reads another entry's cache"
    return None


class FusedDecodePlan:
    @classmethod
    def build(cls, engine):
        """``(plan, None)`` for ``engine``'s model, or ``(None, reason)`` if the model, the
        element type or a size is not what the kernel takes."""
        spec, model = engine.spec, engine.model
        if engine.dtype != torch.bfloat16 or engine.kernels.plain_only:
            return None, "the kernel is for bfloat16 with the fast kernels"
        reason = _mismatch(spec)
        if reason is not None:
            return None, reason
        mixers = [model.layers[e.layer][1]["mixer"] for e in spec.order]
        mlps = [model.layers[e.layer][1]["feed_forward"] for e in spec.order]
        first = mixers[0]
        same = all((m.width, m.n_heads, m.n_kv_heads, m.head_size) == (first.width, first.n_heads, first.n_kv_heads,
                                                                        first.head_size) for m in mixers)
        if not same or any(f.inner != mlps[0].inner for f in mlps):
            return None, "the layers differ in their sizes"
        if len({v.group for v in engine.storage.views}) != 1:
            return None, "the layers keep their caches in more than one group"
        lib = load("fused")
        if ctypes.sizeof(_Layer) != lib.mllm_fused_layer_bytes() or ctypes.sizeof(_Params) != lib.mllm_fused_params_bytes():
            raise KernelError("fused_decode: the binding's structures do not match the library's")
        if not lib.mllm_fused_takes(1, first.width, first.n_heads, first.n_kv_heads, first.head_size, mlps[0].inner,
                                    engine.cache.groups[0].max_blocks):
            return None, (f"the kernel does not take width {first.width}, {first.n_heads} heads of {first.head_size}, "
                          f"inner size {mlps[0].inner} (widths must be multiples of 32, the head size a power of two, "
                          f"and a step's staging must fit in shared memory)")
        return cls(engine, lib), None

    def __init__(self, engine, lib):
        self.engine = engine
        self.lib = lib
        self.grid = lib.mllm_fused_grid()
        spec, model = engine.spec, engine.model
        rows = []
        activations = {"gelu_tanh": ops.EPILOGUES["gelu_tanh"], "gelu_erf": ops.EPILOGUES["gelu_erf"]}
        for index, entry in enumerate(spec.order):
            parts = model.layers[entry.layer][1]
            n1, att, n2, mlp = parts["norm_1"], parts["mixer"], parts["norm_2"], parts["feed_forward"]
            view = engine.storage.views[index]
            rows.append(_Layer(
                n1.w("weight").data_ptr(), n1.w("bias").data_ptr(),
                att.w(f"{att.qkv_name}.weight").data_ptr(), att.w(f"{att.qkv_name}.bias").data_ptr(),
                att.w(f"{att.out_name}.weight").data_ptr(), att.w(f"{att.out_name}.bias").data_ptr(),
                n2.w("weight").data_ptr(), n2.w("bias").data_ptr(),
                mlp.w(f"{mlp.up_name}.weight").data_ptr(), mlp.w(f"{mlp.up_name}.bias").data_ptr(),
                mlp.w(f"{mlp.down_name}.weight").data_ptr(), mlp.w(f"{mlp.down_name}.bias").data_ptr(),
                view.k_pages.data_ptr(), view.v_pages.data_ptr(), att.score_scale, n1.eps, n2.eps,
                activations[mlp.activation], att.window or 0))
        table = (_Layer * len(rows))(*rows)
        raw = torch.frombuffer(bytearray(bytes(table)), dtype=torch.uint8)
        self.layer_table = raw.to(engine.device)
        att, mlp = model.layers[spec.order[0].layer][1]["mixer"], model.layers[spec.order[0].layer][1]["feed_forward"]
        self.sizes = (att.width, att.n_heads, att.n_kv_heads, att.head_size, mlp.inner, spec.vocab_size)
        device = engine.device
        self.max_blocks = engine.cache.groups[0].max_blocks
        self._filled = {}             # step shape -> (filled parameters, logits view, sampled view)
        self.timeline = None          # set to an int64 tensor of 5 * layers + 3 entries to record phase times
        # For tests of the bounded wait (both enter the parameters of every later step):
        self.barrier_limit_ns = 0     # a barrier wait gives up after this long (0: the kernel's two seconds)
        self.skip_arrival = False     # one CTA stays away from the step's first barrier, which then runs out
        self.cand_value = torch.empty(MAX_TOKENS * self.grid, dtype=torch.float32, device=device)
        self.cand_index = torch.empty(MAX_TOKENS * self.grid, dtype=torch.int32, device=device)
        self.cand_done = torch.zeros(1, dtype=torch.int32, device=device)
        self.barrier = torch.zeros(1, dtype=torch.int64, device=device)
        self.out_tokens = torch.zeros(2, MAX_TOKENS, dtype=torch.int32, device=device)     # by the step's parity
        heads, head_size = self.sizes[1], self.sizes[3]
        self.att_partial = torch.empty(MAX_TOKENS * heads * MAX_ATTENTION_PARTS * (head_size + 2), dtype=torch.float32,
                                       device=device)
        self.att_counters = torch.zeros(MAX_TOKENS * heads, dtype=torch.int32, device=device)
        self.force_parts = None       # tests and measurements: this many CTAs share every pair's keys

    def takes(self, ctx) -> bool:
        return self.takes_sizes(ctx.n_tokens, ctx.decode_only)

    def takes_sizes(self, n_tokens: int, decode_only: bool) -> bool:
        width, heads, kv_heads, head_size, inner, _ = self.sizes
        return (decode_only and n_tokens <= MAX_TOKENS
                and bool(self.lib.mllm_fused_takes(n_tokens, width, heads, kv_heads, head_size, inner, self.max_blocks)))

    def attention_parts(self, ctx) -> int:
        """How many CTAs share the keys of one (token, head) pair: as many as leave every CTA at
        most one part (a part's hand-over costs more than a second part would save), with at
        least 64 keys each."""
        if self.force_parts is not None:
            return int(self.force_parts)
        pairs = ctx.n_tokens * self.sizes[1]
        longest = max(ctx.item_starts) + 1
        return max(1, min(MAX_ATTENTION_PARTS, self.grid // pairs, longest // 64))

    def run(self, ctx, block_table, sample_views, any_nucleus):
        """Run the step; returns (logits or None, sampled tokens or None)."""
        engine = self.engine
        sampling = sample_views is not None and ctx.n_want > 0
        # Steps of one shape find all their arrays at the same addresses (the control block's
        # layout depends on the step's sizes only): their parameters are filled once.
        parts = self.attention_parts(ctx)
        key = (ctx.n_tokens, ctx.n_want, sampling, self.timeline is not None, parts, engine.control.parity,
               engine.workspace.generation, engine.control.generation, self.barrier_limit_ns, self.skip_arrival)
        held = self._filled.get(key)
        if held is None:
            if len(self._filled) > 64:
                self._filled.clear()
            held = self._filled[key] = self._fill(ctx, block_table, sample_views if sampling else None, parts)
        params, logits, sampled = held
        _step(ctypes.byref(params), torch.cuda.current_stream().cuda_stream)
        engine.kernels.launches += 1
        if sampled is not None and any_nucleus:
            ops.sample_rows_nucleus(sampled, logits, *sample_views)
            engine.kernels.launches += 1
            engine.kernels.keep_tokens(engine.kept_tokens, ctx.want_slots, sampled)    # the kernel kept its own draw
        return logits, sampled

    def _fill(self, ctx, block_table, sample_views, parts):
        engine = self.engine
        model = engine.model
        width, heads, kv_heads, head_size, inner, vocab = self.sizes
        n = ctx.n_tokens
        hidden = ctx.buffer("hidden", (n, width), torch.float32)
        q = ctx.buffer("q", (n, heads * head_size), torch.bfloat16)
        attn = ctx.buffer("attn_out", (n, heads * head_size), torch.bfloat16)
        up = ctx.buffer("mlp_up", (n, inner), torch.bfloat16)
        logits = ctx.buffer("logits", (ctx.n_want, vocab), torch.float32) if ctx.n_want else None
        params = _Params()
        params.layers, params.n_layers = self.layer_table.data_ptr(), len(engine.spec.order)
        params.E, params.H, params.Hkv, params.D, params.I, params.V, params.T = (width, heads, kv_heads, head_size,
                                                                                    inner, vocab, n)
        params.token_ids, params.positions = ctx.token_ids.data_ptr(), ctx.positions.data_ptr()
        params.token_item, params.block_table = ctx.token_item.data_ptr(), block_table.data_ptr()
        params.max_blocks, params.page_size = block_table.shape[1], engine.page_size
        params.want_rows, params.n_want = ctx.want_rows.data_ptr(), ctx.n_want
        params.wte = model.embedding.w(model.embedding.name).data_ptr()
        params.wpe = model.position.w(model.position.name).data_ptr() if model.position is not None else None
        params.lnf_g, params.lnf_b = model.final_norm.w("weight").data_ptr(), model.final_norm.w("bias").data_ptr()
        params.eps_f, params.w_head = model.final_norm.eps, model.head.w(model.head.weight_name).data_ptr()
        params.hidden, params.q, params.attn, params.up = hidden.data_ptr(), q.data_ptr(), attn.data_ptr(), up.data_ptr()
        params.logits = logits.data_ptr() if logits is not None else None
        params.timeline = self.timeline.data_ptr() if self.timeline is not None else None
        sampled = None
        if sample_views is not None:
            temperature, top_p, seeds, counters = sample_views
            params.sample = 1
            params.temperature, params.top_p = temperature.data_ptr(), top_p.data_ptr()
            params.seeds, params.counters = seeds.data_ptr(), counters.data_ptr()
            sampled = self.out_tokens[engine.control.parity, :ctx.n_want]
        params.out_tokens = self.out_tokens[engine.control.parity].data_ptr()
        params.kept, params.n_kept = engine.kept_tokens.data_ptr(), engine.kept_tokens.shape[0]
        params.want_slots = ctx.want_slots.data_ptr()
        params.cand_value, params.cand_index = self.cand_value.data_ptr(), self.cand_index.data_ptr()
        params.cand_done, params.barrier = self.cand_done.data_ptr(), self.barrier.data_ptr()
        params.status = engine.kernels.status(engine.device).data_ptr()
        params.att_parts = parts
        params.barrier_limit_ns, params.skip_arrival = int(self.barrier_limit_ns), int(self.skip_arrival)
        params.att_partial, params.att_counters = self.att_partial.data_ptr(), self.att_counters.data_ptr()
        return params, logits, sampled

    def reset(self) -> None:
        """After a failed step: the barrier counter and the scratch counters start over."""
        self.barrier.zero_()
        self.cand_done.zero_()
        self.att_counters.zero_()
