"""Which kernel runs an operation.

``Kernels`` is what parts call.  With ``plain_only`` (always the case for the
32-bit path) every operation runs its plain kernel.  Otherwise a fast kernel is
asked first whether it takes the sizes at hand; if it does not, the plain
kernel runs: never a wrong result, never a CPU path.

A norm whose only consumer is a matrix product may be handed over unevaluated
(``DeferredNorm``): the product kernel for few rows normalises on the way in;
every other kernel has it evaluated first.
"""

from __future__ import annotations

import torch

from . import ops

SKINNY_MAX_ROWS = 8           # up to here a product streams the weights once through the SIMT kernel (measured:
                              # from 9 rows on the tensor-core kernel with swapped operands is faster)
SPLIT_ATTENTION_MAX_ROWS = 64 # up to here attention runs one CTA per (token, head, chunk of keys)


class DeferredNorm:
    """A norm that has not run yet: ``rows`` (or all rows) of the fp32 ``x``.

    ``kind`` names the arithmetic ("layer_norm": gain ``gamma``, shift ``beta``, ``eps``).  A
    product kernel that can norm its input on the way in takes a deferred norm only of a
    kind it knows (``Kernels.FUSED_NORM_KINDS``); any other kind is evaluated first by
    ``evaluate(ctx, out)``, the norm's own kernel.  A new norm therefore works everywhere
    from its first day and gets fused once a product kernel learns its kind."""

    def __init__(self, kind, x, rows, tag, evaluate, **params):
        self.kind, self.x, self.rows, self.tag, self.evaluate = kind, x, rows, tag, evaluate
        self.params = params
        self._value = None

    def __getattr__(self, name):
        try:
            return self.__dict__["params"][name]
        except KeyError:
            raise AttributeError(name) from None

    @property
    def shape(self):
        return (self.x.shape[0] if self.rows is None else self.rows.shape[0], self.x.shape[1])

    def materialize(self, ctx):
        if self._value is None:
            out = ctx.buffer(self.tag, self.shape, ctx.act_dtype)
            self.evaluate(ctx, out)
            self._value = out
        return self._value


class Kernels:
    FUSED_NORM_KINDS = ("layer_norm",)    # what the few-row product kernel can apply on the way in

    def __init__(self, act_dtype: torch.dtype, plain_only: bool = False):
        self.act_dtype = act_dtype
        self.plain_only = bool(plain_only) or act_dtype == torch.float32
        self.launches = 0            # kernels launched (or recorded into a graph) since the start
        self.choices = {}            # (operation, sizes...) -> name of the kernel that ran it last
        self._split_scratch = None
        self._sample_scratch = None
        self.scratch_generation = 0  # grows when scratch moves (captured graphs are then stale)
        self._status = None          # device word the tensor-core kernels report a timed-out wait in
        self._att_scratch = None
        self._att_work = None

    # ---- operations without a fast variant --------------------------------------------------
    def keep_tokens(self, kept, slots, tokens):
        self.launches += 1
        return ops.keep_tokens(kept, slots, tokens)

    def resolve_tokens(self, token_ids, kept):
        self.launches += 1
        return ops.resolve_tokens(token_ids, kept)

    def embed(self, out, token_ids, positions, table, position_table=None):
        self.launches += 1
        return ops.embed(out, token_ids, positions, table, position_table)

    def add_position_rows(self, hidden, positions, table):
        self.launches += 1
        return ops.add_position_rows(hidden, positions, table)

    def layernorm(self, out, x, gamma, beta, eps, rows=None):
        self.launches += 1
        if not self.plain_only and out.dtype == torch.bfloat16 and x.shape[1] % 4 == 0:
            return ops.layernorm_warp(out, x, gamma, beta, eps, rows)
        return ops.layernorm(out, x, gamma, beta, eps, rows)

    def kv_store(self, k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size):
        self.launches += 1
        return ops.kv_store(k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size)

    def sample_rows(self, out, logits, temperature=None, top_p=None, seeds=None, counters=None, any_nucleus=True):
        """One token per row.  ``any_nucleus``: whether some row may have a nucleus cut (top_p < 1
        with temperature > 0); rows without are drawn by many blocks each."""
        self.launches += 1
        rows = logits.shape[0]
        held = self._sample_scratch
        if held is None or held[2].numel() < rows:
            capacity = max(rows, 256)
            device = logits.device
            held = self._sample_scratch = (torch.empty(capacity * ops.SAMPLE_SLICES, dtype=torch.float32, device=device),
                                           torch.empty(capacity * ops.SAMPLE_SLICES, dtype=torch.int32, device=device),
                                           torch.zeros(capacity, dtype=torch.int32, device=device))
            self.scratch_generation += 1
        if any_nucleus:
            self.launches += 1
        return ops.sample_rows_sliced(out, logits, temperature, top_p, seeds, counters, held, any_nucleus)

    # ---- matrix products --------------------------------------------------------------------
    def _skinny(self, m, k, n=0) -> bool:
        # a product as wide as a vocabulary streams faster through the tensor-core kernel from
        # three rows on (measured at 50,257 x 768: 23 against 51 us at eight rows)
        rows = 2 if n >= 8192 and k % 8 == 0 else SKINNY_MAX_ROWS
        return not self.plain_only and m <= rows and ops.skinny_linear_takes(m, k)

    def linear(self, ctx, out, a, w, bias=None, epilogue="store"):
        """out = epilogue(a @ w.T + bias).  ``a``: an activation tensor or a ``DeferredNorm``."""
        m, k = a.shape
        self.launches += 1
        skinny = self._skinny(m, k, w.shape[0])
        deferred = isinstance(a, DeferredNorm)
        if deferred and not (skinny and a.kind in self.FUSED_NORM_KINDS):
            a, deferred = a.materialize(ctx), False      # no kernel here norms this kind on the way in: the norm runs first
        if skinny:
            self.chose("linear", "skinny_linear", m, w.shape[0], k)
            if deferred:
                return ops.skinny_linear(out, a.x, w, bias, epilogue, norm=(a.gamma, a.beta, a.eps, a.rows))
            return ops.skinny_linear(out, a, w, bias, epilogue)
        if not self.plain_only and ops.gemm_takes(a, w):
            self.chose("linear", "gemm_tcgen05", m, w.shape[0], k)
            return ops.gemm_bf16(out, a, w, bias, epilogue, self.status(ctx.device))
        self.chose("linear", "linear_plain", m, w.shape[0], k)
        return ops.linear_plain(out, a, w, bias, epilogue)

    def chose(self, operation: str, kernel: str, *sizes) -> None:
        """Note which kernel ran an operation at which sizes (tests pin the choices)."""
        self.choices[(operation, *sizes)] = kernel

    def status(self, device):
        if self._status is None:
            self._status = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status

    def read_status(self) -> int:
        """The code a kernel left when one of its bounded waits ran out, or 0 (synchronises)."""
        return int(self._status.item()) if self._status is not None else 0

    def reset_after_failure(self) -> None:
        """After a kernel gave up: the status word and every counter that kernels leave at
        zero between launches start over (a tile that was given up left its counter)."""
        if self._status is not None:
            self._status.zero_()
        if self._att_scratch is not None:
            self._att_scratch[1].zero_()
        if self._att_work is not None:
            self._att_work.zero_()
        if self._split_scratch is not None:
            self._split_scratch[2].zero_()
        if self._sample_scratch is not None:
            self._sample_scratch[2].zero_()

    def check_status(self) -> None:
        """Raise if a kernel reported that one of its bounded waits ran out (synchronises)."""
        code = self.read_status()
        if code != 0:
            self.reset_after_failure()
            raise ops.KernelError(f"a tensor-core kernel gave up waiting (code {code}): its result is invalid")

    def qkv_projection(self, ctx, a, w, bias, cache, q_width, kv_width):
        """The fused query/key/value projection.  Keys and values of the step's tokens go into
        the cache pages (if this entry writes its cache); returns the queries [T, q_width]."""
        m, k = a.shape
        skinny = cache.writes and self._skinny(m, k)
        deferred = isinstance(a, DeferredNorm)
        if deferred and not (skinny and a.kind in self.FUSED_NORM_KINDS):
            a, deferred = a.materialize(ctx), False
        if skinny:
            q = ctx.buffer("q", (m, q_width), ctx.act_dtype)
            scatter = (cache.k_pages, cache.v_pages, ctx.positions, ctx.token_item, cache.block_table,
                       cache.page_size, q_width, kv_width)
            self.launches += 1
            self.chose("qkv", "skinny_linear", m, w.shape[0], k)
            if deferred:
                ops.skinny_linear(q, a.x, w, bias, "store", norm=(a.gamma, a.beta, a.eps, a.rows), scatter=scatter)
            else:
                ops.skinny_linear(q, a, w, bias, "store", scatter=scatter)
            return q
        if cache.writes and not self.plain_only and ops.gemm_qkv_takes(a, w, q_width, kv_width):
            q = ctx.buffer("q", (m, q_width), ctx.act_dtype)
            self.launches += 1
            self.chose("qkv", "gemm_tcgen05", m, w.shape[0], k)
            return ops.gemm_bf16_qkv(q, a, w, bias, self.status(ctx.device), cache.k_pages, cache.v_pages,
                                     ctx.positions, ctx.token_item, cache.block_table, cache.page_size, q_width,
                                     kv_width)
        qkv = ctx.buffer("qkv", (m, q_width + 2 * kv_width), ctx.act_dtype)
        self.linear(ctx, qkv, a, w, bias)
        if cache.writes:
            self.kv_store(cache.k_pages, cache.v_pages, qkv[:, q_width:q_width + kv_width],
                          qkv[:, q_width + kv_width:], ctx.positions, ctx.token_item, cache.block_table,
                          cache.page_size)
        return qkv[:, :q_width]

    # ---- attention --------------------------------------------------------------------------
    def attention(self, ctx, out, q, cache, n_heads, n_kv_heads, head_size, scale, window=0):
        self.launches += 1
        n = q.shape[0]
        if (not self.plain_only and n <= SPLIT_ATTENTION_MAX_ROWS and head_size in ops.SPLIT_ATTENTION_HEAD_SIZES):
            # chunk of keys per CTA: small when there are few (token, head) pairs, so that the
            # chunks still fill the GPU
            pairs = n * n_heads
            chunk = 64 if pairs < 64 else (128 if pairs < 128 else (256 if pairs < 256 else 512))
            reach = cache.block_table.shape[1] * cache.page_size
            max_chunks = -(-reach // chunk)
            acc, ml, counters = self._scratch(ctx, SPLIT_ATTENTION_MAX_ROWS * n_heads, -(-reach // 64), head_size)
            # query heads that share a key/value head go through the tensor-core tiles together,
            # reading the keys once; with one query head per key/value head the SIMT kernel is
            # as fast or faster (measured at 9 to 64 requests of 12 heads)
            grouped = n_heads // n_kv_heads >= 2 and ops.group_attention_takes(q, n_heads, n_kv_heads, head_size)
            run = ops.group_attention if grouped else ops.split_attention
            self.chose("attention", "group_attention" if grouped else "split_attention", n, n_heads, head_size)
            return run(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions, ctx.token_item,
                       n_heads, n_kv_heads, head_size, cache.page_size, scale, window, chunk, max_chunks, acc, ml,
                       counters)
        if (not self.plain_only and ctx.att_tiles is not None
                and ops.attention_prefill_takes(q, head_size, cache.page_size)):
            scratch = None
            if ctx.att_parts > 1:
                # Room for the most cells a step can have, whatever this one has: a step replayed
                # from a graph brings its number of split tiles as data and passes by here no more.
                # (Tiles are split in steps of at most eight of them; units while records x heads
                # stay within the SMs, of which no GPU has 256.)
                most = max(ctx.n_split_tiles * n_heads, 8 * n_heads, 256)
                # (cells of a unit's 256 rows, also for the kernel with tiles of 128: one size, no regrowth)
                scratch = self._attention_scratch(ctx.device, most, ops.ATTENTION_MAX_PARTS * ops.ATTENTION_UNIT * (head_size + 4))
            if ctx.att_units:
                self.chose("attention", "attention_two_tiles", n, n_heads, head_size)
                return ops.attention_prefill_two_tiles(out, q, cache.k_pages, cache.v_pages, cache.block_table,
                                                       ctx.att_tiles, ctx.n_att_tiles, n_heads, n_kv_heads, head_size,
                                                       cache.page_size, scale, window, self.status(ctx.device),
                                                       self.attention_work(ctx.device), scratch, ctx.n_split_tiles,
                                                       ops.ATTENTION_MAX_PARTS if ctx.att_parts > 1 else 1)
            self.chose("attention", "attention_tcgen05", n, n_heads, head_size)
            return ops.attention_prefill(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.att_tiles,
                                         ctx.n_att_tiles, n_heads, n_kv_heads, head_size, cache.page_size, scale,
                                         window, self.status(ctx.device), self.attention_work(ctx.device), scratch,
                                         ctx.n_split_tiles,
                                         ops.ATTENTION_MAX_PARTS if ctx.att_parts > 1 else 1)
        self.chose("attention", "attention_plain", n, n_heads, head_size)
        return ops.attention_plain(out, q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions,
                                   ctx.token_item, n_heads, n_kv_heads, head_size, cache.page_size, scale, window)

    def attention_work(self, device):
        """The work counter of the persistent prompt-attention kernel (zero between launches)."""
        if self._att_work is None:
            self._att_work = torch.zeros(2, dtype=torch.int32, device=device)
            self.scratch_generation += 1
        return self._att_work

    def _attention_scratch(self, device, cells, floats_per_cell):
        """Partial states and counters of prompt attention tiles that come in parts; grows
        (doubling) when a step has more split tiles than any before."""
        held = self._att_scratch
        if held is None or held[1].shape[0] < 2 * cells or held[0].shape[0] < cells * floats_per_cell:
            cells = max(cells, held[1].shape[0] if held is not None else 256)
            # (two counters a cell: the kernel with two tiles per CTA counts each tile's parts apart)
            self._att_scratch = held = (torch.empty(cells * floats_per_cell, dtype=torch.float32, device=device),
                                        torch.zeros(2 * cells, dtype=torch.int32, device=device))
            self.scratch_generation += 1
        return held

    def _scratch(self, ctx, pairs, chunks, head_size):
        """Scratch of split_attention, sized for the largest step it takes; allocated once
        (the counters must start at zero and the kernel leaves them so)."""
        need = (pairs * chunks * head_size, pairs * chunks * 2, pairs)
        held = self._split_scratch
        if held is None or any(h.numel() < n for h, n in zip(held, need)):
            device = ctx.device
            self._split_scratch = (torch.empty(need[0], dtype=torch.float32, device=device),
                                   torch.empty(need[1], dtype=torch.float32, device=device),
                                   torch.zeros(need[2], dtype=torch.int32, device=device))
            self.scratch_generation += 1
        return self._split_scratch
