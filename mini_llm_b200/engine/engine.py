"""The engine: a model on one GPU, its caches, and the one step function.

``Engine.step(entries)`` takes a batch of (request, its next tokens): portions
of prompts beside single decoded tokens, cut anywhere.  It runs only the
tokens it is given, as one batch, against the cache earlier steps left, and
returns the logits at the wanted places.  The reference has three entry
points instead (whole-prompt prefill, single decode, batched decode of up to
16: engine/include/gpt2_gpu.h:64-68,89-90,161-165) and never mixes a prompt
with decoding requests.

Like the reference (engine/src/gpt2_gpu.cu:197-207,301-304), a step checks all
of its input before it launches anything, and a refused step changes nothing.
"""

from __future__ import annotations

import sys
from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.storage import CacheStorage
from ..config.registry import config_from_folder, describe_model
from ..kernels import ops
from ..kernels.lib import KernelError
from ..kernels.dispatch import SPLIT_ATTENTION_MAX_ROWS, Kernels
from ..sampling import SamplingParams
from .context import ControlBlock, StepContext, Workspace
from .fused_decode import FusedDecodePlan
from .model import Model

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


# As a token id in ``StepEntry.tokens``: "the token this request sampled in its last sampling
# step".  It is taken on the device, so the step can be launched before the host has read it.
PREVIOUS = -1


class StepError(ValueError):
    """The step's input is invalid; nothing was run and nothing changed."""


class OutOfPages(RuntimeError):
    """The page pools cannot hold the step's tokens; nothing was run and nothing changed."""


@dataclass
class StepEntry:
    slot: int                     # the request's slot, from ``open_request``
    tokens: list                  # its next tokens
    want: list = field(default_factory=list)     # places among these tokens whose logits are wanted


class Engine:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", device: str = "cuda:0", page_size: int = 64,
                 cache_tokens: int | None = None, n_pages: int | None = None, max_requests: int = 64,
                 max_tokens_per_step: int = 2048, plain_kernels: bool = False, cuda_graphs: bool = True,
                 fused_decode: bool = True, debug_poison: bool = False):
        """``debug_poison``: every cache slot that holds no live token holds a poison value
        (NaN on the 32-bit path; 1e30 on the bfloat16 path, whose tensor-core attention
        multiplies what lies in a masked slot by a weight of zero), so that a read past a
        request's length or through a stale block-table row ruins the logits instead of
        passing for another request's keys."""
        if not torch.cuda.is_available():
            raise RuntimeError("mini_llm_b200 runs on a CUDA device (sm_100a) only; none is available "
                               "and there is no CPU path")
        if dtype not in DTYPES:
            raise ValueError(f"dtype must be one of {', '.join(sorted(DTYPES))}, got '{dtype}'")
        self.dtype = DTYPES[dtype]
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.config = config_from_folder(model_dir)
        self.spec = describe_model(self.config)
        self.model = Model(self.spec)
        self.kernels = Kernels(self.dtype, plain_only=plain_kernels)
        self.model.load(model_dir, self.dtype, self.device, runtime=self)
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_tokens_per_step = int(max_tokens_per_step)
        self.cuda_graphs = bool(cuda_graphs)
        self._n_sms = torch.cuda.get_device_properties(self.device).multi_processor_count

        needs = self.model.cache_needs()
        per_request = self.spec.max_positions
        if n_pages is None:
            if cache_tokens is None:
                cache_tokens = self.max_requests * (per_request if per_request is not None else 4096)
            n_pages = -(-int(cache_tokens) // self.page_size)
        if per_request is None:
            per_request = n_pages * self.page_size
        self.max_positions = per_request
        self.cache = CacheManager(needs, self.page_size, int(n_pages), self.max_requests, per_request)
        poison = None
        if debug_poison:
            poison = float("nan") if self.kernels.plain_only else 1e30
        self.storage = CacheStorage(self.cache, self.spec.order, self.dtype, self.device, self.max_requests, poison)
        self.workspace = Workspace(self.device, min_rows=min(self.max_tokens_per_step, 256))
        self.control = ControlBlock(self.device, self.cache.groups)
        self.ctx = StepContext(self.kernels, self.workspace, self.dtype, self.device)
        self.steps = 0
        self._sampled = None
        self.kept_tokens = torch.zeros(self.max_requests, dtype=torch.int32, device=self.device)
        self._kept_valid = set()              # slots whose entry of kept_tokens is a sampled token
        self._readback = [None, None]         # per step parity: (pinned host buffer, rows, event)
        self._turn = 0
        self._alternated = False              # whether the last step took its arrays from the alternating buffers
        self._readback_stream = torch.cuda.Stream(device=self.device)    # sampled ids go to the host beside the next step
        self._sampled_events = [torch.cuda.Event(), torch.cuda.Event()]  # a step's sampling is done
        self._graphs = {}
        self._graph_stamp = None
        self.step_kinds = {"one_kernel": 0, "eager": 0, "captured": 0, "replayed": 0}      # how steps ran
        self._can_pad = self.storage.spare_page          # steps may be filled up to round shapes (see _step_reserved)
        self.fused, self.fused_reason = (FusedDecodePlan.build(self) if fused_decode
                                         else (None, "switched off by the caller"))
        if self.fused is None and fused_decode and self.dtype == torch.bfloat16 and not self.kernels.plain_only:
            # not an error, but a cliff in speed (a decode step is then some five launches a layer)
            print(f"[mini_llm_b200] decode steps run part by part, not as one kernel: {self.fused_reason}",
                  file=sys.stderr, flush=True)
        self._status_pinned = torch.zeros(2, dtype=torch.int32).pin_memory()   # per step parity: the kernels' status word
        self._status_host = self._status_pinned.numpy()
        self.hidden_dump = None               # set by step(dump_hidden=True): the residual stream after every run entry

    # ---- requests ---------------------------------------------------------------------------
    def open_request(self) -> int | None:
        """A slot for a new request (its cache starts empty), or None if every slot is taken."""
        slot = self.cache.open()
        if slot is not None:
            self.storage.reset_slot(slot)
            self._kept_valid.discard(slot)
        return slot

    def close_request(self, slot: int) -> None:
        """Give back what the request holds."""
        self.cache.close(slot)
        self._kept_valid.discard(slot)

    def device_info(self) -> dict:
        """Name, compute capability, SM count, memory and CUDA versions of the engine's device."""
        with torch.cuda.device(self.device):
            return ops.device_info()

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def cached_tokens(self, slot: int) -> int:
        return self.cache.length(slot)

    # ---- the step ---------------------------------------------------------------------------
    def _validate(self, entries) -> None:
        if not entries:
            raise StepError("a step needs at least one entry")
        seen = set()
        vocab = self.spec.vocab_size
        total = 0
        for index, entry in enumerate(entries):
            if not self.cache.is_open(entry.slot):
                raise StepError(f"entry {index}: slot {entry.slot} holds no request")
            if entry.slot in seen:
                raise StepError(f"entry {index}: slot {entry.slot} appears twice in one step")
            seen.add(entry.slot)
            n = len(entry.tokens)
            if n == 0:
                raise StepError(f"entry {index}: no tokens")
            total += n
            first = entry.tokens[0]
            if n == 1 and type(first) is int:
                # a decoding request's one token: the common case, checked without an array
                if first == PREVIOUS:
                    if entry.slot not in self._kept_valid:
                        raise StepError(f"entry {index}: slot {entry.slot} has sampled no token that PREVIOUS could name")
                elif not 0 <= first < vocab:
                    raise StepError(f"entry {index}: token id {first} is outside the vocabulary [0, {vocab}) "
                                    f"(PREVIOUS may only be an entry's first token)")
            else:
                try:
                    ids = np.asarray(entry.tokens, dtype=np.int64)
                except (TypeError, ValueError, OverflowError):
                    raise StepError(f"entry {index}: token ids must be integers") from None
                low = int(ids.min()) if ids.ndim == 1 else -2
                if low == PREVIOUS and not (ids[1:] == PREVIOUS).any():
                    if entry.slot not in self._kept_valid:
                        raise StepError(f"entry {index}: slot {entry.slot} has sampled no token that PREVIOUS could name")
                    low = int(ids[1:].min()) if n > 1 else 0
                if ids.ndim != 1 or low < 0 or int(ids.max()) >= vocab:
                    bad = next((t for t in entry.tokens if not 0 <= int(t) < vocab), None)
                    raise StepError(f"entry {index}: token id {bad} is outside the vocabulary [0, {vocab}) "
                                    f"(PREVIOUS may only be an entry's first token)")
            have = self.cache.length(entry.slot)
            if have + n > self.max_positions:
                raise StepError(f"entry {index}: {have} cached + {n} new tokens exceed the {self.max_positions} "
                                f"positions a request may hold")
            for place in entry.want:
                if not 0 <= int(place) < n:
                    raise StepError(f"entry {index}: wanted place {place} is not among its {n} tokens")
        if total > self.max_tokens_per_step:
            raise StepError(f"the step brings {total} tokens, more than the {self.max_tokens_per_step} "
                            f"this engine takes in one step (max_tokens_per_step)")

    def _reserve(self, entries) -> None:
        cache = self.cache
        needed = [0] * len(cache.groups)
        per_entry = []
        for entry in entries:
            mine = cache.pages_needed(entry.slot, len(entry.tokens))
            per_entry.append(mine)
            for g, count in enumerate(mine):
                needed[g] += count
        if any(needed):
            free = cache.pages_free()
            for g, count in enumerate(needed):
                if count > free[g]:
                    raise OutOfPages(f"the step needs {count} more pages in cache group {g}, {free[g]} are free")
        for entry, mine in zip(entries, per_entry):
            if not cache.reserve(entry.slot, len(entry.tokens), mine):
                raise OutOfPages("page reservation failed after it was checked")   # cannot happen

    def step(self, entries, sampling=None, dump_hidden: bool = False):
        """Run one batch.  Returns fp32 logits ``[wanted, vocab]`` on the device
        (in the order of the entries and of each ``want``; valid until the next
        step), or None if nothing is wanted.  With ``sampling`` (one
        ``SamplingParams`` per wanted row) the chosen tokens are then read with
        ``sampled_tokens()``.  With ``dump_hidden`` the step runs part by part and
        ``hidden_dump`` afterwards holds the fp32 residual stream [tokens, width] after the
        embedding and after every run entry (a test hook, as the reference's per-layer
        outputs of ``gpt2_gpu_forward_last``, engine/src/gpt2_gpu.cu:224-250).  A step
        that fails after its check (out of pages, a kernel that reports an error) leaves
        every request as it was."""
        self._validate(entries)
        n_want = sum(len(e.want) for e in entries)
        if sampling is not None and len(sampling) != n_want:
            raise StepError(f"{len(sampling)} sampling parameters for {n_want} wanted rows")
        self._reserve(entries)
        try:
            return self._step_reserved(entries, sampling, n_want, dump_hidden)
        except BaseException:
            # nothing was committed: the pages this step reserved go back, and every request
            # is as long as it was (what the step may have stored lies past that length)
            for entry in entries:
                self.cache.unreserve(entry.slot)
            raise

    def _step_reserved(self, entries, sampling, n_want, dump_hidden):
        n_tokens = sum(len(e.tokens) for e in entries)
        n_items = len(entries)
        any_previous = False
        ctx = self.ctx
        cache_length = self.cache.length
        if n_tokens == n_items and all(type(e.tokens[0]) is int and len(e.want) <= 1 for e in entries):
            # single tokens only (a decode step): the arrays straight from lists, no slices per entry
            slots = [e.slot for e in entries]
            starts = [cache_length(slot) for slot in slots]
            firsts = [e.tokens[0] for e in entries]
            any_previous = PREVIOUS in firsts
            if any_previous:
                firsts = [-1 - slot if t == PREVIOUS else t for t, slot in zip(firsts, slots)]
            token_ids = np.array(firsts, dtype=np.int32)
            positions = np.array(starts, dtype=np.int32)
            token_item = np.arange(n_items, dtype=np.int32)
            wanted = [(index, e.slot) for index, e in enumerate(entries) if e.want]
            want_rows = np.array([index for index, _ in wanted], dtype=np.int32)
            want_slots = np.array([slot for _, slot in wanted], dtype=np.int32)
            ctx.item_slots, ctx.item_starts = slots, starts
            ctx.item_counts, ctx.item_offsets = [1] * n_items, list(range(n_items))
        else:
            token_ids = np.empty(n_tokens, dtype=np.int32)
            positions = np.empty(n_tokens, dtype=np.int32)
            token_item = np.empty(n_tokens, dtype=np.int32)
            want_rows = np.empty(n_want, dtype=np.int32)
            want_slots = np.full(n_want, -1, dtype=np.int32)      # the entry's last wanted row is kept for its slot
            ctx.item_slots, ctx.item_starts, ctx.item_counts, ctx.item_offsets = [], [], [], []
            row = 0
            w = 0
            for index, entry in enumerate(entries):
                n = len(entry.tokens)
                start = cache_length(entry.slot)
                token_ids[row:row + n] = entry.tokens
                if token_ids[row] == PREVIOUS:
                    token_ids[row] = -1 - entry.slot
                    any_previous = True
                positions[row:row + n] = np.arange(start, start + n, dtype=np.int32)
                token_item[row:row + n] = index
                for place in entry.want:
                    want_rows[w] = row + int(place)
                    w += 1
                if entry.want:
                    want_slots[w - 1] = entry.slot
                ctx.item_slots.append(entry.slot)
                ctx.item_starts.append(start)
                ctx.item_counts.append(n)
                ctx.item_offsets.append(row)
                row += n
        tables = {group.index: group.table[ctx.item_slots] for group in self.cache.groups if group.paged}
        # A step of single tokens of few requests goes to the decode attention, which takes no
        # work list: none is made for it.
        decode_only = n_tokens == n_items
        # Where most of the step's tokens lie in portions longer than a tile, the list is made of
        # units of two tiles (measured: 21 against 28.5 us for two prompts of 1,024 tokens of
        # twelve heads, 36 against 30 us for sixteen portions of 128 tokens).
        heads = self.model.attention_unit_heads
        units = heads > 0 and 2 * sum(n for n in ctx.item_counts if n > ops.ATTENTION_TILE) >= n_tokens
        if not self.model.wants_attention_tiles or (decode_only and n_items <= SPLIT_ATTENTION_MAX_ROWS):
            tiles, n_split, most_parts, units = [], 0, 1, False
        elif units:
            tiles, n_split, most_parts = ops.attention_units(ctx.item_offsets, ctx.item_counts, ctx.item_starts, heads,
                                                             self._n_sms)
        else:
            tiles, n_split, most_parts = ops.attention_tiles(ctx.item_offsets, ctx.item_counts, ctx.item_starts)
        temperature = top_p = seeds = counters = None
        if sampling is not None:
            temperature = np.array([s.temperature for s in sampling], dtype=np.float32)
            top_p = np.array([s.top_p for s in sampling], dtype=np.float32)
            seeds = np.array([s.seed & 0xFFFFFFFFFFFFFFFF for s in sampling], dtype=np.uint64)
            counters = np.array([s.counter for s in sampling], dtype=np.int32)
        n_real_want = n_want
        if (not decode_only and not dump_hidden and self.cuda_graphs and self.model.graph_safe
                and n_want <= n_tokens and self._can_pad):
            # Steps with prompt portions come in endless shapes, and a captured graph serves one
            # shape.  So such a step is filled up to a round shape: tokens of a request that does
            # not exist (id 0 at position 0; its block table names the spare page that every
            # pool has beyond its last) bring the token count to a multiple of 64 (128 past 512
            # tokens), the entries to a multiple of 8, the wanted rows to a multiple of 8 (more
            # rows of the filler, or of row 0 when there is no filler row; drawn greedily and kept
            # for no request), the attention work list to a multiple of 4 (more tiles of the
            # filler's first row, if there is one).  Rows never mix, so the real rows' results
            # are what they would be alone; steps of one round shape replay one graph.
            step = 64 if n_tokens < 512 else 128
            filled = -(-n_tokens // step) * step
            extra = filled - n_tokens                     # (none, if the step is round already)
            token_ids = np.concatenate([token_ids, np.zeros(extra, dtype=np.int32)])
            positions = np.concatenate([positions, np.zeros(extra, dtype=np.int32)])
            token_item = np.concatenate([token_item, np.full(extra, n_items, dtype=np.int32)])
            items_filled = -(-(n_items + 1) // 8) * 8
            for group in self.cache.groups:
                if group.paged:
                    spare = np.full((items_filled - n_items, group.max_blocks), group.pool.n_pages, dtype=np.int32)
                    tables[group.index] = np.concatenate([tables[group.index], spare])
            if n_want > 0:
                want_filled = -(-n_want // 8) * 8
                more = want_filled - n_want
                want_rows = np.concatenate([want_rows, np.full(more, n_tokens if extra else 0, dtype=np.int32)])
                want_slots = np.concatenate([want_slots, np.full(more, -1, dtype=np.int32)])
                if sampling is not None:
                    temperature = np.concatenate([temperature, np.zeros(more, dtype=np.float32)])
                    top_p = np.concatenate([top_p, np.ones(more, dtype=np.float32)])
                    seeds = np.concatenate([seeds, np.zeros(more, dtype=np.uint64)])
                    counters = np.concatenate([counters, np.zeros(more, dtype=np.int32)])
                n_want = want_filled
            if tiles and extra:
                tiles = tiles + [(n_items, n_tokens, 1, 0, 0, 1, 0, 1)] * (-len(tiles) % 4)
            n_tokens, n_items = filled, items_filled
        arrays = {"token_ids": token_ids, "positions": positions, "token_item": token_item, "want_rows": want_rows,
                  "want_slots": want_slots, "att_tiles": np.array(tiles, dtype=np.int32)}
        for index, table in tables.items():
            arrays[("block_table", index)] = table
        if sampling is not None:
            arrays.update(temperature=temperature, top_p=top_p, seeds=seeds, counters=counters)
        # the one-kernel decode step takes its arrays from alternating buffers, so that the next
        # step's copy runs beside it; captured graphs have their addresses fixed
        fused = (self.fused is not None and not dump_hidden and n_want <= n_tokens
                 and self.fused.takes_sizes(n_tokens, decode_only))
        alternate = fused
        # a place may be wanted twice: the per-row arrays have room for the larger count
        views = self.control.upload(arrays, max(n_tokens, n_want), n_items, alternate)

        ctx.n_tokens, ctx.n_items, ctx.n_want = n_tokens, n_items, n_want
        ctx.token_ids, ctx.positions = views["token_ids"][:n_tokens], views["positions"][:n_tokens]
        ctx.token_item = views["token_item"][:n_tokens]
        ctx.want_rows = views["want_rows"][:n_want]
        ctx.want_slots = views["want_slots"][:n_want]
        ctx.any_previous = any_previous
        ctx.decode_only = decode_only
        ctx.fused = fused
        ctx.dump = [] if dump_hidden else None
        ctx.att_tiles, ctx.n_att_tiles = (views["att_tiles"] if tiles else None), len(tiles)
        ctx.n_split_tiles, ctx.att_parts, ctx.att_units = n_split, most_parts, units
        for view in self.storage.views:
            if view.kind == "paged":
                view.block_table = views[("block_table", view.group)]

        sample_views = None
        self._any_nucleus = sampling is not None and any(s.temperature > 0 and s.top_p < 1 for s in sampling)
        if sampling is not None and n_want > 0:
            sample_views = (views["temperature"][:n_want], views["top_p"][:n_want], views["seeds"][:n_want],
                            views["counters"][:n_want])
        self._turn ^= 1                       # the slot of the readback ring this step fills
        compute = torch.cuda.current_stream(self.device)
        # This step's kernels write their sampled ids where an earlier step left its own: that
        # step's copy to the host must be done.  Two steps that alternate use different buffers,
        # so the second need not wait for the first one's copy (it runs beside it).
        for slot in (self._turn, self._turn ^ 1):
            beside = slot != self._turn and alternate and self._alternated
            if self._readback[slot] is not None and not beside:
                compute.wait_event(self._readback[slot][2])
        self._alternated = alternate
        logits = self._run(ctx, sample_views)
        self.hidden_dump = ctx.dump
        self.control.consumed()
        for entry in entries:
            self.cache.commit(entry.slot, len(entry.tokens))
        self.steps += 1
        n_want = n_real_want                  # rows of the filler are nobody's
        if logits is not None and logits.shape[0] != n_want:
            logits = logits[:n_want]
        if self._sampled is not None:
            # the sampled ids start for the host right behind the step's kernels; for the steps
            # that alternate on a stream of their own, so that the next step's kernels do not
            # queue behind the copy
            held = self._readback[self._turn]
            if held is None or held[0].shape[0] < n_want:
                held = (torch.empty(max(n_want, 64), dtype=torch.int32).pin_memory(), 0, torch.cuda.Event())
            # with them comes the word in which a kernel reports a wait that ran out, so that
            # no token of a failed step is ever handed on
            status = self.kernels.status(self.device)
            if alternate:
                done = self._sampled_events[self._turn]
                done.record(compute)
                with torch.cuda.stream(self._readback_stream):
                    self._readback_stream.wait_event(done)
                    held[0][:n_want].copy_(self._sampled[:n_want], non_blocking=True)
                    self._status_pinned[self._turn:self._turn + 1].copy_(status, non_blocking=True)
                    held[2].record(self._readback_stream)
            else:
                held[0][:n_want].copy_(self._sampled[:n_want], non_blocking=True)
                self._status_pinned[self._turn:self._turn + 1].copy_(status, non_blocking=True)
                held[2].record(compute)
            self._readback[self._turn] = (held[0], n_want, held[2])
            for entry in entries:
                if entry.want:
                    self._kept_valid.add(entry.slot)
        elif self._readback[self._turn] is not None:
            self._readback[self._turn] = (self._readback[self._turn][0], 0, self._readback[self._turn][2])
        return logits

    # ---- running the model: eagerly, or as a replayed CUDA graph ---------------------------------
    def _forward(self, ctx, sample_views):
        with ops.launches_on_current_stream():
            return self._forward_on_stream(ctx, sample_views)

    def _forward_on_stream(self, ctx, sample_views):
        if ctx.any_previous:
            self.kernels.resolve_tokens(ctx.token_ids, self.kept_tokens)
        logits = self.model.forward(ctx, self.storage.views)
        self._sampled = None
        if sample_views is not None and logits is not None:
            out = self.workspace.get(f"sampled{self.control.parity}", (ctx.n_want,), torch.int32)
            self.kernels.sample_rows(out, logits, *sample_views, any_nucleus=self._any_nucleus)
            self.kernels.keep_tokens(self.kept_tokens, ctx.want_slots, out)
            self._sampled = out
        return logits

    def _run(self, ctx, sample_views):
        """Steps of one shape (tokens, entries, wanted rows, attention tiles) launch the same
        kernels with the same arguments (everything that changes lies in the control block on
        the device), so the second such step is captured into a CUDA graph and later ones
        replay it: a step then costs one launch on the host instead of one per kernel.  The reference removes host work per
        step in the same spirit, by keeping sampled tokens on the device
        (engine/src/gpt2_gpu_greedy.cu:80-119)."""
        if ctx.fused and self.fused is not None:
            block_table = next(v.block_table for v in self.storage.views if v.kind == "paged")
            try:
                logits, self._sampled = self.fused.run(ctx, block_table, sample_views, self._any_nucleus)
                self.step_kinds["one_kernel"] += 1
                return logits
            except KernelError as error:
                # for instance no cooperative launch on this device: say so once, then run the generic path
                print(f"[mini_llm_b200] fused decode step disabled: {error}", file=sys.stderr, flush=True)
                self.fused, self.fused_reason = None, str(error)
        if ctx.dump is not None or not (self.cuda_graphs and self.model.graph_safe):
            self.step_kinds["eager"] += 1
            return self._forward(ctx, sample_views)
        stamp = (self.workspace.generation, self.control.generation, self.kernels.scratch_generation)
        if stamp != self._graph_stamp:
            self._graphs.clear()                      # a buffer moved: captured addresses are stale
            self._graph_stamp = stamp
        # (how many units come in parts is data; that some do decides whether the kernel gets scratch)
        key = (ctx.n_tokens, ctx.n_items, ctx.n_want, ctx.n_att_tiles, ctx.att_parts > 1, ctx.att_units,
               sample_views is not None, self._any_nucleus, ctx.any_previous, self.control.parity)
        held = self._graphs.get(key)
        # A shape runs eagerly the first time (every buffer it needs gets allocated) and is
        # captured when it comes back: a capture costs about as much as two eager steps of a
        # prompt shape, so a shape that was seen twice pays for it at its third appearance.
        if held is None:
            if len(self._graphs) >= 192:
                self._graphs.clear()                  # many shapes came by: start over rather than grow
            self.step_kinds["eager"] += 1
            logits = self._forward(ctx, sample_views)
            self._graphs[key] = 1                     # ran once, its buffers exist: captured when it comes back
            return logits
        if isinstance(held, int):
            before = self.kernels.launches
            graph = torch.cuda.CUDAGraph()
            # "relaxed": only this engine's kernels are launched in here, but the collector may
            # free an older engine's pinned buffers meanwhile, whose allocator then queries events
            with torch.cuda.graph(graph, capture_error_mode="relaxed"):
                logits = self._forward(ctx, sample_views)
            if (self.workspace.generation, self.control.generation, self.kernels.scratch_generation) != stamp:
                raise RuntimeError("a buffer was allocated while a step was captured")
            held = (graph, logits, self._sampled, self.kernels.launches - before)
            self._graphs[key] = held
            self.kernels.launches = before
            self.step_kinds["captured"] += 1
            self.step_kinds["replayed"] -= 1
        graph, logits, self._sampled, launches = held
        graph.replay()
        self.step_kinds["replayed"] += 1
        self.kernels.launches += launches
        return logits

    def sampled_tokens(self, ago: int = 0) -> list:
        """The tokens the last step sampled (``ago=0``; waits for that step), or the step
        before it (``ago=1``: what a caller reads after it has launched the next step, whose
        entries name their tokens as PREVIOUS).  Older steps are not kept."""
        if ago not in (0, 1):
            raise ValueError("only the last two steps' tokens are kept")
        held = self._readback[self._turn ^ ago]
        if held is None or held[1] == 0:
            return []
        held[2].synchronize()
        code = int(self._status_host[self._turn ^ ago])
        if code != 0:
            self._recover(code)
        return held[0][:held[1]].tolist()

    def check_status(self) -> None:
        """Raise if a kernel gave up on one of its bounded waits since the last check
        (synchronises).  ``sampled_tokens`` checks by itself; callers that read logits only
        (trace replay) call this."""
        code = self.kernels.read_status()
        if code != 0:
            self._recover(code)

    def _recover(self, code: int):
        """A kernel gave up on a bounded wait: the step's results are invalid.  CTAs of such a
        kernel leave at different points, so every counter the kernels share across launches
        (the grid barrier's arrival count, the attention kernels' work and merge counters) is
        put back to its start, and captured graphs are dropped, before the error is raised:
        the next step then runs on clean state."""
        torch.cuda.synchronize(self.device)
        self.kernels.reset_after_failure()
        if self.fused is not None:
            self.fused.reset()
        self._graphs.clear()
        self._status_host[:] = 0
        self._readback = [None, None]
        raise KernelError(f"a kernel gave up on a bounded wait (code {code}): the step's results are invalid; "
                          f"the requests of that step should be closed")

    # ---- looking inside (tests) ---------------------------------------------------------------
    def read_kv(self, slot: int, run_entry: int, first: int = 0, count: int | None = None):
        """Keys and values of ``count`` cached tokens of the request in ``slot``, from token
        ``first`` on, as run entry ``run_entry`` holds them: ``(k, v)``, each
        ``[count, kv_heads, head_size]`` on the device, gathered through the request's block
        table (the reference's ``gpt2_gpu_kv_cache_copy_layer``, engine/src/gpt2_gpu.cu:185-195)."""
        length = self.cache.length(slot)
        if count is None:
            count = length - first
        if first < 0 or count < 0 or first + count > length:
            raise ValueError(f"tokens {first}..{first + count - 1} are not among the {length} the request holds")
        torch.cuda.current_stream(self.device).synchronize()
        return self.storage.read_tokens(run_entry, slot, first, count)
