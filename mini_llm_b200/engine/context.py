"""What a step hands to the parts: the flattened batch and scratch memory.

All tokens of a step form one batch of T rows.  For row t: ``token_ids[t]``,
its absolute position in its request ``positions[t]``, and ``token_item[t]``,
the index of its entry in the step (the row of every block table).  These and
the block tables lie in one device buffer that is written with one copy per
step (the reference's ``BatchControl`` idea, engine/src/gpt2_gpu_batch.cu:18-24,
91-113); kernels read everything from there.
"""

from __future__ import annotations

import numpy as np
import torch


class Workspace:
    """Named scratch tensors, reused across layers and steps.  A buffer is
    allocated with room for ``min_rows`` rows and grows when a step needs more."""

    def __init__(self, device, min_rows: int):
        self.device = device
        self.min_rows = int(min_rows)
        self._buffers = {}
        self.generation = 0          # grows whenever a buffer moves (captured graphs are then stale)

    def get(self, tag: str, shape, dtype):
        rows, rest = int(shape[0]), tuple(int(s) for s in shape[1:])
        key = (tag, dtype, rest)
        held = self._buffers.get(key)
        if held is None or held.shape[0] < rows:
            capacity = max(rows, self.min_rows if held is None else 2 * held.shape[0])
            if tag == "logits":
                capacity = rows if held is None else max(rows, held.shape[0])
            held = torch.empty((capacity, *rest), dtype=dtype, device=self.device)
            self._buffers[key] = held
            self.generation += 1
        return held[:rows]


class ControlBlock:
    """One int32 device buffer with the step's token arrays and block tables,
    filled through pinned host memory with a single copy."""

    def __init__(self, device, groups):
        self.device = device
        self.groups = [(g.index, g.max_blocks) for g in groups if g.paged]
        self.capacity = 0
        self.device_buffer = None
        self._host = []
        self._events = []
        self._layouts = {}
        self._turn = 0
        self.generation = 0

    @staticmethod
    def tile_ints(n_tokens: int, n_items: int) -> int:
        """Room for the attention work list: at most n_tokens // 128 + n_items tiles, each in
        at most 8 parts, 8 int32 per record."""
        return 8 * 8 * (n_tokens // 128 + n_items)

    def _layout(self, n_tokens: int, n_items: int):
        """Offsets (in int32 units) as a function of the step's sizes only, so
        that steps of equal sizes find their arrays at equal addresses."""
        offsets = {}
        cursor = 0
        for name in ("token_ids", "positions", "token_item", "want_rows", "want_slots", "counters", "temperature",
                     "top_p"):
            offsets[name] = cursor
            cursor += n_tokens
        cursor += cursor & 1                      # 8-byte alignment for the 64-bit seeds
        offsets["seeds"] = cursor
        cursor += 2 * n_tokens
        offsets["att_tiles"] = cursor             # work list of the prompt-attention kernel
        cursor += self.tile_ints(n_tokens, n_items)
        for index, max_blocks in self.groups:
            offsets[("block_table", index)] = cursor
            cursor += n_items * max_blocks
        return offsets, cursor

    def _ensure(self, size: int):
        if size <= self.capacity:
            return
        self.capacity = max(size, 2 * self.capacity, 4096)
        self.device_buffer = torch.zeros(self.capacity, dtype=torch.int32, device=self.device)
        self._host = [torch.zeros(self.capacity, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._host_np = [h.numpy() for h in self._host]
        self._events = [torch.cuda.Event(), torch.cuda.Event()]
        self._recorded = [False, False]
        self._layouts = {}                   # (tokens, entries) -> (offsets, size, device views)
        self.generation += 1

    def upload(self, arrays: dict, n_tokens: int, n_items: int):
        """``arrays``: name -> numpy array (int32, or float32/int64 viewed as
        int32).  Returns name -> device view."""
        key = (n_tokens, n_items)
        held = self._layouts.get(key)
        if held is None:
            offsets, size = self._layout(n_tokens, n_items)
            self._ensure(size)               # may drop every cached layout
            held = self._layouts[key] = (offsets, size, self._views(offsets, n_tokens, n_items))
        offsets, size, views = held
        self._turn ^= 1
        turn = self._turn
        if self._recorded[turn]:
            self._events[turn].synchronize()  # the copy that last used this host buffer is done
        host_np = self._host_np[turn]
        for name, values in arrays.items():
            flat = np.ascontiguousarray(values).reshape(-1).view(np.int32)
            start = offsets[name]
            host_np[start:start + flat.size] = flat
        self.device_buffer[:size].copy_(self._host[turn][:size], non_blocking=True)
        self._events[turn].record()
        self._recorded[turn] = True
        return views

    def _views(self, offsets, n_tokens: int, n_items: int):
        views = {}
        buffer = self.device_buffer
        for name, start in offsets.items():
            if name == "seeds":
                views[name] = buffer[start:start + 2 * n_tokens].view(torch.int64)
            elif name in ("temperature", "top_p"):
                views[name] = buffer[start:start + n_tokens].view(torch.float32)
            elif name == "att_tiles":
                views[name] = buffer[start:start + self.tile_ints(n_tokens, n_items)]
            elif isinstance(name, tuple):
                max_blocks = dict(self.groups)[name[1]]
                views[name] = buffer[start:start + n_items * max_blocks].view(n_items, max_blocks)
            else:
                views[name] = buffer[start:start + n_tokens]
        return views


class StepContext:
    """The batch of one step, as the parts see it."""

    def __init__(self, kernels, workspace, act_dtype, device):
        self.kernels = kernels
        self.workspace = workspace
        self.act_dtype = act_dtype
        self.device = device
        self.n_tokens = 0
        self.n_items = 0
        self.n_want = 0
        self.token_ids = self.positions = self.token_item = self.want_rows = self.want_slots = None
        self.any_previous = False     # some token id is negative: -1 - slot names that slot's last sampled token
        self.item_slots = []          # host: slot of each entry
        self.item_starts = []         # host: position of each entry's first token
        self.item_counts = []         # host: tokens of each entry
        self.item_offsets = []        # host: row of each entry's first token
        self.decode_only = False      # every entry brings exactly one token
        self.att_tiles = None         # device work list (tiles of up to 128 tokens of one entry), or None
        self.n_att_tiles = 0          # records (CTAs) of the work list
        self.n_split_tiles = 0        # tiles among them that come in several parts
        self.att_parts = 1            # most parts of a tile

    def buffer(self, tag: str, shape, dtype):
        return self.workspace.get(tag, shape, dtype)
