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
    """The step's token arrays and block tables in one int32 device buffer, written with a
    single copy from pinned host memory.

    There are two device buffers.  Steps that ask for it (``alternate``) use them in turn and
    copy on a stream of their own: the arrays of step k+1 are on the device while the kernels
    of step k still read theirs, so no copy stands between two steps' kernels; a step's kernels
    wait for their copy, and a copy waits for the kernels that read the buffer it overwrites
    (``consumed`` records them).  Other steps keep to the first buffer (their kernels are
    replayed from graphs with fixed addresses) and copy in the order of the compute stream."""

    def __init__(self, device, groups):
        self.device = device
        self.groups = [(g.index, g.max_blocks) for g in groups if g.paged]
        self.capacity = 0
        self.device_buffers = [None, None]
        self.copy_stream = torch.cuda.Stream(device=device)
        self._host = []
        self._layouts = {}
        self.parity = 0
        self.generation = 0
        self.last_upload_bytes = 0            # bytes of the last step's host-to-device copy

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
        torch.cuda.synchronize(self.device)      # nothing may still read or fill the old buffers
        self.capacity = max(size, 2 * self.capacity, 4096)
        self.device_buffers = [torch.zeros(self.capacity, dtype=torch.int32, device=self.device) for _ in range(2)]
        self._host = [torch.zeros(self.capacity, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._host_np = [h.numpy() for h in self._host]
        self._copied = [torch.cuda.Event(), torch.cuda.Event()]       # the copy out of host buffer t is done
        self._copied_once = [False, False]
        self._host_turn = 0
        self._consumed = [torch.cuda.Event(), torch.cuda.Event()]     # the kernels that read device buffer p are done
        self._in_use = [False, False]
        self._layouts = {}                   # (parity, tokens, entries) -> (offsets, size, device views)
        self.generation += 1

    def upload(self, arrays: dict, n_tokens: int, n_items: int, alternate: bool = True):
        """``arrays``: name -> numpy array (int32, or float32/int64 viewed as
        int32).  Returns name -> device view (of this step's buffer).  ``alternate=False``
        keeps to the first buffer: steps whose kernels are replayed from a captured graph
        (fixed addresses) use that, and wait for the step before them."""
        self.parity = (self.parity ^ 1) if alternate else 0
        parity = self.parity
        key = (parity, n_tokens, n_items)
        held = self._layouts.get(key)
        if held is None:
            offsets, size = self._layout(n_tokens, n_items)
            self._ensure(size)               # may drop every cached layout
            held = self._layouts[key] = (offsets, size, self._views(self.device_buffers[parity], offsets, n_tokens, n_items))
        offsets, size, views = held
        self.last_upload_bytes = 4 * size
        # host side: two pinned buffers in turn; the copy that last read this one must be done
        self._host_turn ^= 1
        turn = self._host_turn
        if self._copied_once[turn]:
            self._copied[turn].synchronize()
        host_np = self._host_np[turn]
        for name, values in arrays.items():
            flat = np.ascontiguousarray(values).reshape(-1).view(np.int32)
            start = offsets[name]
            host_np[start:start + flat.size] = flat
        compute = torch.cuda.current_stream(self.device)
        if alternate:
            # beside the kernels of the step before; behind the kernels that last read this buffer
            with torch.cuda.stream(self.copy_stream):
                if self._in_use[parity]:
                    self.copy_stream.wait_event(self._consumed[parity])
                self.device_buffers[parity][:size].copy_(self._host[turn][:size], non_blocking=True)
                self._copied[turn].record(self.copy_stream)
            compute.wait_event(self._copied[turn])
        else:
            # in the order of the compute stream: behind everything that read the buffer
            self.device_buffers[parity][:size].copy_(self._host[turn][:size], non_blocking=True)
            self._copied[turn].record(compute)
        self._copied_once[turn] = True
        return views

    def consumed(self) -> None:
        """Call after the step's kernels are enqueued: its buffer may be overwritten once they
        are done."""
        self._consumed[self.parity].record(torch.cuda.current_stream(self.device))
        self._in_use[self.parity] = True

    def _views(self, buffer, offsets, n_tokens: int, n_items: int):
        views = {}
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
        self.fused = False            # the step goes to the one-kernel decode step
        self.dump = None              # a list: the model appends the residual stream after every run entry
        self.att_tiles = None         # device work list (tiles of up to 128 tokens of one entry), or None
        self.n_att_tiles = 0          # records (CTAs) of the work list
        self.n_split_tiles = 0        # tiles among them that come in several parts
        self.att_parts = 1            # most parts of a tile
        self.att_units = False        # the work list holds units of up to 256 tokens (two tiles) instead of tiles

    def buffer(self, tag: str, shape, dtype):
        return self.workspace.get(tag, shape, dtype)
