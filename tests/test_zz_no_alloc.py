"""split_attention for callers that cannot allocate device memory.

Some users of the decode library are plain C hosts: they load ``libmllm_decode`` and call its
exported symbols, with no caching allocator behind them and a device memory budget that was
settled at start-up (and a cudaMalloc or cudaFree in their loop would stall the whole device).
For them ``mllm_decode_split_attention_static`` carries its scratch inside the library.  This
test calls it the way they do, through the exported C symbol, twice in a row on the shared
scratch, and compares with the entry point that takes the caller's scratch.  It is collected
last, so a run that stops at the first failure has run every other test before it.
"""

import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, L, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_long, ctypes.c_float
ATOL = 3.2e-2          # the bfloat16 tolerance the other attention tests use (2 x 1.6e-2)


def load_symbol():
    from mini_llm_b200.kernels import build
    lib = ctypes.CDLL(build.library_path("decode"))
    fn = lib.mllm_decode_split_attention_static
    fn.argtypes = [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, F, I, I, P]
    fn.restype = I
    lib.mllm_decode_last_error.restype = ctypes.c_char_p
    return lib, fn


def make_case(seed, lengths, heads, kv_heads, head, page):
    rng = np.random.default_rng(seed)
    width = kv_heads * head
    max_blocks = max(-(-n // page) for n in lengths) + 2
    n_pages = sum(-(-n // page) for n in lengths) + 3
    order = rng.permutation(n_pages)
    table = np.full((len(lengths), max_blocks), -1, dtype=np.int32)
    used = 0
    for i, n in enumerate(lengths):
        for b in range(-(-n // page)):
            table[i, b] = order[used]
            used += 1
    dev = lambda a, dt=None: (torch.as_tensor(a).cuda().to(dt) if dt else torch.as_tensor(a).cuda())
    return (dev(rng.normal(size=(len(lengths), heads * head)), torch.bfloat16),
            dev(rng.normal(size=(n_pages, page, width)), torch.bfloat16),
            dev(rng.normal(size=(n_pages, page, width)), torch.bfloat16), dev(table),
            dev(np.array([n - 1 for n in lengths], dtype=np.int32)), dev(np.arange(len(lengths), dtype=np.int32)))


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    from mini_llm_b200.kernels import ops
    lib, fn = load_symbol()
    stream = torch.cuda.current_stream().cuda_stream
    # two calls of different shapes, one after the other, on the same built-in scratch
    for seed, (lengths, heads, kv_heads, head, page, chunk, window) in enumerate([
            ([300, 1, 77, 129, 64], 6, 2, 64, 16, 64, 0), ([513, 40, 2], 4, 4, 32, 8, 128, 50)]):
        q, k_pages, v_pages, table, positions, items = make_case(seed, lengths, heads, kv_heads, head, page)
        scale = 1.0 / math.sqrt(head)
        n = len(lengths)
        max_chunks = -(-(table.shape[1] * page) // chunk)
        want = torch.empty_like(q)
        ops.split_attention(want, q, k_pages, v_pages, table, positions, items, heads, kv_heads, head, page, scale,
                            window, chunk, max_chunks,
                            torch.empty(n * heads * max_chunks * head, device="cuda"),
                            torch.empty(n * heads * max_chunks * 2, device="cuda"),
                            torch.zeros(n * heads, dtype=torch.int32, device="cuda"))
        for call in range(2):
            got = torch.full_like(q, float("nan"))
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]
            torch_before = torch.cuda.memory_stats()["allocation.all.allocated"]
            status = fn(got.data_ptr(), got.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(),
                        v_pages.data_ptr(), table.data_ptr(), table.shape[1], positions.data_ptr(), items.data_ptr(),
                        n, heads, kv_heads, head, page, scale, window, chunk, stream)
            assert status == 0, lib.mllm_decode_last_error().decode()
            torch.cuda.synchronize()
            # nothing was allocated: neither through torch nor from the driver (the first call on
            # a device may make the driver load the library's module, so the driver's figure is
            # compared on the later calls)
            assert torch.cuda.memory_stats()["allocation.all.allocated"] == torch_before
            if call > 0 or seed > 0:
                assert torch.cuda.mem_get_info()[0] == free_before
            np.testing.assert_allclose(got.float().cpu().numpy(), want.float().cpu().numpy(), rtol=0, atol=ATOL)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib, fn = load_symbol()
    q, k_pages, v_pages, table, positions, items = make_case(3, [20, 30], 4, 4, 64, 16)
    out = torch.full_like(q, 5.0)
    # 4200 heads: more (token, head) pairs than there are counters
    status = fn(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                table.data_ptr(), table.shape[1], positions.data_ptr(), items.data_ptr(), 2, 4200, 4200, 64, 16,
                0.125, 0, 64, torch.cuda.current_stream().cuda_stream)
    assert status != 0 and b"exceed the built-in scratch" in lib.mllm_decode_last_error()
    torch.cuda.synchronize()
    assert float(out.float().min()) == 5.0 == float(out.float().max())       # nothing ran
