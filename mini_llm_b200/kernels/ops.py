"""The operations of a step, as functions over CUDA tensors.

Every function checks what its kernel assumes (device, element types, inner
stride, sizes), then launches on torch's current stream.  There is no CPU
path: a tensor that is not on a CUDA device is an error.  The plain kernels
take every size; a fast kernel either takes a size or is not chosen for it.
"""

from __future__ import annotations

import ctypes

import torch

from .lib import F, I, L, P, Function, KernelError, set_dependent_launch  # noqa: F401  (re-exported)

DT_F32, DT_BF16 = 0, 1
EPILOGUES = {"store": 0, "gelu_tanh": 1, "gelu_erf": 2, "add": 3}

_DTYPE_CODE = {torch.float32: DT_F32, torch.bfloat16: DT_BF16}


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {dtype}") from None


_pinned_stream = None


def _stream() -> int:
    """The stream launches go to: the current stream, looked up per launch, or the one a
    caller pinned for a run of launches (the lookup costs more than a launch's own checks)."""
    return _pinned_stream if _pinned_stream is not None else torch.cuda.current_stream().cuda_stream


class launches_on_current_stream:
    """Within the block every launch of this module goes to the stream that is current at
    entry (do not switch streams inside)."""

    def __enter__(self):
        global _pinned_stream
        self.before = _pinned_stream
        _pinned_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _pinned_stream
        _pinned_stream = self.before
        return False


def _check(t: torch.Tensor, name: str, dtype=None, dims=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name}: expected a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: expected {dtype}, got {t.dtype}")
    if dims is not None and t.dim() != dims:
        raise KernelError(f"{name}: expected {dims} dimensions, got shape {tuple(t.shape)}")
    if t.dim() > 0 and t.numel() > 0 and t.stride(-1) != 1:
        raise KernelError(f"{name}: the last dimension must be contiguous")


def _ptr(t):
    return None if t is None else t.data_ptr()


_embed = Function("plain", "mllm_plain_embed", [P, P, P, P, P, I, I, I, P])
_add_rows = Function("plain", "mllm_plain_add_rows", [P, P, P, I, I, I, P])
_layernorm = Function("plain", "mllm_plain_layernorm", [P, P, P, P, P, I, I, F, I, P])
_linear = Function("plain", "mllm_plain_linear", [P, P, P, P, I, I, I, L, L, I, I, I, P])
_kv_store = Function("plain", "mllm_plain_kv_store", [P, P, P, P, L, P, P, P, I, I, I, I, I, P])
_attention = Function("plain", "mllm_plain_attention",
                      [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, F, I, I, P])
_sample_rows = Function("sampling", "mllm_sampling_sample_rows", [P, P, L, I, I, P, P, P, P, P])


def embed(out, token_ids, positions, table, position_table=None):
    """out[t] = table[token_ids[t]] (+ position_table[positions[t]]); out is fp32 [T, width]."""
    _check(out, "embed.out", torch.float32, 2)
    _check(token_ids, "embed.token_ids", torch.int32, 1)
    _check(table, "embed.table", None, 2)
    n, width = out.shape
    if not out.is_contiguous() or not table.is_contiguous():
        raise KernelError("embed: out and table must be contiguous")
    if table.shape[1] != width or token_ids.shape[0] < n:
        raise KernelError("embed: sizes do not agree")
    if position_table is not None:
        _check(position_table, "embed.position_table", table.dtype, 2)
        _check(positions, "embed.positions", torch.int32, 1)
        if position_table.shape[1] != width or not position_table.is_contiguous():
            raise KernelError("embed: position table has another width")
    _embed(out.data_ptr(), token_ids.data_ptr(), _ptr(positions), table.data_ptr(), _ptr(position_table),
           n, width, dtype_code(table.dtype), _stream())
    return out


def add_position_rows(hidden, positions, table):
    """hidden[t] += table[positions[t]]."""
    _check(hidden, "add_position_rows.hidden", torch.float32, 2)
    _check(positions, "add_position_rows.positions", torch.int32, 1)
    _check(table, "add_position_rows.table", None, 2)
    if not hidden.is_contiguous() or not table.is_contiguous() or table.shape[1] != hidden.shape[1]:
        raise KernelError("add_position_rows: sizes do not agree")
    _add_rows(hidden.data_ptr(), positions.data_ptr(), table.data_ptr(), hidden.shape[0], hidden.shape[1],
              dtype_code(table.dtype), _stream())
    return hidden


def layernorm(out, x, gamma, beta, eps, rows=None):
    """out[r] = LN(x[rows[r]] or x[r]); x fp32 [*, width]; out fp32 or bf16 [R, width]."""
    _check(out, "layernorm.out", None, 2)
    _check(x, "layernorm.x", torch.float32, 2)
    _check(gamma, "layernorm.gamma", torch.float32, 1)
    _check(beta, "layernorm.beta", torch.float32, 1)
    width = x.shape[1]
    if not x.is_contiguous() or not out.is_contiguous():
        raise KernelError("layernorm: x and out must be contiguous")
    if out.shape[1] != width or gamma.shape[0] != width or beta.shape[0] != width:
        raise KernelError("layernorm: widths do not agree")
    if rows is not None:
        _check(rows, "layernorm.rows", torch.int32, 1)
        if rows.shape[0] < out.shape[0]:
            raise KernelError("layernorm: fewer row indices than output rows")
    elif x.shape[0] < out.shape[0]:
        raise KernelError("layernorm: fewer input rows than output rows")
    _layernorm(out.data_ptr(), x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), _ptr(rows),
               out.shape[0], width, float(eps), dtype_code(out.dtype), _stream())
    return out


def linear_plain(out, a, w, bias=None, epilogue="store"):
    """out = epilogue(a @ w.T + bias); a [M, K], w [N, K] (K contiguous), out [M, N].

    epilogue "add": out (fp32) += a @ w.T + bias.
    """
    _check(out, "linear.out", None, 2)
    _check(a, "linear.a", None, 2)
    _check(w, "linear.w", a.dtype, 2)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n or not w.is_contiguous():
        raise KernelError(f"linear: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if bias is not None:
        _check(bias, "linear.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("linear: bias has another length")
    _linear(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), out.stride(0),
            dtype_code(a.dtype), dtype_code(out.dtype), EPILOGUES[epilogue], _stream())
    return out


def kv_store(k_pages, v_pages, k_src, v_src, positions, token_item, block_table, page_size):
    """Write this step's keys and values (rows of k_src, v_src: [T, width]) into their pages."""
    _check(k_pages, "kv_store.k_pages")
    _check(v_pages, "kv_store.v_pages", k_pages.dtype)
    _check(k_src, "kv_store.k_src", k_pages.dtype, 2)
    _check(v_src, "kv_store.v_src", k_pages.dtype, 2)
    _check(block_table, "kv_store.block_table", torch.int32, 2)
    _check(positions, "kv_store.positions", torch.int32, 1)
    _check(token_item, "kv_store.token_item", torch.int32, 1)
    n, width = k_src.shape
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("kv_store: pages and block table must be contiguous")
    if k_src.stride(0) != v_src.stride(0) or v_src.shape != k_src.shape:
        raise KernelError("kv_store: keys and values must share shape and row stride")
    if k_pages.numel() % (page_size * width) != 0:
        raise KernelError("kv_store: page pool does not hold whole pages of this width")
    _kv_store(k_pages.data_ptr(), v_pages.data_ptr(), k_src.data_ptr(), v_src.data_ptr(), k_src.stride(0),
              positions.data_ptr(), token_item.data_ptr(), block_table.data_ptr(), block_table.shape[1],
              page_size, width, n, dtype_code(k_pages.dtype), _stream())


def attention_plain(out, q, k_pages, v_pages, block_table, positions, token_item, n_heads, n_kv_heads,
                    head_size, page_size, scale, window=0):
    """Causal attention of every token of the step over its request's pages."""
    _check(out, "attention.out", q.dtype, 2)
    _check(q, "attention.q", None, 2)
    _check(k_pages, "attention.k_pages", q.dtype)
    _check(v_pages, "attention.v_pages", q.dtype)
    _check(block_table, "attention.block_table", torch.int32, 2)
    _check(positions, "attention.positions", torch.int32, 1)
    _check(token_item, "attention.token_item", torch.int32, 1)
    n = q.shape[0]
    if q.shape[1] != n_heads * head_size or out.shape[1] != n_heads * head_size or out.shape[0] != n:
        raise KernelError("attention: q / out do not have heads * head_size columns")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("attention: pages and block table must be contiguous")
    _attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
               block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), token_item.data_ptr(), n,
               n_heads, n_kv_heads, head_size, page_size, float(scale), int(window or 0),
               dtype_code(q.dtype), _stream())
    return out


def sample_rows(out, logits, temperature=None, top_p=None, seeds=None, counters=None):
    """One token per row of fp32 logits [R, V] into out (int32 [R]).

    temperature / top_p: fp32 [R] or None (greedy / no cut); seeds: int64 [R]
    (bit pattern of a u64); counters: int32 [R].
    """
    _check(out, "sample_rows.out", torch.int32, 1)
    _check(logits, "sample_rows.logits", torch.float32, 2)
    r, vocab = logits.shape
    if out.shape[0] < r:
        raise KernelError("sample_rows: output too short")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("seeds", seeds, torch.int64), ("counters", counters, torch.int32)):
        if t is not None:
            _check(t, f"sample_rows.{name}", dt, 1)
            if t.shape[0] < r:
                raise KernelError(f"sample_rows: {name} too short")
    _sample_rows(out.data_ptr(), logits.data_ptr(), logits.stride(0), r, vocab, _ptr(temperature), _ptr(top_p),
                 _ptr(seeds), _ptr(counters), _stream())
    return out


# ---- kernels for steps of few tokens (bfloat16) --------------------------------------------------

class _SkinnyParams(ctypes.Structure):
    _fields_ = [("out", P), ("x", P), ("w", P), ("bias", P), ("gamma", P), ("beta", P), ("rows", P),
                ("eps", F), ("M", I), ("N", I), ("K", I), ("ldx", L), ("ldo", L), ("epilogue", I), ("out_f32", I),
                ("k_pages", P), ("v_pages", P), ("positions", P), ("token_item", P), ("block_table", P),
                ("max_blocks", I), ("page_size", I), ("q_width", I), ("kv_width", I)]


_skinny = Function("decode", "mllm_decode_skinny_linear", [ctypes.POINTER(_SkinnyParams), P])
_split_attention = Function("decode", "mllm_decode_split_attention",
                            [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, F, I, I, I, P, P, P, P])

SKINNY_MAX_SMEM = 200 * 1024
SPLIT_ATTENTION_HEAD_SIZES = (16, 32, 64, 128, 256)


def skinny_linear_takes(m, k) -> bool:
    """Whether skinny_linear takes a product with ``m`` rows and inner size ``k``."""
    rows = 1 if m <= 1 else 2 if m <= 2 else 4 if m <= 4 else 8 if m <= 8 else 16
    return k % 8 == 0 and rows * k * 2 <= SKINNY_MAX_SMEM


def skinny_linear(out, x, w, bias=None, epilogue="store", norm=None, scatter=None):
    """out = epilogue(norm?(x) @ w.T + bias) for few rows (bf16 weights, fp32 sums).

    norm: (gamma, beta, eps, rows or None): x is then the fp32 residual stream and is
    layer-normed on the way in.  scatter: (k_pages, v_pages, positions, token_item,
    block_table, page_size, q_width, kv_width): columns past q_width are written into the
    cache pages instead of ``out`` (which then has q_width columns).
    """
    _check(w, "skinny_linear.w", torch.bfloat16, 2)
    n, k = w.shape
    params = _SkinnyParams()
    if norm is not None:
        gamma, beta, eps, rows = norm
        _check(x, "skinny_linear.x", torch.float32, 2)
        _check(gamma, "skinny_linear.gamma", torch.float32, 1)
        _check(beta, "skinny_linear.beta", torch.float32, 1)
        if not x.is_contiguous() or x.shape[1] != k or gamma.shape[0] != k or beta.shape[0] != k:
            raise KernelError("skinny_linear: the normed input does not have K contiguous columns")
        if rows is not None:
            _check(rows, "skinny_linear.rows", torch.int32, 1)
        m = rows.shape[0] if rows is not None else x.shape[0]
        params.gamma, params.beta, params.rows, params.eps = gamma.data_ptr(), beta.data_ptr(), _ptr(rows), float(eps)
    else:
        _check(x, "skinny_linear.x", torch.bfloat16, 2)
        if x.shape[1] != k:
            raise KernelError("skinny_linear: x and w disagree on K")
        m = x.shape[0]
    _check(out, "skinny_linear.out", None, 2)
    if not w.is_contiguous() or not skinny_linear_takes(m, k):
        raise KernelError(f"skinny_linear does not take M={m}, K={k}")
    out_cols = n if scatter is None else scatter[6]
    if out.shape[0] != m or out.shape[1] != out_cols:
        raise KernelError(f"skinny_linear: out is {tuple(out.shape)}, expected {(m, out_cols)}")
    if epilogue == "add" and out.dtype != torch.float32:
        raise KernelError("skinny_linear: the residual sum is kept in 32-bit")
    if epilogue != "add" and out.dtype not in (torch.float32, torch.bfloat16):
        raise KernelError("skinny_linear: out must be bfloat16 or float32")
    if bias is not None:
        _check(bias, "skinny_linear.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("skinny_linear: bias has another length")
    params.out, params.x, params.w, params.bias = out.data_ptr(), x.data_ptr(), w.data_ptr(), _ptr(bias)
    params.M, params.N, params.K = m, n, k
    params.ldx, params.ldo = x.stride(0), out.stride(0)
    params.epilogue = EPILOGUES[epilogue]
    params.out_f32 = int(out.dtype == torch.float32 and epilogue != "add")
    if scatter is not None:
        k_pages, v_pages, positions, token_item, block_table, page_size, q_width, kv_width = scatter
        _check(k_pages, "skinny_linear.k_pages", torch.bfloat16)
        _check(v_pages, "skinny_linear.v_pages", torch.bfloat16)
        _check(block_table, "skinny_linear.block_table", torch.int32, 2)
        if q_width + 2 * kv_width != n or not k_pages.is_contiguous() or not v_pages.is_contiguous():
            raise KernelError("skinny_linear: scatter widths do not add up to N")
        params.k_pages, params.v_pages = k_pages.data_ptr(), v_pages.data_ptr()
        params.positions, params.token_item = positions.data_ptr(), token_item.data_ptr()
        params.block_table, params.max_blocks = block_table.data_ptr(), block_table.shape[1]
        params.page_size, params.q_width, params.kv_width = page_size, q_width, kv_width
    _skinny(ctypes.byref(params), _stream())
    return out


def split_attention(out, q, k_pages, v_pages, block_table, positions, token_item, n_heads, n_kv_heads, head_size,
                    page_size, scale, window, chunk, max_chunks, part_acc, part_ml, counters):
    """Causal attention over the paged cache for few tokens: one CTA per (token, head, chunk
    of ``chunk`` keys); needs fp32 scratch ``part_acc`` [T*H*max_chunks*D], ``part_ml``
    [T*H*max_chunks*2] and zeroed int32 ``counters`` [T*H] (left zero)."""
    _check(out, "split_attention.out", torch.bfloat16, 2)
    _check(q, "split_attention.q", torch.bfloat16, 2)
    _check(k_pages, "split_attention.k_pages", torch.bfloat16)
    _check(v_pages, "split_attention.v_pages", torch.bfloat16)
    _check(block_table, "split_attention.block_table", torch.int32, 2)
    _check(part_acc, "split_attention.part_acc", torch.float32)
    _check(part_ml, "split_attention.part_ml", torch.float32)
    _check(counters, "split_attention.counters", torch.int32)
    n = q.shape[0]
    cells = n * n_heads * max_chunks
    if head_size not in SPLIT_ATTENTION_HEAD_SIZES:
        raise KernelError(f"split_attention does not take head size {head_size}")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape:
        raise KernelError("split_attention: q / out do not have heads * head_size columns")
    if part_acc.numel() < cells * head_size or part_ml.numel() < cells * 2 or counters.numel() < n * n_heads:
        raise KernelError("split_attention: scratch too small")
    if max_chunks * chunk < page_size * block_table.shape[1]:
        raise KernelError("split_attention: the chunks do not cover the longest block table")
    _split_attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                     block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), token_item.data_ptr(), n,
                     n_heads, n_kv_heads, head_size, page_size, float(scale), int(window or 0), int(chunk),
                     int(max_chunks), part_acc.data_ptr(), part_ml.data_ptr(), counters.data_ptr(), _stream())
    return out


_group_attention = Function("decode", "mllm_decode_group_attention",
                            [P, L, P, L, P, P, P, I, P, P, I, I, I, I, I, F, I, I, I, P, P, P, P])
GROUP_ATTENTION_HEAD_SIZES = (64, 128)


def group_attention_takes(q, n_heads, n_kv_heads, head_size) -> bool:
    """Whether ``group_attention`` takes the layout: bfloat16, head size 64 or 128, at most
    eight query heads per key/value head, rows of q on 16-byte boundaries."""
    return (q.dtype == torch.bfloat16 and head_size in GROUP_ATTENTION_HEAD_SIZES and n_kv_heads > 0
            and n_heads % n_kv_heads == 0 and n_heads // n_kv_heads <= 8 and q.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0)


def group_attention(out, q, k_pages, v_pages, block_table, positions, token_item, n_heads, n_kv_heads, head_size,
                    page_size, scale, window, chunk, max_chunks, part_acc, part_ml, counters):
    """``split_attention`` with the products on mma.sync tiles: one CTA per (token, key/value
    head, chunk of keys), the query heads of the group as the rows of the tiles.  Same
    arguments and scratch; ``chunk`` must be a multiple of 16."""
    _check(out, "group_attention.out", torch.bfloat16, 2)
    _check(q, "group_attention.q", torch.bfloat16, 2)
    _check(k_pages, "group_attention.k_pages", torch.bfloat16)
    _check(v_pages, "group_attention.v_pages", torch.bfloat16)
    _check(block_table, "group_attention.block_table", torch.int32, 2)
    _check(part_acc, "group_attention.part_acc", torch.float32)
    _check(part_ml, "group_attention.part_ml", torch.float32)
    _check(counters, "group_attention.counters", torch.int32)
    n = q.shape[0]
    cells = n * n_heads * max_chunks
    if not group_attention_takes(q, n_heads, n_kv_heads, head_size) or chunk % 16 != 0:
        raise KernelError(f"group_attention does not take head size {head_size} with {n_heads}/{n_kv_heads} heads")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape:
        raise KernelError("group_attention: q / out do not have heads * head_size columns")
    if part_acc.numel() < cells * head_size or part_ml.numel() < cells * 2 or counters.numel() < n * n_heads:
        raise KernelError("group_attention: scratch too small")
    if max_chunks * chunk < page_size * block_table.shape[1]:
        raise KernelError("group_attention: the chunks do not cover the longest block table")
    _group_attention(out.data_ptr(), out.stride(0), q.data_ptr(), q.stride(0), k_pages.data_ptr(), v_pages.data_ptr(),
                     block_table.data_ptr(), block_table.shape[1], positions.data_ptr(), token_item.data_ptr(), n,
                     n_heads, n_kv_heads, head_size, page_size, float(scale), int(window or 0), int(chunk),
                     int(max_chunks), part_acc.data_ptr(), part_ml.data_ptr(), counters.data_ptr(), _stream())
    return out


# ---- tensor-core matrix product (bfloat16) -------------------------------------------------------

_gemm_bf16 = Function("gemm", "mllm_gemm_bf16", [P, P, P, P, I, I, I, L, L, I, I, P, P])


def gemm_takes(a, w) -> bool:
    """Whether the tensor-core kernel takes ``a @ w.T``: bf16, K a multiple of 8, 16-byte
    aligned bases and row strides (what its TMA copies need)."""
    if not isinstance(a, torch.Tensor) or a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    k = a.shape[1]
    return (k % 8 == 0 and a.stride(0) % 8 == 0 and a.stride(1) == 1 and a.data_ptr() % 16 == 0
            and w.is_contiguous() and w.data_ptr() % 16 == 0)


def gemm_bf16(out, a, w, bias, epilogue, status):
    """out = epilogue(a @ w.T + bias) on the tensor cores (tcgen05, TMEM accumulators, TMA).

    a [M, K] and w [N, K] bf16; out bf16, or fp32 for logits and for the residual epilogue
    "add".  ``status``: a zeroed int32 device word the kernel writes a code to if one of its
    bounded waits runs out."""
    _check(a, "gemm.a", torch.bfloat16, 2)
    _check(w, "gemm.w", torch.bfloat16, 2)
    _check(out, "gemm.out", None, 2)
    _check(status, "gemm.status", torch.int32)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n:
        raise KernelError(f"gemm: shapes do not agree: a {tuple(a.shape)}, w {tuple(w.shape)}, out {tuple(out.shape)}")
    if not gemm_takes(a, w):
        raise KernelError("gemm: operands are not laid out for the tensor-core kernel")
    if out.dtype not in (torch.bfloat16, torch.float32) or (epilogue == "add" and out.dtype != torch.float32):
        raise KernelError("gemm: out must be bfloat16, or float32 for logits and the residual sum")
    if out.dtype == torch.float32 and epilogue not in ("add", "store"):
        raise KernelError("gemm: an activation is stored in bfloat16")
    if bias is not None:
        _check(bias, "gemm.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("gemm: bias has another length")
    _gemm_bf16(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), out.stride(0),
               EPILOGUES[epilogue], int(out.dtype == torch.float32), status.data_ptr(), _stream())
    return out


_gemm_bf16_tile = Function("gemm", "mllm_gemm_bf16_tile", [P, P, P, P, I, I, I, L, L, I, I, P, I, P, P])
GEMM_TILE_WIDTHS = (64, 96, 128, 192, 256)        # 1000 + width: tiles of 256 tokens on pairs of CTAs; 2000 + width (to 128): two issuing threads; 7000 / 7100 + CTAs: shared along K


def gemm_bf16_tile(out, a, w, bias, epilogue, status, tile_width, timeline=None):
    """``gemm_bf16`` through the persistent kernel with tiles of 128 x ``tile_width``, whatever
    the number of rows (tests run every width; the engine lets the library choose).  A code
    5000 + t runs the kernel with swapped operands and tiles of t tokens (16 to 256) instead; a
    code 7000 + c (7100 + c) tiles of 256 (128) features shared along K by clusters of c = 2 to 4 CTAs.
    ``timeline``: an int64 device tensor of nine entries that receives time stamps of CTA 0
    (start, set-up done, first operands landed, last product of the first tile issued, first
    accumulator ready, first epilogue done, end), in nanoseconds, then the number of blocks of K
    that CTA's first issuing thread took and how many of them had not arrived at its first look."""
    if timeline is not None:
        _check(timeline, "gemm.timeline", torch.int64, 1)
        if timeline.shape[0] < 9:
            raise KernelError("gemm: the timeline has nine entries")
    _check(a, "gemm.a", torch.bfloat16, 2)
    _check(w, "gemm.w", torch.bfloat16, 2)
    _check(out, "gemm.out", None, 2)
    _check(status, "gemm.status", torch.int32)
    m, k = a.shape
    n = w.shape[0]
    if w.shape[1] != k or out.shape[0] != m or out.shape[1] != n or not gemm_takes(a, w):
        raise KernelError("gemm: operands are not laid out for the tensor-core kernel")
    if out.dtype not in (torch.bfloat16, torch.float32) or (epilogue == "add" and out.dtype != torch.float32):
        raise KernelError("gemm: out must be bfloat16, or float32 for logits and the residual sum")
    if bias is not None:
        _check(bias, "gemm.bias", torch.float32, 1)
    _gemm_bf16_tile(out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), out.stride(0),
                    EPILOGUES[epilogue], int(out.dtype == torch.float32), status.data_ptr(), int(tile_width),
                    _ptr(timeline), _stream())
    return out


_gemm_bf16_qkv = Function("gemm", "mllm_gemm_bf16_qkv", [P, P, P, P, I, I, I, L, L, P, P, P, P, P, P, I, I, I, I, P])


def gemm_qkv_takes(a, w, q_width, kv_width) -> bool:
    """Whether ``gemm_bf16_qkv`` takes the product (what ``gemm_takes`` asks, and query and
    key/value widths that are multiples of 32)."""
    return gemm_takes(a, w) and q_width % 32 == 0 and kv_width % 32 == 0 and w.shape[0] == q_width + 2 * kv_width


def gemm_bf16_qkv(q_out, a, w, bias, status, k_pages, v_pages, positions, token_item, block_table, page_size,
                  q_width, kv_width):
    """The fused query/key/value product on the tensor cores: queries into ``q_out``
    [M, q_width]; keys and values into the cache pages, each token at the slot its position
    and its request's block table row name (the epilogue of ``gemm_bf16`` with a scatter)."""
    _check(a, "gemm_qkv.a", torch.bfloat16, 2)
    _check(w, "gemm_qkv.w", torch.bfloat16, 2)
    _check(q_out, "gemm_qkv.q_out", torch.bfloat16, 2)
    _check(k_pages, "gemm_qkv.k_pages", torch.bfloat16)
    _check(v_pages, "gemm_qkv.v_pages", torch.bfloat16)
    _check(positions, "gemm_qkv.positions", torch.int32, 1)
    _check(token_item, "gemm_qkv.token_item", torch.int32, 1)
    _check(block_table, "gemm_qkv.block_table", torch.int32, 2)
    _check(status, "gemm_qkv.status", torch.int32)
    m, k = a.shape
    n = w.shape[0]
    if not gemm_qkv_takes(a, w, q_width, kv_width) or w.shape[1] != k:
        raise KernelError("gemm_qkv: operands are not laid out for the tensor-core kernel with a scatter")
    if q_out.shape[0] != m or q_out.shape[1] != q_width or q_out.stride(1) != 1:
        raise KernelError("gemm_qkv: q_out must be [M, q_width]")
    if not (k_pages.is_contiguous() and v_pages.is_contiguous() and block_table.is_contiguous()):
        raise KernelError("gemm_qkv: pages and block table must be contiguous")
    if positions.shape[0] < m or token_item.shape[0] < m:
        raise KernelError("gemm_qkv: fewer positions than rows")
    if bias is not None:
        _check(bias, "gemm_qkv.bias", torch.float32, 1)
        if bias.shape[0] != n:
            raise KernelError("gemm_qkv: bias has another length")
    _gemm_bf16_qkv(q_out.data_ptr(), a.data_ptr(), w.data_ptr(), _ptr(bias), m, n, k, a.stride(0), q_out.stride(0),
                   status.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), positions.data_ptr(), token_item.data_ptr(),
                   block_table.data_ptr(), block_table.shape[1], page_size, q_width, kv_width, _stream())
    return q_out


# ---- tensor-core attention for prompt portions (bfloat16) ----------------------------------------

_attention_prefill = Function("attention", "mllm_attention_prefill",
                              [P, L, P, L, L, L, P, P, I, I, P, I, P, I, I, I, I, F, I, P, P, P, I, P, P])

PREFILL_ATTENTION_HEAD_SIZES = (64, 128)
PREFILL_ATTENTION_PAGE_SIZES = (8, 16, 32, 64, 128)
ATTENTION_TILE = 128


def attention_prefill_takes(q, head_size, page_size) -> bool:
    return (q.dtype == torch.bfloat16 and head_size in PREFILL_ATTENTION_HEAD_SIZES
            and page_size in PREFILL_ATTENTION_PAGE_SIZES and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


ATTENTION_TILE_RECORD = 8           # int32 per CTA of attention_prefill
ATTENTION_BLOCKS_PER_PART = 4       # a tile with more key blocks than this is shared among several CTAs
ATTENTION_MAX_PARTS = 8


def attention_tiles(item_offsets, item_counts, item_starts, split=None):
    """The work list of attention_prefill: tiles of up to 128 consecutive tokens of one
    entry, one record per unit of work: (entry, first row, rows, position of the first row,
    part, parts, number of the tile among the split ones, key blocks of the part), sorted by
    falling number of key blocks.  A tile that reaches over more than
    four blocks of 128 keys can be given to several CTAs (parts), so that the longest CTA of a
    step stays short.  That pays only while the step has few tiles (measured: two CTAs on one
    SM run no faster than one after the other), so by default tiles are split when there are
    at most eight of them; ``split=True`` / ``False`` forces it (whole tiles need no scratch).
    Returns (records, number of split tiles, most parts of a tile)."""
    records, n_split, most = [], 0, 1
    if split is None:
        split = sum(-(-count // ATTENTION_TILE) for count in item_counts) <= 8
    for item, (offset, count, start) in enumerate(zip(item_offsets, item_counts, item_starts)):
        for first in range(0, count, ATTENTION_TILE):
            rows = min(ATTENTION_TILE, count - first)
            blocks = (start + first + rows - 1) // ATTENTION_TILE + 1
            parts = min(ATTENTION_MAX_PARTS, -(-blocks // ATTENTION_BLOCKS_PER_PART)) if split else 1
            share = -(-blocks // parts)
            for part in range(parts):
                records.append((item, offset + first, rows, start + first, part, parts, n_split if parts > 1 else 0,
                                min(share, blocks - part * share)))
            if parts > 1:
                n_split += 1
                most = max(most, parts)
    # the kernel's CTAs take records in this order: the longest first
    records.sort(key=lambda record: -record[7])
    return records, n_split, most


def attention_prefill(out, q, k_pages, v_pages, block_table, tiles, n_tiles, n_heads, n_kv_heads, head_size,
                      page_size, scale, window, status, work, scratch=None, n_split=0, max_parts=1):
    """Causal attention over the paged cache on the tensor cores (tcgen05): one CTA per
    (record of the work list, head).  ``tiles``: device int32 [>= n_tiles, 8] from
    ``attention_tiles``.  ``work``: two zeroed int32 (the kernel's work counter; left zero).
    ``scratch``: (fp32 partial states, zeroed int32 counters) when tiles
    come in parts: n_split * heads * max_parts * 128 * (head_size + 4) floats and
    n_split * heads counters."""
    _check(out, "attention_prefill.out", torch.bfloat16, 2)
    _check(q, "attention_prefill.q", torch.bfloat16, 2)
    _check(k_pages, "attention_prefill.k_pages", torch.bfloat16, 4)
    _check(v_pages, "attention_prefill.v_pages", torch.bfloat16, 4)
    _check(block_table, "attention_prefill.block_table", torch.int32, 2)
    _check(tiles, "attention_prefill.tiles", torch.int32)
    _check(status, "attention_prefill.status", torch.int32)
    _check(work, "attention_prefill.work", torch.int32, 1)
    if work.shape[0] < 2:
        raise KernelError("attention_prefill: the work counter has two entries")
    if not attention_prefill_takes(q, head_size, page_size):
        raise KernelError(f"attention_prefill does not take head size {head_size} with pages of {page_size}")
    n_pages = k_pages.shape[0]
    if tuple(k_pages.shape) != (n_pages, page_size, n_kv_heads, head_size) or v_pages.shape != k_pages.shape:
        raise KernelError("attention_prefill: pages must be [n_pages, page_size, kv_heads, head_size]")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("attention_prefill: pages and block table must be contiguous")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape or tiles.numel() < ATTENTION_TILE_RECORD * n_tiles:
        raise KernelError("attention_prefill: q / out / tiles do not fit")
    partial = counters = None
    if max_parts > 1:
        if scratch is None:
            raise KernelError("attention_prefill: tiles in parts need scratch")
        partial, counters = scratch
        _check(partial, "attention_prefill.scratch", torch.float32, 1)
        _check(counters, "attention_prefill.scratch", torch.int32, 1)
        if (partial.shape[0] < n_split * n_heads * max_parts * ATTENTION_TILE * (head_size + 4)
                or counters.shape[0] < n_split * n_heads):
            raise KernelError("attention_prefill: scratch too small")
    _attention_prefill(out.data_ptr(), out.stride(0), q.data_ptr(), q.shape[0], q.shape[1], q.stride(0),
                       k_pages.data_ptr(), v_pages.data_ptr(), n_pages, page_size, block_table.data_ptr(),
                       block_table.shape[1], tiles.data_ptr(), n_tiles, n_heads, n_kv_heads, head_size, float(scale),
                       int(window or 0), status.data_ptr(), _ptr(partial), _ptr(counters), int(max_parts),
                       work.data_ptr(), _stream())
    return out


_attention_prefill_two_tiles = Function("attention", "mllm_attention_prefill_two_tiles",
                                        [P, L, P, L, L, L, P, P, I, I, P, I, P, I, I, I, I, F, I, P, P, P, I, P, P])
ATTENTION_UNIT = 2 * ATTENTION_TILE     # queries per CTA of attention_prefill_two_tiles


def attention_units(item_offsets, item_counts, item_starts, n_heads=1, n_sms=148):
    """The work list of attention_prefill_two_tiles: units of up to 256 consecutive tokens of
    one entry, one record per CTA: (entry, first row, rows, position of the first row, part,
    parts, number of the unit among the split ones, key blocks of the part), sorted by falling
    number of key blocks.  While the step's records times ``n_heads`` leave SMs idle, the unit
    with the most key blocks per part is given one more part (up to eight, and not below two
    blocks a part), so that the step's longest CTA gets shorter.
    Returns (records, number of split units, most parts of a unit)."""
    units = []
    for item, (offset, count, start) in enumerate(zip(item_offsets, item_counts, item_starts)):
        for first in range(0, count, ATTENTION_UNIT):
            rows = min(ATTENTION_UNIT, count - first)
            units.append([item, offset + first, rows, start + first, (start + first + rows - 1) // ATTENTION_TILE + 1, 1])
    n_records = len(units)
    while units and (n_records + 1) * n_heads <= n_sms:
        longest = max(units, key=lambda u: -(-u[4] // u[5]))
        if -(-longest[4] // longest[5]) < 3 or longest[5] >= ATTENTION_MAX_PARTS:
            break
        longest[5] += 1
        n_records += 1
    records, n_split, most = [], 0, 1
    for item, first_row, rows, position, blocks, parts in units:
        share = -(-blocks // parts)
        for part in range(parts):
            records.append((item, first_row, rows, position, part, parts, n_split if parts > 1 else 0,
                            max(0, min(share, blocks - part * share))))
        if parts > 1:
            n_split += 1
            most = max(most, parts)
    records.sort(key=lambda record: -record[7])
    return records, n_split, most


def attention_prefill_two_tiles(out, q, k_pages, v_pages, block_table, units, n_units, n_heads, n_kv_heads, head_size,
                                page_size, scale, window, status, work, scratch=None, n_split=0, max_parts=1):
    """``attention_prefill`` for steps with long portions: one CTA per (record of the work
    list, head), each half of the unit with softmax warps of its own, one thread per query
    row; head size 64.  ``units``: device int32 [>= n_units, 8] from ``attention_units``.
    ``scratch``: (fp32 partial states, zeroed int32 counters) when units come in parts:
    n_split * heads * max_parts * 256 * (head_size + 4) floats and 2 * n_split * heads counters."""
    _check(out, "attention_prefill.out", torch.bfloat16, 2)
    _check(q, "attention_prefill.q", torch.bfloat16, 2)
    _check(k_pages, "attention_prefill.k_pages", torch.bfloat16, 4)
    _check(v_pages, "attention_prefill.v_pages", torch.bfloat16, 4)
    _check(block_table, "attention_prefill.block_table", torch.int32, 2)
    _check(units, "attention_prefill.units", torch.int32)
    _check(status, "attention_prefill.status", torch.int32)
    _check(work, "attention_prefill.work", torch.int32, 1)
    if work.shape[0] < 2:
        raise KernelError("attention_prefill: the work counter has two entries")
    if head_size != 64 or not attention_prefill_takes(q, head_size, page_size):
        raise KernelError(f"attention_prefill_two_tiles does not take head size {head_size} with pages of {page_size}")
    n_pages = k_pages.shape[0]
    if tuple(k_pages.shape) != (n_pages, page_size, n_kv_heads, head_size) or v_pages.shape != k_pages.shape:
        raise KernelError("attention_prefill: pages must be [n_pages, page_size, kv_heads, head_size]")
    if not k_pages.is_contiguous() or not v_pages.is_contiguous() or not block_table.is_contiguous():
        raise KernelError("attention_prefill: pages and block table must be contiguous")
    if q.shape[1] != n_heads * head_size or out.shape != q.shape or units.numel() < ATTENTION_TILE_RECORD * n_units:
        raise KernelError("attention_prefill: q / out / units do not fit")
    partial = counters = None
    if max_parts > 1:
        if scratch is None:
            raise KernelError("attention_prefill: units in parts need scratch")
        partial, counters = scratch
        _check(partial, "attention_prefill.scratch", torch.float32, 1)
        _check(counters, "attention_prefill.scratch", torch.int32, 1)
        if (partial.shape[0] < n_split * n_heads * max_parts * ATTENTION_UNIT * (head_size + 4)
                or counters.shape[0] < 2 * n_split * n_heads):
            raise KernelError("attention_prefill: scratch too small")
    _attention_prefill_two_tiles(out.data_ptr(), out.stride(0), q.data_ptr(), q.shape[0], q.shape[1], q.stride(0),
                                 k_pages.data_ptr(), v_pages.data_ptr(), n_pages, page_size, block_table.data_ptr(),
                                 block_table.shape[1], units.data_ptr(), n_units, n_heads, n_kv_heads, head_size,
                                 float(scale), int(window or 0), status.data_ptr(), _ptr(partial), _ptr(counters),
                                 int(max_parts), work.data_ptr(), _stream())
    return out


_sample_rows_sliced = Function("sampling", "mllm_sampling_sample_rows_sliced",
                               [P, P, L, I, I, P, P, P, P, P, P, P, I, P])
SAMPLE_SLICES = 32


def sample_rows_sliced(out, logits, temperature, top_p, seeds, counters, scratch, any_nucleus):
    """``sample_rows`` spread over 32 blocks per row.  scratch: (fp32 [R*32], int32 [R*32],
    zeroed int32 [R]); any_nucleus: whether some row has temperature > 0 and top_p < 1."""
    _check(out, "sample_rows.out", torch.int32, 1)
    _check(logits, "sample_rows.logits", torch.float32, 2)
    r, vocab = logits.shape
    values, indices, done = scratch
    _check(values, "sample_rows.scratch", torch.float32)
    _check(indices, "sample_rows.scratch", torch.int32)
    _check(done, "sample_rows.scratch", torch.int32)
    if values.numel() < r * SAMPLE_SLICES or indices.numel() < r * SAMPLE_SLICES or done.numel() < r or out.shape[0] < r:
        raise KernelError("sample_rows_sliced: scratch or output too small")
    for name, t, dt in (("temperature", temperature, torch.float32), ("top_p", top_p, torch.float32),
                        ("seeds", seeds, torch.int64), ("counters", counters, torch.int32)):
        if t is not None:
            _check(t, f"sample_rows.{name}", dt, 1)
            if t.shape[0] < r:
                raise KernelError(f"sample_rows: {name} too short")
    _sample_rows_sliced(out.data_ptr(), logits.data_ptr(), logits.stride(0), r, vocab, _ptr(temperature), _ptr(top_p),
                        _ptr(seeds), _ptr(counters), values.data_ptr(), indices.data_ptr(), done.data_ptr(),
                        int(bool(any_nucleus)), _stream())
    return out


_sample_rows_nucleus = Function("sampling", "mllm_sampling_sample_rows_nucleus", [P, P, L, I, I, P, P, P, P, P])


def sample_rows_nucleus(out, logits, temperature, top_p, seeds, counters):
    """Draw only the rows with a nucleus cut (temperature > 0, top_p < 1); the rest of ``out`` stays."""
    _check(out, "sample_rows.out", torch.int32, 1)
    _check(logits, "sample_rows.logits", torch.float32, 2)
    _check(temperature, "sample_rows.temperature", torch.float32, 1)
    _check(top_p, "sample_rows.top_p", torch.float32, 1)
    r, vocab = logits.shape
    _sample_rows_nucleus(out.data_ptr(), logits.data_ptr(), logits.stride(0), r, vocab, temperature.data_ptr(),
                         top_p.data_ptr(), _ptr(seeds), _ptr(counters), _stream())
    return out


_layernorm_warp = Function("decode", "mllm_decode_layernorm", [P, P, P, P, P, I, I, F, P])


def layernorm_warp(out, x, gamma, beta, eps, rows=None):
    """``layernorm`` into bfloat16 with one warp per row, the row read once (width % 4 == 0)."""
    _check(out, "layernorm.out", torch.bfloat16, 2)
    _check(x, "layernorm.x", torch.float32, 2)
    _check(gamma, "layernorm.gamma", torch.float32, 1)
    _check(beta, "layernorm.beta", torch.float32, 1)
    width = x.shape[1]
    if not x.is_contiguous() or not out.is_contiguous() or width % 4 != 0:
        raise KernelError("layernorm_warp: x and out must be contiguous, the width a multiple of 4")
    if out.shape[1] != width or gamma.shape[0] != width or beta.shape[0] != width:
        raise KernelError("layernorm_warp: widths do not agree")
    if rows is not None:
        _check(rows, "layernorm.rows", torch.int32, 1)
        if rows.shape[0] < out.shape[0]:
            raise KernelError("layernorm_warp: fewer row indices than output rows")
    elif x.shape[0] < out.shape[0]:
        raise KernelError("layernorm_warp: fewer input rows than output rows")
    _layernorm_warp(out.data_ptr(), x.data_ptr(), gamma.data_ptr(), beta.data_ptr(), _ptr(rows), out.shape[0], width,
                    float(eps), _stream())
    return out


_keep_tokens = Function("sampling", "mllm_sampling_keep_tokens", [P, P, P, I, I, P])
_resolve_tokens = Function("sampling", "mllm_sampling_resolve_tokens", [P, P, I, I, P])


def keep_tokens(kept, slots, tokens):
    """kept[slots[r]] = tokens[r] for every row r with slots[r] >= 0 (all int32, on the device)."""
    _check(kept, "keep_tokens.kept", torch.int32, 1)
    _check(slots, "keep_tokens.slots", torch.int32, 1)
    _check(tokens, "keep_tokens.tokens", torch.int32, 1)
    n = tokens.shape[0]
    if slots.shape[0] < n:
        raise KernelError("keep_tokens: fewer slots than tokens")
    _keep_tokens(kept.data_ptr(), slots.data_ptr(), tokens.data_ptr(), n, kept.shape[0], _stream())
    return kept


def resolve_tokens(token_ids, kept):
    """token_ids[t] = kept[-1 - token_ids[t]] wherever token_ids[t] < 0 (in place)."""
    _check(token_ids, "resolve_tokens.token_ids", torch.int32, 1)
    _check(kept, "resolve_tokens.kept", torch.int32, 1)
    _resolve_tokens(token_ids.data_ptr(), kept.data_ptr(), token_ids.shape[0], kept.shape[0], _stream())
    return token_ids


_device_info = Function("plain", "mllm_plain_device_info", [ctypes.c_char_p, I, ctypes.POINTER(ctypes.c_int),
                                                            ctypes.POINTER(ctypes.c_long)])


def device_info() -> dict:
    """The current device as the kernel library sees it: name, compute capability, SM count,
    memory, CUDA runtime and driver versions."""
    name = ctypes.create_string_buffer(256)
    values = (ctypes.c_int * 5)()
    memory = ctypes.c_long()
    _device_info(name, 256, values, ctypes.byref(memory))
    return {"name": name.value.decode(), "compute": f"{values[0]}.{values[1]}", "sms": values[2],
            "memory_bytes": memory.value, "runtime": values[3], "driver": values[4]}
