"""Python face of the hand-written CUDA kernels.

Each function checks what the kernel assumes (device, dtype, contiguity, sizes), then
calls the C entry point of the lazily built library on the current CUDA stream.  There
is no other implementation behind these functions: if a library cannot be built or
loaded, or a kernel refuses a size, the call raises.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import load_library

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_REFUSALS = {
    -2: "unsupported dtype",
    -3: "unsupported size",
    -4: "misaligned pointer",
    -5: "scratch capacity exceeded",
}


class KernelError(RuntimeError):
    pass


launch_count = 0     # kernels of this package launched so far (the benchmark reports the difference)


def _check(status: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if status == 0:
        return
    if status < 0:
        raise KernelError(f"{what}: kernel refused the call ({_REFUSALS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


_LIBRARIES = {
    torch.float32: ("elementwise", "norm", "rope_cache", "attention_rows", "gemm_f32", "sampling"),
    torch.bfloat16: ("elementwise", "norm", "rope_cache", "attention_mma", "attention_tcgen05", "decode_linear",
                     "gemm_tcgen05", "skinny_tcgen05", "sampling"),
}


def prepare(dtype: torch.dtype) -> None:
    """Build, side by side, the kernel libraries that a model of this dtype uses (they would otherwise be built
    one after the other, each at its first call)."""
    from .csrc.build import ensure_built

    ensure_built(_LIBRARIES.get(dtype, ()))


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, got {dtype}") from None


def _stream() -> ctypes.c_void_p:
    """The current stream's handle.  (``torch.cuda.current_stream()`` builds a Python stream object through several
    layers on every call: a step launched kernel by kernel spent a seventh of its host time there.)"""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def _cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on a CUDA device")


SS_STRIDE = 16      # rows per tile / per CTA in the small side arrays that one kernel leaves for the next

_i32 = ctypes.c_int
_i64 = ctypes.c_int64
_f32 = ctypes.c_float


def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[t] = table[tokens[t]]``; tokens int32 ``[T]``, table ``[V, H]``, out ``[T, H]``."""
    _cuda(tokens, table, out)
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous(), "tokens must be contiguous int32")
    _need(table.is_contiguous() and out.is_contiguous() and table.dtype == out.dtype, "table/out mismatch")
    rows, hidden = out.shape
    _need(tokens.numel() == rows and table.shape[1] == hidden, "embedding shapes disagree")
    lib = load_library("elementwise")
    _check(lib.tb_embedding(_ptr(tokens), _ptr(table), _ptr(out), _i32(rows), _i32(hidden), _i32(table.shape[0]),
                            _i32(_code(out.dtype)), _stream()), "embedding")
    return out


def select_tokens(tokens: torch.Tensor, feed: torch.Tensor, previous: torch.Tensor, out: torch.Tensor,
                  vocab_size: int) -> torch.Tensor:
    """``out[i] = previous[feed[i]] if feed[i] >= 0 else tokens[i]`` (all int32): token ids that stay on the device
    from one decode step to the next."""
    _cuda(tokens, feed, previous, out)
    n = out.numel()
    _need(all(t.dtype == torch.int32 and t.is_contiguous() for t in (tokens, feed, previous, out)),
          "select_tokens takes contiguous int32 tensors")
    _need(tokens.numel() >= n and feed.numel() >= n, "select_tokens: tokens and feed must cover out")
    lib = load_library("elementwise")
    _check(lib.tb_select_tokens(_ptr(tokens), _ptr(feed), _ptr(previous), _ptr(out), _i32(n), _i32(vocab_size),
                                _stream()), "select_tokens")
    return out


def gather_rows(rows_index: torch.Tensor, src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[s] = src[rows_index[s]]``."""
    _cuda(rows_index, src, out)
    _need(rows_index.dtype == torch.int32 and rows_index.is_contiguous(), "row index must be contiguous int32")
    _need(src.is_contiguous() and out.is_contiguous() and src.dtype == out.dtype, "src/out mismatch")
    rows, width = out.shape
    _need(rows_index.numel() == rows and src.shape[1] == width, "gather shapes disagree")
    lib = load_library("elementwise")
    _check(lib.tb_gather_rows(_ptr(rows_index), _ptr(src), _ptr(out), _i32(rows), _i32(width), _i32(src.shape[0]),
                              _i32(_code(out.dtype)), _stream()), "gather_rows")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """``out = silu(gate) * up`` with ``I = out.shape[1]``; gate and up are the two halves of ``gate_up``'s rows,
    or (``interleaved``) alternate in blocks of eight columns: eight gates, their eight up projections, ..."""
    _cuda(gate_up, out)
    rows, inter = out.shape
    _need(gate_up.shape == (rows, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous(), "silu_mul shapes")
    _need(gate_up.dtype == out.dtype, "silu_mul dtypes")
    lib = load_library("elementwise")
    _check(lib.tb_silu_mul(_ptr(gate_up), _ptr(out), _i32(rows), _i32(inter), _i32(1 if interleaved else 0),
                           _i32(_code(out.dtype)), _stream()), "silu_mul")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    _cuda(x, weight, out)
    rows, width = x.shape
    _need(x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype, "rms_norm x/out")
    _need(weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous(),
          "rms_norm weight must be a contiguous float32 vector of the row width")
    lib = load_library("norm")
    _check(lib.tb_rms_norm(_ptr(x), _ptr(weight), _ptr(out), _i32(rows), _i32(width), _f32(eps),
                           _i32(_code(x.dtype)), _stream()), "rms_norm")
    return out


def add_rms_norm(residual: torch.Tensor, update: torch.Tensor, weight: torch.Tensor, eps: float,
                 out: torch.Tensor, residual_out: torch.Tensor) -> None:
    """``c = residual + update``; ``residual_out = c``; ``out = norm(c) * weight``.  ``residual_out`` may be ``residual``."""
    _cuda(residual, update, weight, out, residual_out)
    rows, width = residual.shape
    for t in (update, out, residual_out):
        _need(t.shape == residual.shape and t.dtype == residual.dtype and t.is_contiguous(), "add_rms_norm operands")
    _need(residual.is_contiguous(), "add_rms_norm residual must be contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous(),
          "add_rms_norm weight must be a contiguous float32 vector of the row width")
    lib = load_library("norm")
    _check(lib.tb_add_rms_norm(_ptr(residual), _ptr(update), _ptr(weight), _ptr(out), _ptr(residual_out), _i32(rows),
                               _i32(width), _f32(eps), _i32(_code(residual.dtype)), _stream()), "add_rms_norm")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_row: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], cache: torch.Tensor, num_heads: int, num_kv_heads: int,
                  head_dim: int, page_size: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k, and store rotated k and v into the cache pages.

    ``qkv``: ``[T, (num_heads + 2*num_kv_heads) * head_dim]`` (last dim contiguous).
    ``cache``: one cache entry ``[pages, 2, num_kv_heads, page_size, head_dim]``.
    ``inv_freq``: float32 ``[head_dim/2]`` or ``None`` for no rotation.
    """
    _cuda(qkv, positions, seq_of_row, block_table, cache)
    rows = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim, "qkv layout")
    _need(positions.dtype == torch.int32 and seq_of_row.dtype == torch.int32 and block_table.dtype == torch.int32,
          "positions, seq_of_row and block_table must be int32")
    _need(positions.numel() >= rows and seq_of_row.numel() >= rows, "row metadata shorter than the batch")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1, "block table must be 2-D, rows contiguous")
    _need(cache.is_contiguous() and cache.dtype == qkv.dtype and
          tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache entry layout")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2 and inv_freq.is_cuda, "inv_freq")
    lib = load_library("rope_cache")
    _check(lib.tb_rope_kv_write(_ptr(qkv), _i64(qkv.stride(0)), _ptr(positions), _ptr(seq_of_row), _ptr(block_table),
                                _i32(block_table.stride(0)), _ptr(inv_freq), _ptr(cache), _i32(rows), _i32(num_heads),
                                _i32(num_kv_heads), _i32(head_dim), _i32(page_size), _i32(1 if write_kv else 0),
                                _i32(_code(qkv.dtype)), _stream()), "rope_kv_write")


def attention_rows(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                   seq_of_row: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int,
                   head_dim: int, page_size: int, window: int, scale: float) -> torch.Tensor:
    """Plain paged attention, one warp per (row, head).  ``q``/``out``: ``[T, num_heads*head_dim]`` views."""
    _cuda(q, out, cache, positions, seq_of_row, block_table)
    rows = q.shape[0]
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim and out.shape == q.shape,
          "q/out layout")
    _need(q.dtype == out.dtype == cache.dtype, "attention dtypes disagree")
    _need(positions.dtype == torch.int32 and seq_of_row.dtype == torch.int32 and block_table.dtype == torch.int32,
          "positions, seq_of_row and block_table must be int32")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1, "block table must be 2-D, rows contiguous")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    lib = load_library("attention_rows")
    _check(lib.tb_attention_rows(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                 _ptr(positions), _ptr(seq_of_row), _ptr(block_table), _i32(block_table.stride(0)),
                                 _i32(rows), _i32(num_heads), _i32(num_kv_heads), _i32(head_dim), _i32(page_size),
                                 _i32(window), _f32(scale), _i32(_code(q.dtype)), _stream()), "attention_rows")
    return out


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ w[N,K]^T`` in true 32-bit arithmetic."""
    _cuda(a, w, out)
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32_nt takes float32")
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and out.shape == (m, n), "gemm shapes disagree")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands need contiguous rows")
    lib = load_library("gemm_f32")
    _check(lib.tb_gemm_f32_nt(_ptr(a), _i64(a.stride(0)), _ptr(w), _i64(w.stride(0)), _ptr(out), _i64(out.stride(0)),
                              _i32(m), _i32(n), _i32(k), _stream()), "gemm_f32_nt")
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Lowest index of each row's maximum; logits float32 ``[S, V]``, out int32 ``[S]``."""
    _cuda(logits, out)
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 with contiguous rows")
    _need(out.dtype == torch.int32 and out.numel() >= logits.shape[0] and out.is_contiguous(), "argmax out")
    lib = load_library("sampling")
    _check(lib.tb_argmax(_ptr(logits), _i64(logits.stride(0)), _ptr(out), _i32(logits.shape[0]),
                         _i32(logits.shape[1]), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor,
           partials: Optional[tuple] = None) -> torch.Tensor:
    """Per row: argmax if ``temperature <= 0`` else inverse-CDF sampling with the given uniform draw.
    ``partials=(values, indices)``: float32 / int32 ``[parts, 16]``, the best value and token of every row that each
    CTA of the product that wrote ``logits`` left (``decode_linear(..., best=...)``): a greedy row is then decided
    from those alone and a sampled row skips the pass over its logits that finds the maximum."""
    _cuda(logits, temperature, uniform, out)
    rows = logits.shape[0]
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 with contiguous rows")
    _need(temperature.dtype == torch.float32 and temperature.numel() >= rows, "temperature must be float32 [S]")
    _need(uniform.dtype == torch.float64 and uniform.numel() >= rows, "uniform must be float64 [S]")
    _need(out.dtype == torch.int32 and out.numel() >= rows and out.is_contiguous(), "sample out")
    values = indices = None
    parts = 0
    if partials is not None:
        values, indices = partials
        _cuda(values, indices)
        _need(values.dtype == torch.float32 and indices.dtype == torch.int32 and values.shape == indices.shape
              and values.dim() == 2 and values.shape[1] == SS_STRIDE and values.is_contiguous()
              and indices.is_contiguous() and rows <= SS_STRIDE, "sample partial results")
        parts = values.shape[0]
    lib = load_library("sampling")
    _check(lib.tb_sample(_ptr(logits), _i64(logits.stride(0)), _ptr(temperature), _ptr(uniform), _ptr(out),
                         _i32(rows), _i32(logits.shape[1]), _ptr(values), _ptr(indices), _i32(parts), _stream()),
           "sample")
    return out


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device, never assumed)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    count = _sm_counts.get(index)
    if count is None:
        count = int(torch.cuda.get_device_properties(index).multi_processor_count)
        _sm_counts[index] = count
    return count


MAX_ATTENTION_SPLITS = 32
_CLUSTER_SPLITS = 8          # up to this many splits merge inside a thread-block cluster and use no scratch


class _AttentionWorkspace:
    """The split decode attention's scratch memory on one device: partial results and arrival counters for more
    than eight splits.  It is allocated once, at the largest size ``plan.attention_splits`` can ask for, and never
    replaced or freed: a captured CUDA graph holds its addresses for as long as the process lives.

    A (split, sequence, kv head) CTA owns sixteen folded rows of ``padded`` floats, and ``plan.attention_splits``
    never chooses more CTAs than are resident at once (two per SM), so ``2 * SMs * 16 * 256`` floats cover every
    choice of it at every head size, whatever the step's row count.  A caller that names its own split count may
    bring more CTAs of narrower heads into the same floats (the narrowest padded head is 32 wide), so the maxima
    and sums are sized for that many."""

    def __init__(self, device):
        ctas = 2 * sm_count(device)
        self.part_o = torch.empty(ctas * 16 * 256, dtype=torch.float32, device=device)
        self.max_ctas = self.part_o.numel() // (16 * 32)
        self.part_ml = torch.empty(self.max_ctas * 16 * 2, dtype=torch.float32, device=device)
        self.counters = torch.zeros(max(4096, self.max_ctas), dtype=torch.int32, device=device)   # left zero by every launch
        # the prompt kernel's key splits (attention_tcgen05): one CTA's 128 rows of up to 128 floats, their maxima
        # and sums, for as many CTAs as are resident at once; a counter per tile
        self.prompt_o = torch.empty(ctas * 128 * 128, dtype=torch.float32, device=device)
        self.prompt_ml = torch.empty(ctas * 128 * 2, dtype=torch.float32, device=device)
        self.prompt_counters = torch.zeros(ctas, dtype=torch.int32, device=device)                # left zero as well


_attention_workspaces = {}


def _split_scratch(device, splits: int, num_seqs: int, num_kv_heads: int, padded: int):
    """``(part_o, part_ml, counters)`` for a launch of more than eight splits.  What fits the device's permanent
    workspace uses it; a larger call (only a caller that names its own split count can make one) gets buffers of
    its own for this launch, which the allocator keeps valid in stream order and, inside a graph capture, for the
    life of the graph."""
    work = _attention_workspaces.get(device)
    if work is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace must exist before a graph is captured "
                              "(call kernels.attention_workspace(device) first)")
        work = _AttentionWorkspace(device)
        _attention_workspaces[device] = work
    ctas = splits * num_seqs * num_kv_heads
    if ctas * 16 * padded <= work.part_o.numel() and ctas <= work.max_ctas:
        return work.part_o, work.part_ml, work.counters
    return (torch.empty(ctas * 16 * padded, dtype=torch.float32, device=device),
            torch.empty(ctas * 16 * 2, dtype=torch.float32, device=device),
            torch.zeros(num_seqs * num_kv_heads, dtype=torch.int32, device=device))


def attention_workspace(device) -> None:
    """Create the device's permanent attention workspace now (before any graph capture)."""
    device = torch.device(device)
    if device not in _attention_workspaces:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace must exist before a graph is captured "
                              "(call kernels.attention_workspace(device) first)")
        _attention_workspaces[device] = _AttentionWorkspace(device)


def attention_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, row_start: torch.Tensor,
                  seq_begin: torch.Tensor, block_table: torch.Tensor, num_seqs: int, max_new: int, num_heads: int,
                  num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, run_tiles: bool,
                  run_decode: bool, splits: int) -> torch.Tensor:
    """Tensor-core paged attention (bfloat16).  Sequences with more than 16 folded rows
    (``new tokens * num_heads / num_kv_heads``) go through the tile kernel, the others through the split kernel."""
    _cuda(q, out, cache, row_start, seq_begin, block_table)
    rows = q.shape[0]
    _need(q.dtype == out.dtype == cache.dtype == torch.bfloat16, "attention_mma takes bfloat16")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim and out.shape == q.shape,
          "q/out layout")
    _need(row_start.dtype == torch.int32 and seq_begin.dtype == torch.int32 and block_table.dtype == torch.int32,
          "row_start, seq_begin and block_table must be int32")
    _need(row_start.numel() >= num_seqs + 1 and seq_begin.numel() >= num_seqs, "sequence metadata too short")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[0] >= num_seqs, "block table")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    lib = load_library("attention_mma")
    padded = lib.tb_attention_mma_padded_dim(_i32(head_dim))
    if padded < 0:
        raise KernelError(f"attention_mma: head_dim {head_dim} is not a multiple of 16 up to 256")
    part_o = part_ml = counters = None
    capacity = 0
    if run_decode and splits > _CLUSTER_SPLITS:
        part_o, part_ml, counters = _split_scratch(q.device, splits, num_seqs, num_kv_heads, padded)
        capacity = part_o.numel()
    _check(lib.tb_attention_mma(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                _ptr(row_start), _ptr(seq_begin), _ptr(block_table), _i32(block_table.stride(0)),
                                _i32(num_seqs), _i32(rows), _i32(max_new), _i32(num_heads), _i32(num_kv_heads),
                                _i32(head_dim), _i32(page_size), _i32(window), _f32(scale),
                                _i32(1 if run_tiles else 0), _i32(1 if run_decode else 0), _i32(splits),
                                _ptr(part_o), _ptr(part_ml), _i64(capacity), _ptr(counters), _stream()),
           "attention_mma")
    return out


def attention_decode_rope(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, row_start: torch.Tensor,
                          seq_begin: torch.Tensor, block_table: torch.Tensor, num_seqs: int, num_heads: int,
                          num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                          inv_freq: Optional[torch.Tensor], write_kv: bool, splits: int) -> torch.Tensor:
    """Decode attention with the rotation and the cache write folded in (bfloat16, one row per sequence).

    ``qkv`` holds the unrotated packed projections ``[q heads | k heads | v heads]`` of the ``num_seqs`` rows.
    Queries and new keys are rotated inside the kernel (``inv_freq`` None: no rotation); with ``write_kv`` the new
    key and value go into the cache page of their position."""
    _cuda(qkv, out, cache, row_start, seq_begin, block_table, inv_freq)
    _need(qkv.dtype == out.dtype == cache.dtype == torch.bfloat16, "attention_decode_rope takes bfloat16")
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[0] == num_seqs
          and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim, "qkv layout")
    _need(out.stride(1) == 1 and tuple(out.shape) == (num_seqs, num_heads * head_dim), "out layout")
    _need(row_start.dtype == torch.int32 and seq_begin.dtype == torch.int32 and block_table.dtype == torch.int32,
          "row_start, seq_begin and block_table must be int32")
    _need(row_start.numel() >= num_seqs + 1 and seq_begin.numel() >= num_seqs, "sequence metadata too short")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[0] >= num_seqs, "block table")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    _need(num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16, "at most 16 query heads per kv head")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous() and inv_freq.numel() == head_dim // 2,
              "inv_freq must be float32 [head_dim / 2]")
    lib = load_library("attention_mma")
    padded = lib.tb_attention_mma_padded_dim(_i32(head_dim))
    if padded < 0:
        raise KernelError(f"attention_decode_rope: head_dim {head_dim} is not a multiple of 16 up to 256")
    part_o = part_ml = counters = None
    capacity = 0
    if splits > _CLUSTER_SPLITS:
        part_o, part_ml, counters = _split_scratch(qkv.device, splits, num_seqs, num_kv_heads, padded)
        capacity = part_o.numel()
    _check(lib.tb_attention_decode_rope(_ptr(qkv), _i64(qkv.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                        _ptr(row_start), _ptr(seq_begin), _ptr(block_table),
                                        _i32(block_table.stride(0)), _i32(num_seqs), _i32(num_heads),
                                        _i32(num_kv_heads), _i32(head_dim), _i32(page_size), _i32(window),
                                        _f32(scale), _ptr(inv_freq), _i32(1 if write_kv else 0), _i32(splits),
                                        _ptr(part_o), _ptr(part_ml), _i64(capacity), _ptr(counters), _stream()),
           "attention_decode_rope")
    return out


PRO_NONE, PRO_NORM, PRO_ADD_NORM = 0, 1, 2
EPI_BF16, EPI_SWIGLU, EPI_F32 = 0, 1, 2

def decode_linear_supported(rows: int, out_features: int, in_features: int, prologue: int = PRO_NONE) -> bool:
    """Whether the skinny decode product takes these sizes (else the caller uses the general path)."""
    return bool(load_library("decode_linear").tb_decode_linear_supported(_i32(rows), _i32(out_features),
                                                                        _i32(in_features), _i32(prologue)))


EPI_ADD_NORM = 3
PRO_SCALED = 3


def decode_linear_tile_features(out_features: int) -> int:
    """Features per tile of the skinny decode product at this output width (16 or 32)."""
    return int(load_library("decode_linear").tb_decode_linear_tile_features(_i32(out_features)))


def decode_linear_ctas(out_features: int) -> int:
    """CTAs that the skinny decode product of this output width is launched with."""
    return int(load_library("decode_linear").tb_decode_linear_ctas(_i32(out_features)))


def decode_linear(weight: torch.Tensor, out: Optional[torch.Tensor], *, x: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None, update: Optional[torch.Tensor] = None,
                  norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                  residual_out: Optional[torch.Tensor] = None, epilogue: int = EPI_BF16,
                  scaled_by: Optional[torch.Tensor] = None, prepare: Optional[tuple] = None,
                  best: Optional[tuple] = None) -> Optional[torch.Tensor]:
    """``out = X @ weight^T`` for at most 16 rows (bfloat16 weights, 32-bit accumulation).

    ``X`` is ``x``, or ``rms_norm(residual)`` (``norm_weight`` given), or ``rms_norm(residual + update)``
    with the rounded sum stored in ``residual_out`` (which must not be ``residual``).  ``epilogue``:
    ``EPI_BF16`` / ``EPI_F32`` store ``[M, N]``; ``EPI_SWIGLU`` treats the weight's rows as blocks of eight gates
    and eight up projections and stores ``silu(gate) * up`` as ``[M, N / 2]``.

    Two forms move the work of the norm that FOLLOWS a product into that product:
    ``prepare=(residual, norm_weight, residual_out, scaled_rows, sums)`` (with ``x``; ``out`` is not written and
    may be None): with ``c = residual + round(x @ weight^T)`` it stores ``residual_out = round(c)``,
    ``scaled_rows = round(c * norm_weight)`` and per tile of output features the rows' sums of ``c^2`` into
    ``sums`` (float32 ``[N / decode_linear_tile_features(N), 16]``).  ``scaled_by=sums`` (with ``x`` = such
    ``scaled_rows`` and ``eps``): ``out = rsqrt(sum(sums) / K + eps) * (x @ weight^T)``, row by row: together the
    norm's scale meets the 32-bit sums of the product behind it.

    ``best=(values, indices)`` (with ``EPI_F32``; float32 / int32 ``[decode_linear_ctas(N), 16]``): every CTA also
    leaves its best output value of each row and that value's lowest column: the first stage of a two-stage argmax.
    """
    _cuda(weight, out, x, residual, update, norm_weight, residual_out, scaled_by)
    n, k = weight.shape
    _need(weight.dtype == torch.bfloat16 and weight.is_contiguous(), "decode_linear weight must be contiguous bfloat16")
    ss_in, ss_tiles = None, 0
    if norm_weight is None:
        prologue, source = PRO_NONE, x
        _need(x is not None and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.shape[1] == k, "decode_linear x")
        if scaled_by is not None:
            prologue = PRO_SCALED
            _need(scaled_by.dtype == torch.float32 and scaled_by.dim() == 2 and scaled_by.shape[1] == SS_STRIDE
                  and scaled_by.is_contiguous() and scaled_by.shape[0] >= 1, "decode_linear sums of squares")
            ss_in, ss_tiles = scaled_by, scaled_by.shape[0]
    else:
        _need(scaled_by is None and prepare is None, "decode_linear: a norm in front excludes scaled_by and prepare")
        prologue, source = (PRO_ADD_NORM if update is not None else PRO_NORM), residual
        _need(residual is not None and residual.dtype == torch.bfloat16 and residual.is_contiguous()
              and residual.shape[1] == k, "decode_linear residual")
        _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == k, "decode_linear norm weight")
        if update is not None:
            _need(update.shape == residual.shape and update.dtype == torch.bfloat16 and update.is_contiguous(),
                  "decode_linear update")
            _need(residual_out is not None and residual_out.shape == residual.shape and residual_out.is_contiguous()
                  and residual_out.dtype == torch.bfloat16 and residual_out.data_ptr() != residual.data_ptr(),
                  "decode_linear residual_out must be a separate bfloat16 buffer")
    m = source.shape[0]
    epi = (None,) * 5
    if prepare is not None:
        _need(prologue == PRO_NONE and epilogue == EPI_BF16, "decode_linear: prepare goes with plain rows and a bfloat16 product")
        epilogue = EPI_ADD_NORM
        p_res, p_norm, p_res_out, p_rows, p_sums = prepare
        _cuda(p_res, p_norm, p_res_out, p_rows, p_sums)
        for t in (p_res, p_res_out, p_rows):
            _need(t.shape == (m, n) and t.dtype == torch.bfloat16 and t.is_contiguous(), "decode_linear prepare rows")
        _need(p_res_out.data_ptr() != p_res.data_ptr(), "decode_linear prepare: the new residual needs a buffer of its own")
        _need(p_norm.dtype == torch.float32 and p_norm.numel() == n and p_norm.is_contiguous(), "decode_linear prepare norm weight")
        tiles = n // decode_linear_tile_features(n)
        _need(p_sums.dtype == torch.float32 and tuple(p_sums.shape) == (tiles, SS_STRIDE) and p_sums.is_contiguous(),
              f"decode_linear prepare sums must be float32 [{tiles}, {SS_STRIDE}]")
        epi = (p_res, p_norm, p_res_out, p_rows, p_sums)
    else:
        width = n // 2 if epilogue == EPI_SWIGLU else n
        _need(out is not None and out.shape == (m, width) and out.stride(1) == 1, "decode_linear out shape")
        _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16), "decode_linear out dtype")
    best_values = best_indices = None
    if best is not None:
        best_values, best_indices = best
        _cuda(best_values, best_indices)
        shape = (decode_linear_ctas(n), SS_STRIDE)
        _need(epilogue == EPI_F32 and best_values.dtype == torch.float32 and best_indices.dtype == torch.int32
              and tuple(best_values.shape) == shape and tuple(best_indices.shape) == shape
              and best_values.is_contiguous() and best_indices.is_contiguous(),
              f"decode_linear best values and indices must be float32 / int32 {list(shape)} (32-bit output only)")
    lib = load_library("decode_linear")
    _check(lib.tb_decode_linear_ex(_ptr(x), _i64(x.stride(0) if x is not None else 0), _ptr(residual), _ptr(update),
                                   _ptr(norm_weight), _f32(eps), _ptr(residual_out), _ptr(weight), _ptr(out),
                                   _i64(out.stride(0) if out is not None else 0), _i32(m), _i32(n), _i32(k),
                                   _i32(prologue), _i32(epilogue), _ptr(ss_in), _i32(ss_tiles), _ptr(epi[0]),
                                   _ptr(epi[1]), _ptr(epi[2]), _ptr(epi[3]), _ptr(epi[4]), _ptr(best_values),
                                   _ptr(best_indices), _stream()), "decode_linear")
    return out


_tcgen05_error = {}


def _error_word(device) -> torch.Tensor:
    word = _tcgen05_error.get(device)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _tcgen05_error[device] = word
    return word


def gemm_tcgen05_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(load_library("gemm_tcgen05").tb_gemm_tcgen05_supported(_i32(rows), _i32(out_features),
                                                                      _i32(in_features), _i32(epilogue)))


GEMM_PAIR_MIN_ROWS = 129       # from here on two CTAs share a 256 x 256 tile (tcgen05.mma.cta_group::2)


def gemm_tcgen05(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_BF16,
                 pair: Optional[bool] = None, tile_width: int = 0) -> torch.Tensor:
    """``out = a @ weight^T`` on the tcgen05 tensor cores (bfloat16 in, 32-bit accumulation).

    ``EPI_BF16`` / ``EPI_F32`` store ``[M, N]``; ``EPI_SWIGLU`` takes a weight whose rows interleave eight gate rows
    and their eight up rows and stores ``silu(gate) * up`` as ``[M, N / 2]``.  ``pair``: CTA pairs on 256 x 256
    tiles instead of single CTAs on 128 x 256 (default: from ``GEMM_PAIR_MIN_ROWS`` rows on); ``tile_width``: the
    width of the pairs' tiles (256 or 448; 0: the one whose tiles fill the pairs in the cheaper rounds).
    """
    _cuda(a, weight, out)
    m, k = a.shape
    n = weight.shape[0]
    _need(a.dtype == weight.dtype == torch.bfloat16, "gemm_tcgen05 takes bfloat16 operands")
    _need(weight.shape[1] == k and a.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1, "gemm layout")
    width = n // 2 if epilogue == EPI_SWIGLU else n
    _need(out.shape == (m, width), "gemm_tcgen05 out shape")
    _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16), "gemm_tcgen05 out dtype")
    lib = load_library("gemm_tcgen05")
    if pair is None:
        pair = m >= GEMM_PAIR_MIN_ROWS
    if pair:
        _check(lib.tb_gemm_pair_tcgen05(_ptr(a), _i64(a.stride(0)), _ptr(weight), _i64(weight.stride(0)), _ptr(out),
                                        _i64(out.stride(0)), _i32(m), _i32(n), _i32(k), _i32(epilogue),
                                        _i32(tile_width), _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05")
        return out
    _check(lib.tb_gemm_tcgen05(_ptr(a), _i64(a.stride(0)), _ptr(weight), _i64(weight.stride(0)), _ptr(out),
                               _i64(out.stride(0)), _i32(m), _i32(n), _i32(k), _i32(epilogue),
                               _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05")
    return out


SKINNY_MAX_ROWS = 128          # rows of the widest product that skinny_tcgen05 takes


def skinny_tcgen05_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(load_library("skinny_tcgen05").tb_skinny_tcgen05_supported(_i32(rows), _i32(out_features),
                                                                          _i32(in_features), _i32(epilogue)))


_skinny_sums_shapes: Dict[int, tuple] = {}


def skinny_tcgen05_sums_shape(out_features: int):
    """Shape of the sums-of-squares array that a product of this width leaves with ``prepare``."""
    shape = _skinny_sums_shapes.get(out_features)
    if shape is None:
        lib = load_library("skinny_tcgen05")
        shape = (int(lib.tb_skinny_tcgen05_sums_tiles(_i32(out_features))), int(lib.tb_skinny_tcgen05_sums_stride()))
        _skinny_sums_shapes[out_features] = shape
    return shape


def skinny_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor], epilogue: int = EPI_BF16,
                   scaled_by: Optional[torch.Tensor] = None, eps: float = 0.0, prepare=None) -> Optional[torch.Tensor]:
    """``out = x @ weight^T`` for 1 to 128 rows on the tcgen05 tensor cores, the weights streamed once.

    ``epilogue`` as for :func:`gemm_tcgen05`.  ``scaled_by``: sums of squares ``[tiles, 128]`` that a product with
    ``prepare`` left; every row of the result is then scaled by ``rsqrt(sum / in_features + eps)`` (the product
    behind a prepared norm).  ``prepare = (residual, norm_weight, new_residual, scaled_rows, sums)``: instead of
    storing ``out`` the product adds its (rounded) result to ``residual`` and leaves the new residual, that sum
    times the following norm's weights, and the rows' sums of squares per tile of 128 features.
    """
    _cuda(x, weight)
    m, k = x.shape
    n = weight.shape[0]
    _need(x.dtype == weight.dtype == torch.bfloat16, "skinny_tcgen05 takes bfloat16 operands")
    _need(weight.shape[1] == k and x.stride(1) == 1 and weight.stride(1) == 1, "skinny_tcgen05 layout")
    null = ctypes.c_void_p(0)
    ss_in, ss_tiles = null, 0
    if scaled_by is not None:
        _need(scaled_by.dtype == torch.float32 and scaled_by.is_contiguous() and scaled_by.dim() == 2
              and scaled_by.shape[1] == 128, "skinny_tcgen05 sums of squares")
        ss_in, ss_tiles = _ptr(scaled_by), scaled_by.shape[0]
    epi = [null] * 5
    out_ptr, out_stride = null, 0
    if prepare is not None:
        residual, norm_weight, new_residual, scaled_rows, sums = prepare
        _cuda(residual, norm_weight, new_residual, scaled_rows, sums)
        _need(scaled_by is None and epilogue == EPI_BF16, "a preparing product is a plain bfloat16 product")
        _need(residual.shape == (m, n) and new_residual.shape == (m, n) and scaled_rows.shape == (m, n)
              and residual.is_contiguous() and new_residual.is_contiguous() and scaled_rows.is_contiguous()
              and residual.dtype == new_residual.dtype == scaled_rows.dtype == torch.bfloat16, "prepare rows")
        _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == n and norm_weight.is_contiguous(),
              "prepare norm weights")
        _need(tuple(sums.shape) == skinny_tcgen05_sums_shape(n) and sums.dtype == torch.float32
              and sums.is_contiguous(), "prepare sums")
        epi = [_ptr(residual), _ptr(norm_weight), _ptr(new_residual), _ptr(scaled_rows), _ptr(sums)]
        epilogue = EPI_ADD_NORM
    else:
        width = n // 2 if epilogue == EPI_SWIGLU else n
        _cuda(out)
        _need(out.shape == (m, width) and out.stride(1) == 1, "skinny_tcgen05 out shape")
        _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16), "skinny_tcgen05 out dtype")
        out_ptr, out_stride = _ptr(out), out.stride(0)
    lib = load_library("skinny_tcgen05")
    _check(lib.tb_skinny_tcgen05(_ptr(x), _i64(x.stride(0)), _ptr(weight), _i64(weight.stride(0)), out_ptr,
                                 _i64(out_stride), _i32(m), _i32(n), _i32(k), _i32(epilogue), ss_in, _i32(ss_tiles),
                                 _f32(eps), *epi, _ptr(_error_word(x.device)), _stream()), "skinny_tcgen05")
    return out


def tcgen05_error(device=None) -> int:
    """Non-zero if a bounded wait inside a tcgen05 kernel ran out since the last call (synchronises)."""
    total = 0
    for dev, word in _tcgen05_error.items():
        if device is None or dev == device:
            total |= int(word.item())
            word.zero_()
    return total


def attention_tcgen05_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return bool(load_library("attention_tcgen05").tb_attention_tcgen05_supported(
        _i32(num_heads), _i32(num_kv_heads), _i32(head_dim), _i32(page_size)))


def attention_tcgen05_tile_ctas(num_seqs: int, max_new: int, num_heads: int, num_kv_heads: int) -> int:
    """CTAs that :func:`attention_tcgen05` launches per key split: tiles of 128 folded rows per kv head and
    sequence (the grid is laid out for the longest sequence)."""
    fold = num_heads // num_kv_heads
    return -(-(max_new * fold) // 128) * num_kv_heads * num_seqs


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, row_start: torch.Tensor,
                      seq_begin: torch.Tensor, block_table: torch.Tensor, num_seqs: int, max_new: int, num_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                      key_splits: int = 1) -> torch.Tensor:
    """Prompt-portion attention on the tcgen05 tensor cores: the sequences of the batch with more than 16 folded
    rows (``new tokens * num_heads / num_kv_heads``); rows of shorter sequences are left untouched.  With
    ``key_splits`` > 1 every tile of 128 folded rows is shared by that many CTAs, each over a contiguous run of the
    tile's keys, and the last to finish adds the runs in order (for steps with too few tiles to fill the GPU); the
    partial rows go through the device's permanent workspace, which holds ``2 * SMs`` CTAs."""
    _cuda(q, out, cache, row_start, seq_begin, block_table)
    _need(q.dtype == out.dtype == cache.dtype == torch.bfloat16, "attention_tcgen05 takes bfloat16")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim and out.shape == q.shape,
          "q/out layout")
    _need(row_start.dtype == torch.int32 and seq_begin.dtype == torch.int32 and block_table.dtype == torch.int32,
          "row_start, seq_begin and block_table must be int32")
    _need(row_start.numel() >= num_seqs + 1 and seq_begin.numel() >= num_seqs, "sequence metadata too short")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[0] >= num_seqs, "block table")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    lib = load_library("attention_tcgen05")
    part_o = part_ml = counters = None
    if key_splits > 1:
        attention_workspace(q.device)
        work = _attention_workspaces[q.device]
        ctas = attention_tcgen05_tile_ctas(num_seqs, max_new, num_heads, num_kv_heads) * key_splits
        _need(1 < key_splits <= 8 and ctas * 128 * head_dim <= work.prompt_o.numel(),
              "attention_tcgen05: more key splits than the workspace holds")
        part_o, part_ml, counters = work.prompt_o, work.prompt_ml, work.prompt_counters
    _check(lib.tb_attention_tcgen05(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                    _ptr(row_start), _ptr(seq_begin), _ptr(block_table), _i32(block_table.stride(0)),
                                    _i32(num_seqs), _i32(max_new), _i32(num_heads), _i32(num_kv_heads),
                                    _i32(head_dim), _i32(page_size), _i32(cache.shape[0]), _i32(window), _f32(scale),
                                    _i32(key_splits), _ptr(part_o), _i64(part_o.numel() if part_o is not None else 0),
                                    _ptr(part_ml), _i64(part_ml.numel() if part_ml is not None else 0),
                                    _ptr(counters), _i64(counters.numel() if counters is not None else 0),
                                    _ptr(_error_word(q.device)), _stream()), "attention_tcgen05")
    return out
