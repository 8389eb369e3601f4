"""Python bindings of the hand-written CUDA kernels.

Every function takes torch tensors that live on a CUDA device, checks dtypes,
shapes and strides on the host, and launches on torch's current stream through
the library's ``extern "C"`` entry points.  There is no CPU fallback: a tensor
on another device, or a missing library, is an error.

Kernels that can meet a bad index (a token id outside the vocabulary, a block
table entry without a page) do not fault: they skip the access and set a device
flag that ``check_device_errors`` reads.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import build as _build

_lib = None
_error_flags = {}

_ERROR_NAMES = {
    1: "a token id is outside the vocabulary",
    2: "a token's position has no page in its request's block table (cache write)",
    3: "a key position has no page in its request's block table (attention read)",
    4: "a bounded wait inside a kernel ran out",
    5: "a row of logits has no maximum (every entry is NaN or -inf); token 0 was written for it",
}

_REFUSALS = {
    -2: "a size is outside what the kernel takes",
    -3: "a pointer or stride is not aligned as the kernel needs",
    -4: "this combination of options is not built",
}


class KernelError(RuntimeError):
    pass


def library() -> ctypes.CDLL:
    """The shared library, built on first use."""
    global _lib
    if _lib is None:
        path = _build.build()
        _lib = ctypes.CDLL(path)
    return _lib


def _check(status: int, name: str) -> None:
    if status == 0:
        return
    if status in _REFUSALS:
        raise KernelError(f"{name}: refused: {_REFUSALS[status]}")
    raise KernelError(f"{name}: CUDA error {status} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_raw_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> ctypes.c_void_p:
    """The current device's current stream.  Asked of the library's C entry points where it has them: the public
    call builds a stream object on the way and took 5 us of the 25 us that a launch cost the host."""
    if _raw_stream is not None and _raw_device is not None:
        return ctypes.c_void_p(_raw_stream(_raw_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(tensor: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("kernels run on CUDA tensors only; there is no CPU path")


def _suffix(dtype: torch.dtype) -> str:
    if dtype == torch.float32:
        return "f32"
    if dtype == torch.bfloat16:
        return "bf16"
    raise KernelError(f"kernels take float32 or bfloat16 activations, got {dtype}")


launch_count = 0  # entry points called so far (each launches one to three kernels); read by measurements
launch_counts: dict = {}  # the same by entry point: which kernels a step used, and how often (Engine.stats reports it)


def _call(name: str, *args, detail: str = "") -> None:
    """Launches one entry point on the current stream.  Products that were held back to be launched together
    (see ``chained_products``) go first: launches keep the order in which they were asked for."""
    if _pending:
        flush_products()
    _launch(name, *args, detail=detail)


def _launch(name: str, *args, detail: str = "") -> None:
    global launch_count
    fn = getattr(library(), name)
    fn.restype = ctypes.c_int
    if _timer is not None:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        _check(fn(*args), name)
        stop.record()
        _timer.records.append((name + detail, start, stop))
    else:
        _check(fn(*args), name)
    launch_count += 1
    launch_counts[name] = launch_counts.get(name, 0) + 1


_timer = None


class launch_timer:
    """``with ops.launch_timer() as timer: ...`` brackets every entry point launched inside with CUDA events on the
    current stream; ``timer.summary()`` (which waits for the device) gives {entry point (products with their sizes):
    (launches, total ms)}.  For measurements only: the events keep a kernel from starting beside the end of the one
    before it, so a step takes longer under the timer than without."""

    def __init__(self):
        self.records = []

    def __enter__(self):
        global _timer
        _timer = self
        return self

    def __exit__(self, kind, value, traceback):
        global _timer
        _timer = None
        return False

    def summary(self) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for name, start, stop in self.records:
            count, total = out.get(name, (0, 0.0))
            out[name] = (count + 1, total + start.elapsed_time(stop))
        return out


_i = ctypes.c_int
_l = ctypes.c_long
_f = ctypes.c_float


def error_flag(device: torch.device) -> torch.Tensor:
    """The int32 device word that kernels set instead of faulting."""
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    if key not in _error_flags:
        _error_flags[key] = torch.zeros(1, dtype=torch.int32, device=key)
    return _error_flags[key]


def check_device_errors(device: torch.device) -> None:
    """Reads the device flag (synchronises) and raises if a kernel set it."""
    flag = error_flag(device)
    value = int(flag.item())
    if value != 0:
        flag.zero_()
        if value == 4:  # a kernel gave up in mid-work: counters that it shares with its next launch start from zero again
            for workspace in _chain_workspaces.values():
                workspace.zero_()
        raise KernelError(f"a kernel reported: {_ERROR_NAMES.get(value, f'error {value}')}")


def wait_selftest(device: torch.device, limit: int = 10_000, arrive: bool = False) -> int:
    """Launches the self-test of the bounded waits: a kernel that waits, at most ``limit`` polls, for a barrier on
    which nothing arrives (or, with ``arrive``, on which another thread does).  A wait that runs out sets the device
    error word, which ``check_device_errors`` turns into a KernelError; the kernel returns either way.  Returns the
    number of polls after which the wait gave up (0 if it was answered)."""
    polls = torch.zeros(1, dtype=torch.int32, device=device)
    _call("kirai_wait_selftest", ctypes.c_uint(limit), _i(1 if arrive else 0), _ptr(error_flag(device)), _ptr(polls), _stream())
    return int(polls.item())


def stream_read(data: torch.Tensor) -> None:
    """Reads ``data`` (a multiple of 16 KB) once, one CTA per SM, with bulk copies into shared memory, and drops it: a
    measurement of what a read-only stream reaches on this device (time it with CUDA events)."""
    _need_cuda(data)
    assert data.is_contiguous() and (data.numel() * data.element_size()) % 16384 == 0
    _call("kirai_stream_read", _ptr(data), _l(data.numel() * data.element_size()), _i(sm_count(data.device)),
          _ptr(error_flag(data.device)), _stream())


# ------------------------------------------------------------------- embedding
def embedding(table, ids: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows ``ids`` of ``table`` [V, H] (a tensor, or a ``TiledWeight`` shared with the output head) widened to
    the 32-bit residual stream [T, H]."""
    assert ids.dtype == torch.int32 and ids.is_contiguous()
    tokens, hidden = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    if isinstance(table, TiledWeight):
        _need_cuda(table.boxes, ids)
        _call("kirai_embedding_tiled_bf16", _ptr(table.boxes), _ptr(ids), _ptr(out), _i(tokens), _i(hidden),
              _i(table.shape[0]), _ptr(error_flag(table.device)), _stream())
        return out
    _need_cuda(table, ids)
    assert table.dim() == 2 and table.is_contiguous()
    _call(f"kirai_embedding_{_suffix(table.dtype)}", _ptr(table), _ptr(ids), _ptr(out), _i(tokens), _i(hidden),
          _i(table.shape[0]), _ptr(error_flag(table.device)), _stream())
    return out


# --------------------------------------------------------------------- RMSNorm
def add_rmsnorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None):
    """``resid += delta`` (32-bit, in place), then RMSNorm of the sum in ``out_dtype``.

    With ``row_index`` only those rows are produced; the residual stream is left as it
    is and the summed rows are returned as the second value.
    """
    _need_cuda(resid, delta, weight, row_index)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == resid.shape[1]
    hidden = resid.shape[1]
    if delta is not None:
        assert delta.shape == resid.shape and delta.dtype == out_dtype and delta.is_contiguous()
    rows = resid.shape[0] if row_index is None else row_index.numel()
    out = torch.empty((rows, hidden), dtype=out_dtype, device=resid.device)
    summed = None
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_contiguous()
        summed = torch.empty((rows, hidden), dtype=torch.float32, device=resid.device)
    _call(f"kirai_add_rmsnorm_{_suffix(out_dtype)}", _ptr(resid), _ptr(delta), _ptr(weight), _ptr(out),
          _ptr(row_index), _ptr(summed), _i(rows), _i(hidden), _f(eps), _stream())
    return (out, summed) if row_index is not None else out


def add_into_residual(resid: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """``resid`` (32-bit) += ``delta``, in place."""
    _need_cuda(resid, delta)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and delta.is_contiguous() and delta.shape == resid.shape
    _call(f"kirai_add_residual_{_suffix(delta.dtype)}", _ptr(resid), _ptr(delta), _l(resid.numel()), _stream())
    return resid


def _head_view(x: torch.Tensor):
    """[rows, heads, width] with a dense (heads, width) part; returns the row stride."""
    assert x.dim() == 3 and x.stride(2) == 1 and x.stride(1) == x.shape[2], "heads must be dense within a row"
    return x.shape[0], x.shape[1], x.shape[2], x.stride(0)


def head_rmsnorm_(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last axis of ``x`` [rows, heads, width], in place, one weight [width] for all heads."""
    _need_cuda(x, weight)
    rows, heads, width, stride = _head_view(x)
    assert weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous()
    _call(f"kirai_head_rmsnorm_{_suffix(x.dtype)}", _ptr(x), _ptr(weight), _i(rows), _i(heads), _i(width), _l(stride),
          _f(eps), _stream())
    return x


# ---------------------------------------------------------------------- rotary
def rope_(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Half-split rotary embedding of ``x`` [rows, heads, width] in place."""
    _need_cuda(x, positions, inv_freq)
    rows, heads, width, stride = _head_view(x)
    assert positions.dtype == torch.int32 and positions.numel() == rows and positions.is_contiguous()
    assert inv_freq.dtype == torch.float32 and inv_freq.numel() == rotary_dim // 2 and inv_freq.is_contiguous()
    _call(f"kirai_rope_{_suffix(x.dtype)}", _ptr(x), _ptr(positions), _ptr(inv_freq), _i(rows), _i(heads), _i(width),
          _i(rotary_dim), _l(stride), _stream())
    return x


# ------------------------------------------------- forms of other layer designs
def embedding_scaled(table: torch.Tensor, ids: torch.Tensor, scale: float, positions: Optional[torch.Tensor] = None,
                     frequencies: Optional[torch.Tensor] = None, copy_dtype: Optional[torch.dtype] = None):
    """Rows ``ids`` of the row-major ``table`` [V, H] times ``scale`` as the 32-bit stream [T, H]; with ``frequencies``
    [ceil(H / 2)] (float32) the sinusoid of each token's position is added: column 2i gets sin(position * f_i), column
    2i + 1 the cosine.  Returns (stream, copy): ``copy`` is the stream rounded to bfloat16 when ``copy_dtype`` asks for
    it, else None."""
    _need_cuda(table, ids, positions, frequencies)
    assert ids.dtype == torch.int32 and ids.is_contiguous() and table.dim() == 2 and table.is_contiguous()
    tokens, hidden = ids.numel(), table.shape[1]
    if frequencies is not None:
        assert positions is not None and positions.dtype == torch.int32 and positions.numel() == tokens and positions.is_contiguous()
        assert frequencies.dtype == torch.float32 and frequencies.numel() == (hidden + 1) // 2 and frequencies.is_contiguous()
    out = torch.empty((tokens, hidden), dtype=torch.float32, device=table.device)
    copy = None
    if copy_dtype == torch.bfloat16:
        copy = torch.empty((tokens, hidden), dtype=torch.bfloat16, device=table.device)
    _call(f"kirai_embedding_sinusoid_{_suffix(table.dtype)}", _ptr(table), _ptr(ids), _ptr(positions), _ptr(frequencies),
          _ptr(out), _ptr(copy), _i(tokens), _i(hidden), _i(table.shape[0]), _f(scale), _ptr(error_flag(table.device)), _stream())
    return out, copy


def norm_add(resid: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, copy_dtype: Optional[torch.dtype] = None):
    """The norm on a sub-layer's output: ``resid`` (32-bit, in place) += RMSNorm(``y``) with ``weight``; ``y`` [T, H] is
    32-bit.  Returns the new stream rounded to bfloat16 when ``copy_dtype`` asks for it (what the next sub-layer
    reads), else None."""
    _need_cuda(resid, y, weight)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    assert y.dtype == torch.float32 and y.shape == resid.shape and y.is_contiguous()
    assert weight.dtype == torch.float32 and weight.numel() == resid.shape[1] and weight.is_contiguous()
    copy = torch.empty(resid.shape, dtype=torch.bfloat16, device=resid.device) if copy_dtype == torch.bfloat16 else None
    _call("kirai_norm_add", _ptr(resid), _ptr(y), _ptr(weight), _ptr(copy), _i(resid.shape[0]), _i(resid.shape[1]), _f(eps), _stream())
    return copy


def norm_add_norm(resid: torch.Tensor, y: torch.Tensor, weight_add: torch.Tensor, eps_add: float, weight_next: torch.Tensor,
                  eps_next: float, out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """The norm on a sub-layer's output and the norm that reads the stream next, in one pass: ``resid`` (32-bit, in
    place) += RMSNorm(``y``) with ``weight_add``; returns RMSNorm(the sum) with ``weight_next`` in ``out_dtype``.  With
    ``row_index`` only those rows are produced and the stream is left as it is."""
    _need_cuda(resid, y, weight_add, weight_next, row_index)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    assert y.dtype == torch.float32 and y.shape == resid.shape and y.is_contiguous()
    hidden = resid.shape[1]
    for weight in (weight_add, weight_next):
        assert weight.dtype == torch.float32 and weight.numel() == hidden and weight.is_contiguous()
    rows = resid.shape[0] if row_index is None else row_index.numel()
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_contiguous()
    out = torch.empty((rows, hidden), dtype=out_dtype, device=resid.device)
    _call(f"kirai_norm_add_norm_{_suffix(out_dtype)}", _ptr(resid), _ptr(y), _ptr(weight_add), _ptr(weight_next), _ptr(out),
          _ptr(row_index), _i(rows), _i(hidden), _f(eps_add), _f(eps_next), _stream())
    return out


def stream_copy(resid: torch.Tensor, out: torch.Tensor, y: Optional[torch.Tensor] = None, weight: Optional[torch.Tensor] = None,
                eps: float = 0.0) -> torch.Tensor:
    """``out`` [T, H] (a run of columns of a wider buffer is allowed) receives the stream ``resid`` [T, H] (32-bit) in
    its own dtype; with ``y`` the stream first takes RMSNorm(``y``) with ``weight`` (in place), as ``norm_add`` does."""
    _need_cuda(resid, out, y, weight)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    assert out.dim() == 2 and out.shape == resid.shape and out.stride(1) == 1
    if y is not None:
        assert y.dtype == torch.float32 and y.shape == resid.shape and y.is_contiguous()
        assert weight is not None and weight.dtype == torch.float32 and weight.numel() == resid.shape[1] and weight.is_contiguous()
    _call(f"kirai_stream_copy_{_suffix(out.dtype)}", _ptr(resid), _ptr(y), _ptr(weight), _ptr(out), _l(out.stride(0)),
          _i(resid.shape[0]), _i(resid.shape[1]), _f(eps), _stream())
    return out


def relu2_(x: torch.Tensor) -> torch.Tensor:
    """``x`` (in place) <- relu(x)^2."""
    _need_cuda(x)
    assert x.is_contiguous()
    _call(f"kirai_relu2_{_suffix(x.dtype)}", _ptr(x), _l(x.numel()), _stream())
    return x


HEAD_GROUPED_MIN_ROWS = 256  # tokens from which the per-head product runs on the tensor cores as a grouped product
_head_tiles: dict = {}


def head_linear_gate(x: torch.Tensor, weight: torch.Tensor, heads: int, used: int, gate: Optional[torch.Tensor] = None,
                     padded_weight: Optional[torch.Tensor] = None) -> torch.Tensor:
    """A product per head: ``x`` [T, heads * pad] (the first ``used`` columns of every head count), ``weight``
    [heads, N, used] in the dtype of ``x``; returns [T, heads * N], row t's head h = weight[h] x[t, h], times
    sigmoid(``gate`` [T, heads * N]) where a gate is given (float32; a run of columns of a wider product is allowed).
    ``padded_weight`` [heads * N, pad] (bfloat16, zero columns beyond ``used``; the columns of ``x`` beyond ``used``
    must then be finite): with it, steps of many tokens run the product on the tensor cores, the heads as the groups of
    a grouped product over rows laid out head by head."""
    _need_cuda(x, weight, gate)
    if (padded_weight is not None and x.dtype == torch.bfloat16 and x.shape[0] >= HEAD_GROUPED_MIN_ROWS and (x.shape[1] // heads) % 8 == 0
            and x.is_contiguous() and x.data_ptr() % 16 == 0):
        return _head_linear_gate_grouped(x, padded_weight, heads, weight.shape[1], gate)
    assert x.dim() == 2 and x.is_contiguous() and x.shape[1] % heads == 0
    pad = x.shape[1] // heads
    assert weight.dim() == 3 and weight.is_contiguous() and weight.dtype == x.dtype and weight.shape[0] == heads and weight.shape[2] == used <= pad
    n = weight.shape[1]
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == (x.shape[0], heads * n)
    out = torch.empty((x.shape[0], heads * n), dtype=x.dtype, device=x.device)
    _call(f"kirai_head_linear_gate_{_suffix(x.dtype)}", _ptr(x), _ptr(weight), _ptr(gate), _l(gate.stride(0) if gate is not None else 0),
          _ptr(out), _i(x.shape[0]), _i(heads), _i(pad), _i(used), _i(n), _stream(),
          detail=f" t={x.shape[0]} heads={heads} k={used} n={n}" if _timer is not None else "")
    return out


def _head_linear_gate_grouped(x: torch.Tensor, padded_weight: torch.Tensor, heads: int, n: int, gate: Optional[torch.Tensor]) -> torch.Tensor:
    tokens, pad = x.shape[0], x.shape[1] // heads
    padded = -(-tokens // 128) * 128
    assert padded_weight.dtype == torch.bfloat16 and padded_weight.shape == (heads * n, pad) and padded_weight.is_contiguous()
    key = (x.device, heads, padded)
    tile_group = _head_tiles.get(key)
    if tile_group is None:  # tile i of the head-major rows belongs to head i // (padded / 128)
        if len(_head_tiles) > 64:
            _head_tiles.clear()
        tile_group = (torch.arange(heads * (padded // 128), dtype=torch.int32) // (padded // 128)).to(torch.int32).to(x.device)
        _head_tiles[key] = tile_group
    rows = torch.empty((heads * padded, pad), dtype=torch.bfloat16, device=x.device)
    _call("kirai_head_major_bf16", _ptr(x), _ptr(rows), _i(tokens), _i(padded), _i(heads), _i(pad), _stream())
    y = linear_grouped(rows, padded_weight, heads, tile_group, out_dtype=torch.float32)
    out = torch.empty((tokens, heads * n), dtype=torch.bfloat16, device=x.device)
    if gate is not None:
        assert gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == (tokens, heads * n)
    _call("kirai_head_gate_rows_bf16", _ptr(y), _ptr(gate), _l(gate.stride(0) if gate is not None else 0), _ptr(out), _i(tokens),
          _i(padded), _i(heads), _i(n), _stream())
    return out


def round_rows(x: torch.Tensor) -> torch.Tensor:
    """The 32-bit rows ``x`` rounded to bfloat16."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    out = torch.empty(x.shape, dtype=torch.bfloat16, device=x.device)
    _call("kirai_round_rows_bf16", _ptr(x), _ptr(out), _l(x.numel()), _stream())
    return out


def qkv_wide_norm_write(qkv: torch.Tensor, q_heads: int, kv_heads: int, key_dim: int, value_dim: int, pad_dim: int,
                        q_bias: Optional[torch.Tensor], k_bias: Optional[torch.Tensor], v_bias: Optional[torch.Tensor],
                        q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                        cache: Optional[torch.Tensor], block_table: torch.Tensor, request_of_token: torch.Tensor,
                        positions: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """Prepares attention whose queries and keys are normed over the whole projection: ``qkv`` [T, nq dk + nkv dk +
    nkv dv] (float32, the stacked product; ``kv_heads`` 0 for a layer that projects queries only) gets its biases, the
    queries and the keys are divided by the root mean square over ALL their columns and multiplied by a weight per
    column, keys and values go to the token's page row in ``cache`` [pages, 2, nkv, page, pad_dim] (first dk and dv
    columns), and the queries come back as [T, nq, pad_dim] in ``out_dtype`` with zero columns beyond dk."""
    _need_cuda(qkv, q_bias, k_bias, v_bias, q_weight, k_weight, cache, block_table, request_of_token, positions)
    assert qkv.dtype == torch.float32 and qkv.dim() == 2 and qkv.stride(1) == 1
    assert qkv.shape[1] == q_heads * key_dim + kv_heads * (key_dim + value_dim)
    for t, n in ((q_bias, q_heads * key_dim), (k_bias, kv_heads * key_dim), (v_bias, kv_heads * value_dim),
                 (q_weight, q_heads * key_dim), (k_weight, kv_heads * key_dim)):
        assert t is None or (t.dtype == torch.float32 and t.numel() == n and t.is_contiguous())
    num_pages, page_size = 0, 1
    if kv_heads:
        num_pages, c_heads, page_size, c_dim = _cache_dims(cache)
        assert (c_heads, c_dim) == (kv_heads, pad_dim) and cache.dtype == out_dtype
    tokens = qkv.shape[0]
    q_out = torch.empty((tokens, q_heads, pad_dim), dtype=out_dtype, device=qkv.device)
    _call(f"kirai_qkv_wide_norm_write_{_suffix(out_dtype)}", _ptr(qkv), _l(qkv.stride(0)), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
          _ptr(q_weight), _ptr(k_weight), _f(eps), _ptr(q_out), _ptr(cache if kv_heads else None), _ptr(block_table),
          _ptr(request_of_token), _ptr(positions), _i(tokens), _i(q_heads), _i(kv_heads), _i(key_dim), _i(value_dim), _i(pad_dim),
          _i(page_size), _i(block_table.shape[1]), _i(num_pages), _ptr(error_flag(qkv.device)), _stream())
    return q_out


# ------------------------------------------------ layer norm, token shift, recurrences
def add_layernorm(resid: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                  out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None, delta_bias: Optional[torch.Tensor] = None,
                  wide: bool = False, shift: Optional[tuple] = None) -> torch.Tensor:
    """``resid += delta + delta_bias`` (32-bit, in place), then the layer norm with a weight and no bias of the sum:
    (x - mean) / sqrt(var + eps) * weight, in ``out_dtype`` (``wide``: in 32-bit whatever the runtime dtype, for a
    step that goes on in 32-bit).  With ``row_index`` only those rows are produced and the stream is left as it is.
    ``shift`` = (mu [H], state [slots, H], slots [rows]), all on the device, for a step in which every request brings
    one token and row r is request r's: the token shift runs in the same kernel (normed row h becomes
    h + (state[slot] - h) * mu, and the slot gets h)."""
    _need_cuda(resid, delta, weight, row_index, delta_bias)
    mu = state = slots = None
    if shift is not None:
        mu, state, slots = shift
        _need_cuda(mu, state, slots)
        assert row_index is None and not wide and slots.dtype == torch.int32 and slots.numel() == resid.shape[0]
        assert mu.dtype == torch.float32 and mu.numel() == resid.shape[1] and mu.is_contiguous()
        assert state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == resid.shape[1] and state.is_contiguous()
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    hidden = resid.shape[1]
    assert weight.dtype == torch.float32 and weight.is_contiguous() and weight.numel() == hidden
    if delta is not None:
        assert delta.shape == resid.shape and delta.dtype == out_dtype and delta.is_contiguous()
    if delta_bias is not None:
        assert delta_bias.dtype == torch.float32 and delta_bias.numel() == hidden and delta_bias.is_contiguous()
    if row_index is not None:
        assert row_index.dtype == torch.int32 and row_index.is_contiguous()
    rows = resid.shape[0] if row_index is None else row_index.numel()
    out = torch.empty((rows, hidden), dtype=torch.float32 if wide else out_dtype, device=resid.device)
    _call(f"kirai_add_layernorm_{_suffix(out_dtype)}", _ptr(resid), _ptr(delta), _ptr(delta_bias), _ptr(weight), _ptr(out),
          _ptr(row_index), _i(rows), _i(hidden), _f(eps), _i(1 if wide else 0), _ptr(mu), _ptr(state), _ptr(slots),
          _i(state.shape[0] if state is not None else 0), _stream())
    return out


def token_shift(h: torch.Tensor, mu: torch.Tensor, state: torch.Tensor, batch, out_dtype: torch.dtype) -> torch.Tensor:
    """Rows ``h`` [T, H] (float32) mixed with the row of the token before: h_t + (h_{t-1} - h_t) * mu.  The row before
    a request's first row of this step is the request's slot of ``state`` [slots, H] (float32), which afterwards holds
    the request's last row of this step."""
    _need_cuda(h, mu, state)
    assert h.dtype == torch.float32 and h.dim() == 2 and h.is_contiguous()
    assert mu.dtype == torch.float32 and mu.numel() == h.shape[1] and mu.is_contiguous()
    assert state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == h.shape[1] and state.is_contiguous()
    out = torch.empty(h.shape, dtype=out_dtype, device=h.device)
    _call(f"kirai_token_shift_{_suffix(out_dtype)}", _ptr(h), _ptr(mu), _ptr(state), _ptr(batch.request_of_token),
          _ptr(batch.query_start), _ptr(batch.slots), _ptr(out), _i(h.shape[0]), _i(h.shape[1]), _i(state.shape[0]), _stream())
    return out


MINGRU_WALK_LIMIT = 16  # steps whose longest run of tokens is at most this walk it; longer runs are scanned in pieces


def mingru(zxg: torch.Tensor, z_bias: Optional[torch.Tensor], x_bias: Optional[torch.Tensor], state: torch.Tensor, batch,
           out_dtype: torch.dtype, walk_limit: Optional[int] = None) -> torch.Tensor:
    """The minGRU recurrence over each request's tokens of this step.  ``zxg`` [T, 3 W] (float32): pre-activations of
    the gate z, the candidate and the output gate.  z = sigmoid(. + z_bias); u = . + x_bias; candidate u + 1/2 where
    u >= 0 and sigmoid(u) below; S <- (1 - z) S + z candidate, from the request's slot of ``state`` [slots, W]
    (float32), which afterwards holds the last S; returns S * silu(g) as [T, W] in ``out_dtype``."""
    _need_cuda(zxg, z_bias, x_bias, state)
    assert zxg.dtype == torch.float32 and zxg.dim() == 2 and zxg.stride(1) == 1 and zxg.shape[1] % 3 == 0
    width = zxg.shape[1] // 3
    assert state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == width and state.is_contiguous()
    for bias in (z_bias, x_bias):
        assert bias is None or (bias.dtype == torch.float32 and bias.numel() == width and bias.is_contiguous())
    walk_limit = MINGRU_WALK_LIMIT if walk_limit is None else walk_limit
    out = torch.empty((zxg.shape[0], width), dtype=out_dtype, device=zxg.device)
    scratch = None
    if batch.max_query_len > walk_limit:
        fn = library().kirai_mingru_piece_tokens
        fn.restype = ctypes.c_int
        pieces = -(-batch.max_query_len // int(fn()))
        scratch = torch.empty((2, batch.num_requests, pieces, width), dtype=torch.float32, device=zxg.device)
    _call(f"kirai_mingru_{_suffix(out_dtype)}", _ptr(zxg), _l(zxg.stride(0)), _ptr(z_bias), _ptr(x_bias), _ptr(state),
          _ptr(batch.query_start), _ptr(batch.slots), _ptr(out), _ptr(scratch), _i(batch.num_requests),
          _i(batch.max_query_len), _i(width), _i(state.shape[0]), _i(walk_limit), _stream())
    return out


def qkv_rope_write(qkv: torch.Tensor, q_heads: int, kv_heads: int, key_dim: int, value_dim: int, pad_dim: int,
                   q_bias: Optional[torch.Tensor], k_bias: Optional[torch.Tensor], v_bias: Optional[torch.Tensor],
                   q_factor: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], rot_offset: int, rot_dims: int,
                   cache: Optional[torch.Tensor], block_table: torch.Tensor, request_of_token: torch.Tensor,
                   positions: torch.Tensor, out_dtype: torch.dtype, rot_amplitude: float = 1.0) -> torch.Tensor:
    """Prepares attention whose projections carry biases and whose heads are rotated in part: ``qkv`` [T, >= nq dk +
    nkv dk + nkv dv] (float32, the stacked product; further columns are left alone; ``kv_heads`` 0 for queries only)
    gets its biases, columns [rot_offset, rot_offset + rot_dims) of every query and key head are rotated (column i of
    the first half with column i + rot_dims / 2, by position * inv_freq[i], cosine and sine times ``rot_amplitude``), query head h is multiplied by
    ``q_factor[h]``, keys and values go to the token's page row in ``cache`` [pages, 2, nkv, page, pad_dim], and the
    queries come back as [T, nq, pad_dim] in ``out_dtype`` with zero columns beyond dk."""
    _need_cuda(qkv, q_bias, k_bias, v_bias, q_factor, inv_freq, cache, block_table, request_of_token, positions)
    assert qkv.dtype == torch.float32 and qkv.dim() == 2 and qkv.stride(1) == 1
    assert qkv.shape[1] >= q_heads * key_dim + kv_heads * (key_dim + value_dim)
    for t, n in ((q_bias, q_heads * key_dim), (k_bias, kv_heads * key_dim), (v_bias, kv_heads * value_dim),
                 (q_factor, q_heads), (inv_freq, rot_dims // 2)):
        assert t is None or (t.dtype == torch.float32 and t.numel() == n and t.is_contiguous())
    num_pages, page_size = 0, 1
    if kv_heads:
        num_pages, c_heads, page_size, c_dim = _cache_dims(cache)
        assert (c_heads, c_dim) == (kv_heads, pad_dim) and cache.dtype == out_dtype
    tokens = qkv.shape[0]
    q_out = torch.empty((tokens, q_heads, pad_dim), dtype=out_dtype, device=qkv.device)
    _call(f"kirai_qkv_rope_write_{_suffix(out_dtype)}", _ptr(qkv), _l(qkv.stride(0)), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
          _ptr(q_factor), _ptr(inv_freq if rot_dims else None), _i(rot_offset), _i(rot_dims), _f(rot_amplitude), _ptr(q_out),
          _ptr(cache if kv_heads else None), _ptr(block_table), _ptr(request_of_token), _ptr(positions), _i(tokens),
          _i(q_heads), _i(kv_heads), _i(key_dim), _i(value_dim), _i(pad_dim), _i(page_size), _i(block_table.shape[1]),
          _i(num_pages), _ptr(error_flag(qkv.device)), _stream())
    return q_out


def latent_prepare(down: torch.Tensor, q_rank: int, kv_rank: int, rot_dims: int, q_weight: Optional[torch.Tensor],
                   kv_weight: torch.Tensor, inv_freq: Optional[torch.Tensor], eps: float, cache: torch.Tensor,
                   block_table: torch.Tensor, request_of_token: torch.Tensor, positions: torch.Tensor,
                   out_dtype: torch.dtype, rot_amplitude: float = 1.0) -> torch.Tensor:
    """Prepares latent attention from ``down`` [T, >= q_rank + kv_rank + rot_dims] (float32, the stacked down
    projections; further columns are left alone): both latents get their RMS norm (a weight per column, ``eps`` inside
    the root), the ``rot_dims`` columns behind them, the key part that all heads share, are rotated whole by position *
    inv_freq (cosine and sine times ``rot_amplitude``), and the token's
    page row in ``cache`` [pages, 2, 1, page, pad] gets [latent, rotated part] as its key row and [latent] as its value
    row.  Returns the normed query latent [T, q_rank] in ``out_dtype``."""
    _need_cuda(down, q_weight, kv_weight, inv_freq, cache, block_table, request_of_token, positions)
    assert down.dtype == torch.float32 and down.dim() == 2 and down.stride(1) == 1 and down.shape[1] >= q_rank + kv_rank + rot_dims
    for t, n in ((q_weight, q_rank), (kv_weight, kv_rank), (inv_freq, rot_dims // 2)):
        assert t is None or (t.dtype == torch.float32 and t.numel() == n and t.is_contiguous())
    num_pages, c_heads, page_size, pad_dim = _cache_dims(cache)
    assert c_heads == 1 and pad_dim >= kv_rank + rot_dims and cache.dtype == out_dtype
    tokens = down.shape[0]
    q_latent = torch.empty((tokens, q_rank), dtype=out_dtype, device=down.device)
    _call(f"kirai_latent_prepare_{_suffix(out_dtype)}", _ptr(down), _l(down.stride(0)), _ptr(q_weight), _ptr(kv_weight),
          _ptr(inv_freq if rot_dims else None), _f(rot_amplitude), _f(eps), _ptr(q_latent), _ptr(cache), _ptr(block_table), _ptr(request_of_token),
          _ptr(positions), _i(tokens), _i(q_rank), _i(kv_rank), _i(rot_dims), _i(pad_dim), _i(page_size),
          _i(block_table.shape[1]), _i(num_pages), _ptr(error_flag(down.device)), _stream())
    return q_latent


def sigmoid_gate_(x: torch.Tensor, gate: torch.Tensor, heads: int, used: int, pad_dim: int) -> torch.Tensor:
    """``x`` [T, heads * pad_dim] (in place): the first ``used`` columns of every head times sigmoid of ``gate``
    [T, heads * used] (float32; a run of columns of a wider product is allowed)."""
    _need_cuda(x, gate)
    assert x.dim() == 2 and x.is_contiguous() and x.shape[1] == heads * pad_dim
    assert gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == (x.shape[0], heads * used)
    _call(f"kirai_sigmoid_gate_{_suffix(x.dtype)}", _ptr(x), _ptr(gate), _l(gate.stride(0)), _i(x.shape[0]), _i(heads),
          _i(used), _i(pad_dim), _stream())
    return x


GATED_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "clamped": 2}


def gated_activation(gate_up: torch.Tensor, activation: str, limit: float = 0.0, slope: float = 1.0) -> torch.Tensor:
    """act(gate) * up for ``gate_up`` [T, 2 I] (gate half first); ``activation`` is ``silu`` or ``gelu_tanh``
    (0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3)))), or ``clamped``: with g = min(gate, limit) and
    u = clamp(up, -limit, limit) the result is g * sigmoid(slope * g) * (u + 1).  Returns [T, I]."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call(f"kirai_gated_activation_{_suffix(gate_up.dtype)}", _ptr(gate_up), _ptr(out), _i(rows), _i(inter),
          _i(GATED_ACTIVATIONS[activation]), _f(limit), _f(slope), _stream())
    return out


def add_bias_(x: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``x`` [T, W] (in place) += ``bias`` [W] (float32)."""
    _need_cuda(x, bias)
    assert x.dim() == 2 and x.is_contiguous() and bias.dtype == torch.float32 and bias.numel() == x.shape[1] and bias.is_contiguous()
    _call(f"kirai_add_bias_{_suffix(x.dtype)}", _ptr(x), _ptr(bias), _i(x.shape[0]), _i(x.shape[1]), _stream())
    return x


# ------------------------------------------------- Dynamic Tanh, matrix states, convolution
def add_dyt(resid: torch.Tensor, deltas, factor: float, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
            out_dtype: torch.dtype, row_index: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``resid`` [T, W] (float32, in place) += factor * sum(deltas) (up to two float32 tensors [T, W], or none), then
    the rows leave as tanh(alpha * x) * weight + bias in ``out_dtype``.  With ``row_index`` (int32 rows) only those rows
    are produced and the stream is left as it is."""
    deltas = [d for d in (deltas or []) if d is not None]
    _need_cuda(resid, alpha, weight, bias, row_index, *deltas)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous() and len(deltas) <= 2
    width = resid.shape[1]
    for d in deltas:
        assert d.dtype == torch.float32 and d.shape == resid.shape and d.is_contiguous()
    for t, n in ((alpha, 1), (weight, width), (bias, width)):
        assert t.dtype == torch.float32 and t.numel() == n and t.is_contiguous()
    rows = resid.shape[0] if row_index is None else row_index.numel()
    out = torch.empty((rows, width), dtype=out_dtype, device=resid.device)
    _call(f"kirai_add_dyt_{_suffix(out_dtype)}", _ptr(resid), _ptr(deltas[0] if deltas else None),
          _ptr(deltas[1] if len(deltas) > 1 else None), _f(factor), _ptr(alpha), _ptr(weight), _ptr(bias), _ptr(out),
          _ptr(row_index), _i(rows), _i(width), _stream())
    return out


def add_scaled_into_residual(resid: torch.Tensor, deltas, factor: float) -> torch.Tensor:
    """``resid`` (float32, in place) += factor * sum(deltas) (one or two float32 tensors of its shape)."""
    deltas = [d for d in deltas if d is not None]
    _need_cuda(resid, *deltas)
    assert resid.dtype == torch.float32 and resid.is_contiguous() and 1 <= len(deltas) <= 2
    for d in deltas:
        assert d.dtype == torch.float32 and d.shape == resid.shape and d.is_contiguous()
    _call("kirai_add_scaled", _ptr(resid), _ptr(deltas[0]), _ptr(deltas[1] if len(deltas) > 1 else None), _f(factor),
          _l(resid.numel()), _stream())
    return resid


def rms_pair_mean(a: torch.Tensor, b: torch.Tensor, weight_a: torch.Tensor, weight_b: torch.Tensor, eps: float) -> torch.Tensor:
    """(a / rms(a) * weight_a + b / rms(b) * weight_b) / 2 row by row, rms with ``eps`` inside the root; all float32."""
    _need_cuda(a, b, weight_a, weight_b)
    assert a.dtype == b.dtype == torch.float32 and a.dim() == 2 and a.shape == b.shape and a.is_contiguous() and b.is_contiguous()
    for w in (weight_a, weight_b):
        assert w.dtype == torch.float32 and w.numel() == a.shape[1] and w.is_contiguous()
    out = torch.empty_like(a)
    _call("kirai_rms_pair_mean", _ptr(a), _ptr(b), _ptr(weight_a), _ptr(weight_b), _f(eps), _ptr(out), _i(a.shape[0]),
          _i(a.shape[1]), _stream())
    return out


def gated_group_norm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, eps: float, groups: int, gate_first: bool,
                     out_dtype: torch.dtype) -> torch.Tensor:
    """``y`` [T, W] (float32; a run of columns of a wider tensor is allowed, as for ``gate``) through a gate and a
    unit-RMS norm over ``groups`` equal parts of a row (``eps`` inside the root), times ``weight`` [W].
    ``gate_first``: (y * silu(gate)) is normed; else y is normed and then multiplied by sigmoid(gate)."""
    _need_cuda(y, gate, weight)
    assert y.dtype == gate.dtype == torch.float32 and y.dim() == 2 and y.shape == gate.shape and y.stride(1) == gate.stride(1) == 1
    width = y.shape[1]
    assert width % groups == 0 and weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous()
    out = torch.empty((y.shape[0], width), dtype=out_dtype, device=y.device)
    _call(f"kirai_gated_group_norm_{_suffix(out_dtype)}", _ptr(y), _l(y.stride(0)), _ptr(gate), _l(gate.stride(0)), _ptr(weight),
          _f(eps), _ptr(out), _i(y.shape[0]), _i(groups), _i(width // groups), _i(0 if gate_first else 1), _stream())
    return out


def conv_silu(x: torch.Tensor, taps: torch.Tensor, bias: Optional[torch.Tensor], state: torch.Tensor, conv_offset: int,
              batch) -> torch.Tensor:
    """Causal convolution per channel with silu over each request's tokens of this step.  ``x`` [T, C] (float32, a
    run of columns of a wider tensor is allowed); ``taps`` [C, K] (float32), whose last column weighs the token
    itself; the K - 1 rows before a request's first row of this step come from its slot of ``state`` [slots, L]
    (float32) at columns [conv_offset, conv_offset + (K - 1) C), which afterwards hold the request's last K - 1 rows."""
    _need_cuda(x, taps, bias, state)
    assert x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
    channels, width = x.shape[1], taps.shape[1]
    assert taps.dtype == torch.float32 and taps.shape == (channels, width) and taps.is_contiguous()
    assert bias is None or (bias.dtype == torch.float32 and bias.numel() == channels and bias.is_contiguous())
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    out = torch.empty((x.shape[0], channels), dtype=torch.float32, device=x.device)
    _call("kirai_conv_silu", _ptr(x), _l(x.stride(0)), _ptr(taps), _ptr(bias), _ptr(state), _l(state.shape[1]), _l(conv_offset),
          _ptr(batch.request_of_token), _ptr(batch.query_start), _ptr(batch.slots), _ptr(out), _i(x.shape[0]),
          _i(batch.num_requests), _i(channels), _i(width), _i(state.shape[0]), _stream())
    return out


STATE_WALK_LIMIT = 8  # steps whose longest run of tokens is at most this walk a matrix state token by token
STATE_CHAIN_LIMIT = 256  # steps with a longer run take their chunks side by side (a carry between them) instead of in a chain
STATE_SIDE_BYTES = 1 << 30  # ... unless the states at the chunks' starts would take more than this


def _state_chunked(batch, state_rows: int, walk_limit: Optional[int]) -> bool:
    """Whether this step's runs go through a matrix state in chunks: some run is longer than the walk's limit, and a
    head of ``state_rows`` rows fits the chunked kernels' shared memory."""
    if batch.max_query_len <= (STATE_WALK_LIMIT if walk_limit is None else walk_limit):
        return False
    fn = library().kirai_state_chunks_fit
    fn.restype = ctypes.c_int
    return bool(fn(ctypes.c_int(state_rows)))


def _state_side(batch, tokens: int, heads: int, rows: int, cols: int, normaliser: bool, device, chain_limit: Optional[int]):
    """(units, state, normaliser, marks): the buffers of a step whose chunks run side by side, or (0, None, None, None)."""
    fn = library().kirai_state_chunk_tokens
    fn.restype = ctypes.c_int
    units = tokens // int(fn()) + batch.num_requests
    limit = STATE_CHAIN_LIMIT if chain_limit is None else chain_limit
    if batch.max_query_len <= limit or units * heads * rows * cols * 4 > STATE_SIDE_BYTES:
        return 0, None, None, None
    state = torch.empty((units, heads, rows, cols), dtype=torch.float32, device=device)
    norm = torch.empty((units, heads, rows), dtype=torch.float32, device=device) if normaliser else None
    marks = torch.empty((units, heads, 3), dtype=torch.float32, device=device)
    return units, state, norm, marks


def ssm_walk(xbc: torch.Tensor, dt: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, skip: torch.Tensor,
             state: torch.Tensor, ssm_offset: int, batch, heads: int, groups: int, state_size: int, head_dim: int,
             walk_limit: Optional[int] = None, chain_limit: Optional[int] = None) -> torch.Tensor:
    """The state-space recurrence over each request's tokens of this step.  ``xbc`` [T, H P + 2 G N] (float32): x, B
    and C; ``dt`` [T, H] (float32, a run of columns of a wider tensor is allowed): step sizes before softplus.  Per
    head h (group h // (H / G)): dt = softplus(dt + dt_bias), S <- exp(-exp(a_log) dt) S + dt B x^T, y = S^T C +
    skip x, S [N, P] in the request's slot of ``state`` [slots, L] from column ``ssm_offset``.  Returns y [T, H P]
    (float32).  A step whose longest run of tokens is above ``walk_limit`` takes the runs a chunk of tokens at a time."""
    _need_cuda(xbc, dt, dt_bias, a_log, skip, state)
    inner = heads * head_dim
    assert xbc.dtype == torch.float32 and xbc.is_contiguous() and xbc.shape[1] == inner + 2 * groups * state_size
    assert dt.dtype == torch.float32 and dt.shape == (xbc.shape[0], heads) and dt.stride(1) == 1
    for t in (dt_bias, a_log, skip):
        assert t.dtype == torch.float32 and t.numel() == heads and t.is_contiguous()
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    y = torch.empty((xbc.shape[0], inner), dtype=torch.float32, device=xbc.device)
    if _state_chunked(batch, state_size, walk_limit):
        units, side, _, marks = _state_side(batch, xbc.shape[0], heads, state_size, head_dim, False, xbc.device, chain_limit)
        _call("kirai_ssm_chunks", _ptr(xbc), _ptr(dt), _l(dt.stride(0)), _ptr(dt_bias), _ptr(a_log), _ptr(skip), _ptr(state),
              _l(state.shape[1]), _l(ssm_offset), _ptr(batch.query_start), _ptr(batch.slots), _ptr(y), _i(batch.num_requests),
              _i(heads), _i(groups), _i(state_size), _i(head_dim), _i(state.shape[0]), _i(units), _ptr(side), _ptr(marks), _stream())
        return y
    _call("kirai_ssm_walk", _ptr(xbc), _ptr(dt), _l(dt.stride(0)), _ptr(dt_bias), _ptr(a_log), _ptr(skip), _ptr(state),
          _l(state.shape[1]), _l(ssm_offset), _ptr(batch.query_start), _ptr(batch.slots), _ptr(y), _i(batch.num_requests),
          _i(heads), _i(groups), _i(state_size), _i(head_dim), _i(state.shape[0]), _stream())
    return y


def matrix_memory_walk(rows: torch.Tensor, in_bias: Optional[torch.Tensor], keep_bias: Optional[torch.Tensor], cap: float,
                       q_scale: float, state: torch.Tensor, batch, heads: int, key_dim: int, value_dim: int,
                       walk_limit: Optional[int] = None, chain_limit: Optional[int] = None) -> torch.Tensor:
    """The matrix memory with exponential gates over each request's tokens of this step.  ``rows`` (float32; further
    columns are left alone): q [H d], k [H d], v [H dv], the input gates' [H] and the forget gates' [H]
    pre-activations.  log_in = cap tanh((. + in_bias) / cap), log_keep = logsigmoid(cap tanh((. + keep_bias) / cap)),
    m' = max(log_keep + m, log_in), S <- exp(log_keep + m - m') S + exp(log_in - m') k v^T, n likewise with k alone,
    o = S^T (q q_scale) / (max(|n . q q_scale|, exp(-m')) + 1e-6).  The request's slot of ``state`` [slots, L] holds
    S [H, d, dv], n [H, d], m [H].  Returns o [T, H dv] (float32).  A step whose longest run of tokens is above
    ``walk_limit`` takes the runs a chunk of tokens at a time."""
    _need_cuda(rows, in_bias, keep_bias, state)
    assert rows.dtype == torch.float32 and rows.dim() == 2 and rows.stride(1) == 1
    assert rows.shape[1] >= heads * (2 * key_dim + value_dim + 2)
    for t in (in_bias, keep_bias):
        assert t is None or (t.dtype == torch.float32 and t.numel() == heads and t.is_contiguous())
    assert state.dtype == torch.float32 and state.dim() == 2 and state.is_contiguous()
    o = torch.empty((rows.shape[0], heads * value_dim), dtype=torch.float32, device=rows.device)
    if _state_chunked(batch, key_dim, walk_limit):
        units, side, norm, marks = _state_side(batch, rows.shape[0], heads, key_dim, value_dim, True, rows.device, chain_limit)
        tail = None if units else torch.empty((batch.num_requests, heads, key_dim + 1), dtype=torch.float32, device=rows.device)
        _call("kirai_matrix_memory_chunks", _ptr(rows), _l(rows.stride(0)), _ptr(in_bias), _ptr(keep_bias), _f(cap), _f(q_scale),
              _ptr(state), _l(state.shape[1]), _ptr(batch.query_start), _ptr(batch.slots), _ptr(o), _ptr(tail),
              _i(batch.num_requests), _i(heads), _i(key_dim), _i(value_dim), _i(state.shape[0]), _i(units), _ptr(side), _ptr(norm),
              _ptr(marks), _stream())
        return o
    _call("kirai_matrix_memory_walk", _ptr(rows), _l(rows.stride(0)), _ptr(in_bias), _ptr(keep_bias), _f(cap), _f(q_scale),
          _ptr(state), _l(state.shape[1]), _ptr(batch.query_start), _ptr(batch.slots), _ptr(o), _i(batch.num_requests), _i(heads),
          _i(key_dim), _i(value_dim), _i(state.shape[0]), _stream())
    return o


def head_gate_(x: torch.Tensor, gate: torch.Tensor, heads: int, used: int, pad_dim: int) -> torch.Tensor:
    """``x`` [T, heads * pad_dim] (in place): the first ``used`` columns of head h times sigmoid(gate[t, h]); ``gate``
    [T, heads] (float32; a run of columns of a wider product is allowed)."""
    _need_cuda(x, gate)
    assert x.dim() == 2 and x.is_contiguous() and x.shape[1] == heads * pad_dim
    assert gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == (x.shape[0], heads)
    _call(f"kirai_head_gate_{_suffix(x.dtype)}", _ptr(x), _ptr(gate), _l(gate.stride(0)), _i(x.shape[0]), _i(heads), _i(used),
          _i(pad_dim), _stream())
    return x


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """``x`` (float32, in place) <- cap * tanh(x / cap)."""
    _need_cuda(x)
    assert x.dtype == torch.float32 and x.is_contiguous()
    _call("kirai_softcap_rows", _ptr(x), _f(cap), _l(x.numel()), _stream())
    return x


def gated_expert_gate(gate_up: torch.Tensor, gates: torch.Tensor, ff: int, activation: str = "silu", limit: float = 0.0,
                      slope: float = 1.0, interleaved: bool = False) -> torch.Tensor:
    """Stacked gated experts: ``gate_up`` [T, experts * 2 ff] (per expert ff gate columns, then ff up columns) becomes
    [T, experts * ff] = act(gate) * up * gates[t, expert] (``gates`` float32 [T, experts], zero where not chosen);
    the activations are those of ``gated_activation``.  ``interleaved``: an expert's columns come as 8 gate columns,
    their 8 up columns, 8 gate columns, ... (see ``interleave_gate_up``)."""
    _need_cuda(gate_up, gates)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gates.dtype == torch.float32 and gates.is_contiguous()
    experts = gates.shape[1]
    assert gate_up.shape == (gates.shape[0], experts * 2 * ff)
    out = torch.empty((gate_up.shape[0], experts * ff), dtype=gate_up.dtype, device=gate_up.device)
    _call(f"kirai_gated_expert_gate_{_suffix(gate_up.dtype)}", _ptr(gate_up), _ptr(gates), _ptr(out), _i(gate_up.shape[0]),
          _i(experts), _i(ff), _i(GATED_ACTIVATIONS[activation]), _f(limit), _f(slope), _i(int(interleaved)), _stream())
    return out


_arrival_counters: dict = {}


def _router_arrivals(device: torch.device, tokens: int) -> torch.Tensor:
    """The router kernel's counters, one per token: zero between launches (the kernel sets them back), one buffer per
    device that grows with the largest step seen.  Launches on one device run one after the other, as a step's do."""
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    counters = _arrival_counters.get(key)
    if counters is None or counters.numel() < tokens:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the router's counters must exist before a stream capture begins: run the step once outside the capture")
        counters = torch.zeros(max(4096, 2 * tokens), dtype=torch.int32, device=key)
        _arrival_counters[key] = counters
    return counters


def _router_rule(over_all: bool, rule: Optional[dict], experts: int, device):
    """The kernels' arguments for how weights come from logits: (mode, correction, groups, keep).  ``rule`` is None
    (softmax over the chosen logits, or over all with ``over_all``) or a dict with ``correction`` (a tensor [experts],
    float32, or None), ``groups`` and ``keep``: sigmoid scores, the choice by score + correction among the ``keep``
    best of ``groups`` equal groups of neighbouring experts (a group's mark is the sum of its two largest choice
    scores), the weights the chosen scores as they are."""
    if rule is None:
        return _i(int(over_all)), _ptr(None), _i(1), _i(1)
    correction = rule.get("correction")
    if correction is not None:
        _need_cuda(correction)
        assert correction.dtype == torch.float32 and correction.numel() == experts and correction.is_contiguous()
    return _i(2), _ptr(correction), _i(int(rule.get("groups", 1))), _i(int(rule.get("keep", 1)))


def router_gates(x: torch.Tensor, router: torch.Tensor, top: int, want_chosen: bool = False, over_all: bool = False,
                 rule: Optional[dict] = None):
    """Routing weights of every token: logits ``router`` [experts, H] (float32) times ``x`` [T, H] in 32-bit, the ``top``
    largest chosen (the lower index on a tie), softmax over the chosen logits alone.  Returns gates [T, experts]
    (float32, zero where not chosen); with ``want_chosen`` also (ids [T, top] int32, weights [T, top] float32) in the
    order of choice.  ``over_all``: the weights are the chosen experts' shares of the softmax over ALL logits instead
    (they then do not sum to one).  ``rule``: sigmoid scores with a correction and groups, see ``_router_rule``."""
    _need_cuda(x, router)
    assert x.dim() == 2 and x.stride(1) == 1 and router.dtype == torch.float32 and router.is_contiguous()
    assert router.shape[1] == x.shape[1] and 0 < top <= router.shape[0]
    tokens, experts = x.shape[0], router.shape[0]
    gates = torch.empty((tokens, experts), dtype=torch.float32, device=x.device)
    ids = torch.empty((tokens, top), dtype=torch.int32, device=x.device) if want_chosen else None
    weights = torch.empty((tokens, top), dtype=torch.float32, device=x.device) if want_chosen else None
    _call(f"kirai_router_gates_{_suffix(x.dtype)}", _ptr(x), _l(x.stride(0)), _ptr(router), _ptr(gates), _ptr(ids), _ptr(weights),
          _ptr(_router_arrivals(x.device, tokens)), _i(tokens), _i(x.shape[1]), _i(experts), _i(top),
          *_router_rule(over_all, rule, experts, x.device), _stream())
    return (gates, ids, weights) if want_chosen else gates


def router_choose_(logits: torch.Tensor, top: int, want_chosen: bool = False, over_all: bool = False, rule: Optional[dict] = None):
    """The choice alone: ``logits`` [T, experts] (float32, as a product left them) become the routing weights in place
    (see ``router_gates``).  Returns what ``router_gates`` returns."""
    _need_cuda(logits)
    assert logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous() and 0 < top <= logits.shape[1]
    tokens, experts = logits.shape
    ids = torch.empty((tokens, top), dtype=torch.int32, device=logits.device) if want_chosen else None
    weights = torch.empty((tokens, top), dtype=torch.float32, device=logits.device) if want_chosen else None
    _call("kirai_router_choose", _ptr(logits), _ptr(ids), _ptr(weights), _i(tokens), _i(experts), _i(top),
          *_router_rule(over_all, rule, experts, logits.device), _stream())
    return (logits, ids, weights) if want_chosen else logits


def relu2_gate_(up: torch.Tensor, gates: torch.Tensor, ff: int) -> torch.Tensor:
    """In place on ``up`` [T, experts * ff]: relu(z)^2 times the token's gate of the column's expert."""
    _need_cuda(up, gates)
    assert up.dim() == 2 and up.is_contiguous() and gates.dtype == torch.float32 and gates.is_contiguous()
    experts = gates.shape[1]
    assert up.shape == (gates.shape[0], experts * ff)
    _call(f"kirai_relu2_gate_{_suffix(up.dtype)}", _ptr(up), _ptr(gates), _i(up.shape[0]), _i(experts), _i(ff), _stream())
    return up


def grouped_rows_capacity(tokens: int, top: int, experts: int) -> int:
    """Tiles of 128 rows that always hold ``tokens * top`` rows sorted by expert, every expert's stretch padded to whole tiles."""
    return (tokens * top + experts * 127 + 127) // 128


def route_plan(chosen_ids: torch.Tensor, experts: int):
    """Lays the (token, chosen expert) pairs of ``chosen_ids`` [T, top] (int32) out as rows sorted by expert, each
    expert's stretch padded to whole tiles of 128 rows.  Returns (tile_group [tiles] = the expert of each tile, slot_of
    [T, top] = the row of each pair, row_of_slot [tiles * 128] = the token of each row, -1 for padding)."""
    _need_cuda(chosen_ids)
    assert chosen_ids.dtype == torch.int32 and chosen_ids.dim() == 2 and chosen_ids.is_contiguous()
    tokens, top = chosen_ids.shape
    tiles = grouped_rows_capacity(tokens, top, experts)
    tile_group = torch.empty(tiles, dtype=torch.int32, device=chosen_ids.device)
    slot_of = torch.empty((tokens, top), dtype=torch.int32, device=chosen_ids.device)
    row_of_slot = torch.empty(tiles * 128, dtype=torch.int32, device=chosen_ids.device)
    _call("kirai_route_plan", _ptr(chosen_ids), _ptr(tile_group), _ptr(slot_of), _ptr(row_of_slot), _i(tokens), _i(top),
          _i(experts), _i(tiles), _stream())
    return tile_group, slot_of, row_of_slot


def route_gather(x: torch.Tensor, row_of_slot: torch.Tensor) -> torch.Tensor:
    """sorted[slot] = x[row_of_slot[slot]] (zeros where the slot is padding); ``x`` [T, H] bfloat16."""
    _need_cuda(x, row_of_slot)
    assert x.dtype == torch.bfloat16 and x.dim() == 2 and x.stride(1) == 1 and row_of_slot.dtype == torch.int32
    out = torch.empty((row_of_slot.numel(), x.shape[1]), dtype=torch.bfloat16, device=x.device)
    _call("kirai_route_gather_bf16", _ptr(x), _l(x.stride(0)), _ptr(row_of_slot), _ptr(out), _i(row_of_slot.numel()),
          _i(x.shape[1]), _stream())
    return out


def route_combine(y: torch.Tensor, slot_of: torch.Tensor, weights: torch.Tensor) -> torch.Tensor:
    """out[t] = sum_j weights[t, j] * y[slot_of[t, j]] in 32-bit; ``y`` [slots, H]."""
    _need_cuda(y, slot_of, weights)
    assert y.dim() == 2 and y.is_contiguous() and slot_of.dtype == torch.int32 and slot_of.is_contiguous()
    assert weights.dtype == torch.float32 and weights.shape == slot_of.shape and weights.is_contiguous()
    tokens, top = slot_of.shape
    out = torch.empty((tokens, y.shape[1]), dtype=torch.float32, device=y.device)
    _call(f"kirai_route_combine_{_suffix(y.dtype)}", _ptr(y), _ptr(slot_of), _ptr(weights), _ptr(out), _i(tokens), _i(y.shape[1]),
          _i(top), _stream())
    return out


def route_combine_norm_add_takes(hidden: int) -> bool:
    """Whether ``route_combine_norm_add`` takes rows of this width (a multiple of 4 up to 8,192)."""
    return hidden % 4 == 0 and 0 < hidden <= 8192


def route_combine_norm_add(resid: torch.Tensor, y: torch.Tensor, slot_of: torch.Tensor, weights: torch.Tensor,
                           norm_weight: torch.Tensor, eps: float, copy_dtype: Optional[torch.dtype] = None):
    """``route_combine`` and ``norm_add`` in one pass: ``resid`` (32-bit, in place) += RMSNorm(sum_j weights[t, j] *
    y[slot_of[t, j]]) with ``norm_weight``; the weighted sum is formed in 32-bit and never written out.  ``y`` [slots, H]
    bfloat16.  Returns the stream's bfloat16 copy when ``copy_dtype`` asks for it."""
    _need_cuda(resid, y, slot_of, weights, norm_weight)
    assert resid.dtype == torch.float32 and resid.dim() == 2 and resid.is_contiguous()
    assert y.dtype == torch.bfloat16 and y.dim() == 2 and y.is_contiguous() and y.shape[1] == resid.shape[1]
    assert slot_of.dtype == torch.int32 and slot_of.is_contiguous() and slot_of.shape[0] == resid.shape[0]
    assert weights.dtype == torch.float32 and weights.shape == slot_of.shape and weights.is_contiguous()
    assert norm_weight.dtype == torch.float32 and norm_weight.numel() == resid.shape[1] and norm_weight.is_contiguous()
    copy = torch.empty(resid.shape, dtype=torch.bfloat16, device=resid.device) if copy_dtype == torch.bfloat16 else None
    _call("kirai_route_combine_norm_add_bf16", _ptr(resid), _ptr(y), _ptr(slot_of), _ptr(weights), _ptr(norm_weight), _ptr(copy),
          _i(resid.shape[0]), _i(resid.shape[1]), _i(slot_of.shape[1]), _f(eps), _stream())
    return copy


def linear_grouped(x: torch.Tensor, weight, groups: int, tile_group: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16,
                   relu2: bool = False, gated: Optional[tuple] = None) -> torch.Tensor:
    """Rows sorted by group times one of ``groups`` stacked matrices each: ``x`` [tiles * 128, K] (bfloat16), ``weight``
    [groups * N, K] (row-major, or a ``TiledWeight`` with N a multiple of 128), ``tile_group`` [tiles] the matrix of each
    128-row tile.  Returns [tiles * 128, N]; with ``relu2`` relu(product)^2 (bfloat16).  ``gated`` = (activation, limit,
    slope): every matrix holds 8 gate rows, their 8 up rows, 8 gate rows, ... and the result is act(gate) * up,
    [tiles * 128, N / 2] (bfloat16), the activations those of ``gated_activation``."""
    m, k, total = _check_product(x, weight)
    _need_cuda(tile_group)
    assert total % groups == 0 and m % 128 == 0 and tile_group.dtype == torch.int32 and tile_group.numel() == m // 128
    n = total // groups
    tiled = isinstance(weight, TiledWeight)
    assert not (relu2 or gated) or out_dtype == torch.bfloat16
    assert not (relu2 and gated) and (gated is None or n % 16 == 0)
    width = n // 2 if gated else n
    out = torch.empty((m, width), dtype=out_dtype, device=x.device)
    form = 6 if gated else (4 if relu2 else (0 if out_dtype == torch.bfloat16 else 1))
    act, limit, slope = (GATED_ACTIVATIONS[gated[0]], float(gated[1]), float(gated[2])) if gated else (0, 0.0, 1.0)
    _call("kirai_gemm_bf16_grouped", _ptr(x), _ptr(weight.boxes if tiled else weight), _i(tiled), _ptr(out), _i(m), _i(n), _i(k),
          _l(x.stride(0)), _l(width), _i(groups), _ptr(tile_group), _i(form), _i(act), _f(limit), _f(slope),
          _ptr(error_flag(x.device)), _stream(),
          detail=f" m={m} n={n} k={k} form={form}" if _timer is not None else "")
    return out


# ------------------------------------------------------------------- cache write
def _cache_dims(cache: torch.Tensor):
    assert cache.dim() == 5 and cache.shape[1] == 2 and cache.is_contiguous(), "cache layer is [pages, 2, kv_heads, page, d]"
    return cache.shape[0], cache.shape[2], cache.shape[3], cache.shape[4]


def kv_write(k: torch.Tensor, v: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
             request_of_token: torch.Tensor, positions: torch.Tensor) -> None:
    """Writes key rows ``k`` and value rows ``v`` [T, kv_heads, d] to their pages."""
    _need_cuda(k, v, cache, block_table, request_of_token, positions)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, kh, kd, k_stride = _head_view(k)
    rows_v, vh, vd, v_stride = _head_view(v)
    assert (rows, kh, kd) == (rows_v, vh, vd) and (kh, kd) == (kv_heads, head_dim)
    assert k.dtype == cache.dtype == v.dtype
    assert block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous()
    _call(f"kirai_kv_write_{_suffix(k.dtype)}", _ptr(k), _ptr(v), _ptr(cache), _ptr(block_table),
          _ptr(request_of_token), _ptr(positions), _i(rows), _i(kv_heads), _i(head_dim), _l(k_stride), _l(v_stride),
          _i(page_size), _i(block_table.shape[1]), _i(num_pages), _ptr(error_flag(k.device)), _stream())


def qk_norm_rope_kv_write_(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
                           q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
                           inv_freq: Optional[torch.Tensor], eps: float, cache: Optional[torch.Tensor],
                           block_table: torch.Tensor, request_of_token: torch.Tensor, positions: torch.Tensor,
                           write_cache: bool = True) -> None:
    """Fused per-head q/k RMSNorm, rotation and paged cache write on ``qkv`` [T, (nq + 2 nkv) d], in place."""
    _need_cuda(qkv, q_weight, k_weight, inv_freq, cache, block_table, request_of_token, positions)
    assert qkv.dim() == 2 and qkv.is_contiguous() and qkv.shape[1] == (q_heads + 2 * kv_heads) * head_dim
    num_pages, page_size = 0, 1
    if kv_heads == 0:
        write_cache = False
    if write_cache:
        num_pages, c_heads, page_size, c_dim = _cache_dims(cache)
        assert (c_heads, c_dim) == (kv_heads, head_dim) and cache.dtype == qkv.dtype
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == head_dim and w.is_contiguous())
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2)
    _call(f"kirai_qk_norm_rope_kv_write_{_suffix(qkv.dtype)}", _ptr(qkv), _ptr(q_weight), _ptr(k_weight),
          _ptr(inv_freq), _ptr(cache if write_cache else None), _ptr(block_table), _ptr(request_of_token),
          _ptr(positions), _i(qkv.shape[0]), _i(q_heads), _i(kv_heads), _i(head_dim), _i(head_dim), _f(eps),
          _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(1 if write_cache else 0),
          _ptr(error_flag(qkv.device)), _stream())


# --------------------------------------------------------------------- attention
MASK_KEEP_SHIFT = 20  # as in common.cuh


def mask_code(window: Optional[int], chunk: Optional[int] = None, keep_first: int = 0) -> int:
    """How the kernels are told which keys a query sees: 0 every key up to its own position, W > 0 the last W of
    them, -C < 0 those of its own chunk of C positions (chunks counted from position 0 of the sequence).  A window
    under which the sequence's first F keys stay visible to every later position is W + (F << 20)."""
    if window and chunk:
        raise KernelError("a layer has a window or a chunked mask, not both")
    if keep_first:
        if not window:
            raise KernelError("kept first keys go with a window")
        if not (0 < window < (1 << MASK_KEEP_SHIFT) and 0 < keep_first < (1 << 11)):
            raise KernelError(f"a window of {window} keys that keeps the first {keep_first} is outside what the kernels take "
                              f"(window below {1 << MASK_KEEP_SHIFT}, kept keys below {1 << 11})")
        return int(window) + (int(keep_first) << MASK_KEEP_SHIFT)
    if window and window >= (1 << MASK_KEEP_SHIFT):
        raise KernelError(f"a window of {window} keys is outside what the kernels take (below {1 << MASK_KEEP_SHIFT})")
    return -int(chunk) if chunk else int(window or 0)


def _attention_detail(q_heads: int, kv_heads: int, head_dim: int, window: Optional[int], chunk: Optional[int], keep_first: int = 0) -> str:
    """What a launch timer's record says of an attention launch beside its entry point (nothing when no timer runs)."""
    if _timer is None:
        return ""
    return f" heads={q_heads} kv={kv_heads} d={head_dim} mask={mask_code(window, chunk, keep_first)}"


def _capped(name: str, softcap: Optional[float]):
    """The entry point ``name`` or its form with a soft cap on the scores, and that form's extra argument."""
    if softcap:
        return name.replace("_bf16", "_softcap_bf16").replace("_f32", "_softcap_f32"), (_f(softcap),)
    return name, ()


def paged_attention_plain(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor,
                          request_of_token: torch.Tensor, positions: torch.Tensor, window: Optional[int],
                          scale: float, chunk: Optional[int] = None, softcap: Optional[float] = None, keep_first: int = 0) -> torch.Tensor:
    """Causal grouped-query attention of ``q`` [T, nq, d] over the paged cache; returns [T, nq * d].  ``chunk``: a
    query sees the keys of its own chunk of that many positions only; ``softcap`` c: scores become c tanh(score / c)."""
    _need_cuda(q, cache, block_table, request_of_token, positions)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == cache.dtype
    out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    name, cap = _capped(f"kirai_paged_attention_plain_{_suffix(q.dtype)}", softcap)
    _call(name, _ptr(q), _ptr(cache), _ptr(out), _ptr(block_table),
          _ptr(request_of_token), _ptr(positions), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(q_stride),
          _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(mask_code(window, chunk, keep_first)), _f(scale), *cap,
          _ptr(error_flag(q.device)), _stream(), detail=_attention_detail(q_heads, kv_heads, head_dim, window, chunk, keep_first))
    return out


def attention_takes_tensor_cores(dtype: torch.dtype, head_dim: int) -> bool:
    """Whether attention over a cache of this dtype and head size runs on the tensor-core kernels (else the
    CUDA-core kernel, which takes any size)."""
    return dtype == torch.bfloat16 and head_dim % 8 == 0 and 0 < head_dim <= 256


def page_size_refusal(dtype: torch.dtype, head_dim: int, page_size: int) -> Optional[str]:
    """Why the attention kernels for this dtype and head size cannot read pages of ``page_size`` tokens, or None.
    The tensor-core kernels fetch keys and values by TMA in boxes of whole page rows that tile their 16- and 64-key
    tiles: a page must be a power of two up to 64 tokens, or a multiple of 64.  The CUDA-core kernel (32-bit, and
    head sizes the others do not take) reads row by row and takes any page size."""
    if page_size < 1:
        return f"a cache page holds at least one token, got {page_size}"
    if not attention_takes_tensor_cores(dtype, head_dim):
        return None
    if page_size <= 64 and page_size & (page_size - 1) == 0:
        return None
    if page_size % 64 == 0:
        return None
    return (f"pages of {page_size} tokens: the bfloat16 attention kernels (head size {head_dim}) take pages of "
            "1, 2, 4, 8, 16, 32 or 64 tokens, or a multiple of 64")


def attention_prefill_takes_tcgen05(q_heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes this shape: head size up to 256 (above 128 a CTA takes a
    whole SM's tensor memory), a group size that divides its 128 query rows, pages of a power-of-two size."""
    group = q_heads // kv_heads
    return head_dim <= 256 and head_dim % 8 == 0 and 128 % group == 0 and page_size & (page_size - 1) == 0


def attention_prefill(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, query_start: torch.Tensor,
                      context_len: torch.Tensor, max_query_len: int, window: Optional[int], scale: float,
                      tcgen05: Optional[bool] = None, out: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                      softcap: Optional[float] = None, keep_first: int = 0) -> torch.Tensor:
    """bf16 tensor-core attention for runs of new tokens (prompt portions, or any mix): q [T, nq, d].
    ``query_start`` holds rows of ``q`` and of the result, so the requests given may be a part of a larger batch
    (``out`` is then the whole batch's result, of which only their rows are written).  ``tcgen05`` picks the kernel (None: the tcgen05 kernel where it takes the shape, else the
    warp-level ``mma.sync`` kernel)."""
    _need_cuda(q, cache, block_table, query_start, context_len)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
    requests = context_len.numel()
    assert query_start.numel() == requests + 1 and query_start.dtype == torch.int32 and context_len.dtype == torch.int32
    if tcgen05 is None:
        tcgen05 = attention_prefill_takes_tcgen05(q_heads, kv_heads, head_dim, page_size)
    if out is None:
        out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    assert out.shape == (rows, q_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous()
    name, cap = _capped("kirai_attention_prefill_tc_bf16" if tcgen05 else "kirai_attention_prefill_bf16", softcap)
    _call(name, _ptr(q), _ptr(cache), _ptr(out),
          _ptr(block_table), _ptr(query_start), _ptr(context_len), _i(requests), _i(max_query_len), _i(q_heads), _i(kv_heads),
          _i(head_dim), _l(q_stride), _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(mask_code(window, chunk, keep_first)), _f(scale),
          *cap, _ptr(error_flag(q.device)), _stream(), detail=_attention_detail(q_heads, kv_heads, head_dim, window, chunk, keep_first))
    return out


DEFAULT_SMS = 148  # for planning on a host without the device (tests); launches ask the device


def decode_splits(requests: int, kv_heads: int, max_context_len: int, tile: int = 16, warps: int = 8,
                  sms: int = DEFAULT_SMS, room=None, head_dim: int = 128, group: int = 4) -> int:
    """How many CTAs share one (request, kv head) in the decode kernel.  A CTA's warps take key tiles in turn, so a
    CTA with n tiles runs ceil(n / warps) rounds plus a fixed cost (set-up, merge); CTAs run in waves of ``sms``; more
    than one range needs the buffer and the second kernel, about three rounds' time (a pair of ranges that merges in
    the kernel, see ``decode_pair_merges``, one round).  A launch that fills all but a
    few SMs pays one round more: the kernel after it finds no SM on which to start early and fetch its weights
    (3.15 against 3.06 ms a step with 144 and with 128 CTAs at two requests of 4,096 tokens, 3.11 against 2.98 at one).
    The split count with the fewest estimated rounds wins."""
    room = room or _default_cluster_room(sms)
    pairs = max(1, requests * kv_heads)
    tiles = max(1, -(-max_context_len // tile))
    best, best_cost = 1, None
    for splits in range(1, min(64, tiles) + 1):
        ctas = pairs * splits
        waves = -(-ctas // sms)
        rounds = -(-(-(-tiles // splits)) // warps) + 3
        merge = 0.0 if splits == 1 else (1.0 if decode_pair_merges(pairs, splits, head_dim, room, group) else 2.75)
        cost = waves * rounds + merge + (1.0 if waves == 1 and ctas > sms - 12 else 0.0)
        if best_cost is None or cost < best_cost:
            best, best_cost = splits, cost
    return best


DECODE_CLUSTER_RANGES = 5  # ranges of a (request, kv head) that may merge inside the decode kernel


def _default_cluster_room(sms: int):
    """Clusters of a size that a device of ``sms`` SMs is taken to hold at once when nobody asked it (planning on a
    host without the device): what one B200 said for clusters of one-per-SM CTAs, scaled."""
    return lambda cluster: {1: sms, 2: sms // 2, 3: (sms * 39) // 148, 4: (sms * 33) // 148, 5: (sms * 26) // 148}.get(cluster, 0)


_cluster_rooms: dict = {}


def decode_cluster_room(device: torch.device, head_dim: int, group: int = 1):
    """cluster size -> how many clusters of the decode kernel ``device`` holds at once (0: it refuses the size).  A CTA
    of that kernel fills an SM and a cluster must lie inside one GPC, so the answer is the device's to give: chips of
    one kind differ in the SMs of their GPCs."""
    key = (torch.device(device), head_dim, group <= 8)
    if key not in _cluster_rooms:
        with torch.cuda.device(key[0]):
            fn = getattr(library(), "kirai_attention_decode_resident_clusters")
            fn.restype = ctypes.c_int
            _cluster_rooms[key] = [0] + [int(fn(_i(head_dim), _i(group), _i(c))) for c in range(1, DECODE_CLUSTER_RANGES + 1)]
    counts = _cluster_rooms[key]
    return lambda cluster: counts[cluster] if 0 < cluster < len(counts) else 0


def decode_pair_merges(pairs: int, splits: int, head_dim: int, room, group: int = 4) -> bool:
    """Whether the ranges of every (request, kv head) merge inside the decode kernel, as a cluster of CTAs that write
    their rows into slots in the first one's shared memory: two to five ranges, all clusters running at once (``room``:
    cluster size -> how many the device holds; in a launch of several waves the CTAs that a cluster must place
    together left SMs idle: 6 requests as 48 clusters of 3, of which 39 to 45 fit, 3.92 against 3.44 ms a step), heads
    of up to 128, and the other CTAs' rows (``group`` each) fitting the slots' 16 rows."""
    return (2 <= splits <= DECODE_CLUSTER_RANGES and pairs <= room(splits) and head_dim <= 128
            and (splits - 1) * group <= 16)


def decode_plan(context_lens, kv_heads: int, window: Optional[int] = None, tile: int = 16, warps: int = 8,
                sms: int = DEFAULT_SMS, room=None, head_dim: int = 128, group: int = 4) -> tuple:
    """Which decode attention kernel a batch should take: (balanced, splits).

    The split kernel gives every request the same number of CTAs, so its time is that of the longest request and
    comes in waves of ``sms`` CTAs; the balanced kernel cuts all key tiles into ``sms`` equal ranges, which costs
    it a second start inside most CTAs and a longer merge.  Costs are in rounds of one key tile per warp (about
    1.35 us on the 8B layer sizes); the fixed parts were fitted to measurements of both kernels at batches of 1 to
    64.  Balanced is chosen only when it is expected to be clearly faster: contexts of unequal length, or a batch
    whose CTAs fill the last wave badly."""
    lens = [min(int(n), window) if window else int(n) for n in context_lens]
    if not lens:
        return False, 1
    longest = max(1, max(lens))
    room = room or _default_cluster_room(sms)
    splits = decode_splits(len(lens), kv_heads, longest, tile, warps, sms, room, head_dim, group)
    tiles = [max(1, -(-n // tile)) for n in lens]
    waves = -(-len(lens) * kv_heads * splits // sms)
    rounds_split = -(-(-(-max(tiles) // splits)) // warps)
    cost_split = waves * (rounds_split + 2.5) + (0.0 if splits == 1 else (1.0 if decode_pair_merges(len(lens) * kv_heads, splits, head_dim, room, group) else 2.5))
    rounds_balanced = -(-(-(-kv_heads * sum(tiles) // sms)) // warps)
    cost_balanced = rounds_balanced + 9.5
    return cost_balanced < 0.92 * cost_split, splits


def attention_decode(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, context_len: torch.Tensor,
                     window: Optional[int], scale: float, num_splits: int = 1, out: Optional[torch.Tensor] = None,
                     chunk: Optional[int] = None, softcap: Optional[float] = None, keep_first: int = 0) -> torch.Tensor:
    """bf16 tensor-core attention for a batch in which every request brings one token: q [R, nq, d] (row r of ``q``,
    of the tables and of the result belongs to request r; ``out`` may be the head of a larger result)."""
    _need_cuda(q, cache, block_table, context_len)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
    assert context_len.numel() == rows and context_len.dtype == torch.int32
    if out is None:
        out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    assert out.shape == (rows, q_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous()
    partial = None
    if num_splits > 1 and not decode_pair_merges(rows * kv_heads, num_splits, head_dim, decode_cluster_room(q.device, head_dim, q_heads // kv_heads), q_heads // kv_heads):
        # the ranges' results go through a buffer and a second kernel
        partial = torch.empty((rows, q_heads, num_splits, head_dim + 2), dtype=torch.float32, device=q.device)
    name, cap = _capped("kirai_attention_decode_bf16", softcap)
    _call(name, _ptr(q), _ptr(cache), _ptr(out), _ptr(partial), _ptr(block_table),
          _ptr(context_len), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(q_stride), _i(page_size),
          _i(block_table.shape[1]), _i(num_pages), _i(mask_code(window, chunk, keep_first)), _f(scale), *cap, _i(num_splits),
          _ptr(error_flag(q.device)), _stream(), detail=_attention_detail(q_heads, kv_heads, head_dim, window, chunk, keep_first))
    return out


_sm_counts = {}


def sm_count(device: torch.device) -> int:
    key = torch.device(device)
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(key).multi_processor_count
    return _sm_counts[key]


def attention_decode_balanced(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, context_len: torch.Tensor,
                              window: Optional[int], scale: float, ctas: Optional[int] = None,
                              out: Optional[torch.Tensor] = None, chunk: Optional[int] = None,
                              softcap: Optional[float] = None, keep_first: int = 0) -> torch.Tensor:
    """The decode attention with the key tiles of all (request, kv head) pairs cut into ``ctas`` equal ranges
    (default: one per SM), so that every CTA reads the same number of keys whatever the batch looks like."""
    _need_cuda(q, cache, block_table, context_len)
    num_pages, kv_heads, page_size, head_dim = _cache_dims(cache)
    rows, q_heads, qd, q_stride = _head_view(q)
    assert qd == head_dim and q.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16
    assert context_len.numel() == rows and context_len.dtype == torch.int32
    ctas = ctas or sm_count(q.device)
    if out is None:
        out = torch.empty((rows, q_heads * head_dim), dtype=q.dtype, device=q.device)
    assert out.shape == (rows, q_heads * head_dim) and out.dtype == q.dtype and out.is_contiguous()
    partial = torch.empty((ctas, 2, 16, head_dim + 2), dtype=torch.float32, device=q.device)
    name, cap = _capped("kirai_attention_decode_balanced_bf16", softcap)
    _call(name, _ptr(q), _ptr(cache), _ptr(out), _ptr(partial), _ptr(block_table),
          _ptr(context_len), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(q_stride), _i(page_size),
          _i(block_table.shape[1]), _i(num_pages), _i(mask_code(window, chunk, keep_first)), _f(scale), *cap, _i(ctas),
          _ptr(error_flag(q.device)), _stream(), detail=_attention_detail(q_heads, kv_heads, head_dim, window, chunk, keep_first))
    return out


def paged_attention(q: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, batch, window: Optional[int],
                    scale: float, chunk: Optional[int] = None, softcap: Optional[float] = None, keep_first: int = 0) -> torch.Tensor:
    """Attention of the product path over the paged cache for the tokens of ``batch``
    (a kirai_b200.engine.batch.StepBatch).  float32 takes the plain kernel; bfloat16 takes the
    tensor-core kernels (the decode kernel when every request brings one token), or the plain
    kernel for head sizes they do not take (not a multiple of 8, or above 256)."""
    head_dim, q_heads, kv_heads = q.shape[2], q.shape[1], cache.shape[2]
    fast = attention_takes_tensor_cores(q.dtype, head_dim) and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
    if not fast:
        return paged_attention_plain(q, cache, block_table, batch.request_of_token, batch.positions, window, scale,
                                     chunk, softcap, keep_first)
    decode_rows = batch.num_requests if batch.decode_only else getattr(batch, "num_decode", 0)
    if decode_rows and q_heads // kv_heads <= 16:
        # The requests that bring one token stand first in the batch (the batch builder puts them there) and take the
        # decode kernels, which split a long context over many CTAs; prompt portions take the prompt kernel, and both
        # write their rows of one result.  A prompt kernel alone would give a decoding request one CTA per kv head.
        out = torch.empty((q.shape[0], q_heads * head_dim), dtype=q.dtype, device=q.device)
        _decode_rows(q[:decode_rows], cache, block_table[:decode_rows], batch, decode_rows, window, scale, out[:decode_rows],
                     chunk, softcap, keep_first)
        if decode_rows < batch.num_requests:
            attention_prefill(q, cache, block_table[decode_rows:], batch.query_start[decode_rows:], batch.context_len[decode_rows:],
                              batch.max_query_len, window, scale, out=out, chunk=chunk, softcap=softcap, keep_first=keep_first)
        return out
    return attention_prefill(q, cache, block_table, batch.query_start, batch.context_len, batch.max_query_len, window, scale,
                             chunk=chunk, softcap=softcap, keep_first=keep_first)


def _decode_rows(q, cache, block_table, batch, rows: int, window: Optional[int], scale: float, out: torch.Tensor,
                 chunk: Optional[int] = None, softcap: Optional[float] = None, keep_first: int = 0) -> None:
    """The decode attention of the first ``rows`` requests of ``batch`` (one token each)."""
    kv_heads = cache.shape[2]
    mask = dict(chunk=chunk, softcap=softcap, keep_first=keep_first)
    if chunk:
        window = None
    reach = (window + keep_first if window else None) or chunk  # the most keys a token sees: what the launch is planned for
    room = decode_cluster_room(q.device, q.shape[2], q.shape[1] // kv_heads)
    context_len = batch.context_len[:rows]
    # the batch may say which kernel (a captured step does: its lengths change between replays); otherwise
    # the host's copy of the lengths decides; KIRAI_DECODE_BALANCED=0 or 1 overrides both
    balanced = getattr(batch, "decode_balanced", None)
    longest = batch.max_context_len
    if balanced is None:
        lens = [start + count for start, count in zip(batch.start_positions[:rows], batch.query_lens[:rows])]
        balanced, _ = decode_plan(lens, kv_heads, reach, sms=sm_count(q.device), room=room, head_dim=q.shape[2],
                                  group=q.shape[1] // kv_heads)
        longest = max(lens)
    forced = os.environ.get("KIRAI_DECODE_BALANCED")
    if forced in ("0", "1"):
        balanced = forced == "1"
    if balanced and rows <= 1024:
        attention_decode_balanced(q, cache, block_table, context_len, window, scale, out=out, **mask)
        return
    # (a captured step says how many ranges, planned for its requests' lengths; else the longest context decides)
    splits = getattr(batch, "decode_splits", None) or decode_splits(rows, kv_heads, min(longest, reach or longest), sms=sm_count(q.device),
                                                                    room=room, head_dim=q.shape[2], group=q.shape[1] // kv_heads)
    attention_decode(q, cache, block_table, context_len, window, scale, splits, out=out, **mask)


def decode_prepares_qk(qkv: torch.Tensor, cache: Optional[torch.Tensor], batch, q_heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether ``attention_decode_qk`` takes this step: every request brings one token, bfloat16, heads of 64, 128 or
    256 in groups of at most 16, rows on 16-byte boundaries, and no more (request, kv head) pairs than SMs: with more,
    every one of the many CTAs repeats the preparation, and the separate kernel, which runs beside the end of the
    product before it, is faster (10.37 against 10.13 ms a step at 64 requests of the 8B shape; 3.29 against 3.31 ms
    at one request)."""
    return (cache is not None and batch.num_requests * kv_heads <= sm_count(qkv.device) and qkv.dtype == torch.bfloat16 and cache.dtype == torch.bfloat16 and batch.decode_only
            and head_dim in (64, 128, 256) and kv_heads > 0 and q_heads // kv_heads <= 16 and qkv.is_contiguous()
            and qkv.data_ptr() % 16 == 0 and batch.num_requests == qkv.shape[0])


def attention_decode_qk(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, q_weight: Optional[torch.Tensor],
                        k_weight: Optional[torch.Tensor], inv_freq: Optional[torch.Tensor], eps: float, cache: torch.Tensor,
                        block_table: torch.Tensor, batch, window: Optional[int], scale: float) -> torch.Tensor:
    """A decode step's attention with its preparation inside the kernel: ``qkv`` [R, (nq + 2 nkv) d] as the q, k, v
    product left it (not modified).  Per-head RMSNorm of q and k, rotation at each request's position, the new token's
    key and value appended to its page, attention over the pages: one kernel, where the separate path runs
    ``qk_norm_rope_kv_write_`` and then the decode kernel.  The result equals that path's bit for bit."""
    _need_cuda(qkv, q_weight, k_weight, inv_freq, cache, block_table, batch.context_len)
    num_pages, c_heads, page_size, c_dim = _cache_dims(cache)
    rows = qkv.shape[0]
    assert (c_heads, c_dim) == (kv_heads, head_dim) and qkv.shape[1] == (q_heads + 2 * kv_heads) * head_dim
    for w in (q_weight, k_weight):
        assert w is None or (w.dtype == torch.float32 and w.numel() == head_dim and w.is_contiguous())
    assert inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2 and inv_freq.is_contiguous())
    context_len = batch.context_len
    out = torch.empty((rows, q_heads * head_dim), dtype=qkv.dtype, device=qkv.device)
    balanced = getattr(batch, "decode_balanced", None)
    longest = batch.max_context_len
    room = decode_cluster_room(qkv.device, head_dim, q_heads // kv_heads)
    if balanced is None:
        lens = [start + count for start, count in zip(batch.start_positions, batch.query_lens)]
        balanced, _ = decode_plan(lens, kv_heads, window, sms=sm_count(qkv.device), room=room, head_dim=head_dim,
                                  group=q_heads // kv_heads)
        longest = max(lens)
    forced = os.environ.get("KIRAI_DECODE_BALANCED")
    if forced in ("0", "1"):
        balanced = forced == "1"
    tail = (_ptr(q_weight), _ptr(k_weight), _ptr(inv_freq), _f(eps), _ptr(error_flag(qkv.device)), _stream())
    common = (_ptr(block_table), _ptr(context_len), _i(rows), _i(q_heads), _i(kv_heads), _i(head_dim), _l(qkv.stride(0)),
              _i(page_size), _i(block_table.shape[1]), _i(num_pages), _i(window or 0), _f(scale))
    if balanced and rows <= 1024:
        ctas = sm_count(qkv.device)
        partial = torch.empty((ctas, 2, 16, head_dim + 2), dtype=torch.float32, device=qkv.device)
        _call("kirai_attention_decode_balanced_qk_bf16", _ptr(qkv), _ptr(cache), _ptr(out), _ptr(partial), *common, _i(ctas), *tail)
        return out
    splits = getattr(batch, "decode_splits", None) or decode_splits(rows, kv_heads, min(longest, window or longest), sms=sm_count(qkv.device),
                                                                    room=room, head_dim=head_dim, group=q_heads // kv_heads)
    partial = None
    if splits > 1 and not decode_pair_merges(rows * kv_heads, splits, head_dim, room, q_heads // kv_heads):
        partial = torch.empty((rows, q_heads, splits, head_dim + 2), dtype=torch.float32, device=qkv.device)
    _call("kirai_attention_decode_qk_bf16", _ptr(qkv), _ptr(cache), _ptr(out), _ptr(partial), *common, _i(splits), *tail)
    return out


# ------------------------------------------------------------------------ linear
def linear_plain(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x`` [M, K] times ``weight`` [N, K] transposed on the CUDA cores with 32-bit FMAs."""
    _need_cuda(x, weight)
    assert x.dim() == 2 and x.stride(1) == 1 and weight.dim() == 2 and weight.is_contiguous()
    assert x.shape[1] == weight.shape[1] and x.dtype == weight.dtype
    out_dtype = out_dtype or x.dtype
    m, k, n = x.shape[0], x.shape[1], weight.shape[0]
    out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32
        name = "kirai_gemm_simt_f32"
    else:
        name = "kirai_gemm_simt_bf16" if out_dtype == torch.bfloat16 else "kirai_gemm_simt_bf16_out_f32"
    _call(name, _ptr(x), _ptr(weight), _ptr(out), _i(m), _i(n), _i(k), _l(x.stride(0)), _l(n), _stream())
    return out


class TiledWeight:
    """A bf16 weight matrix [N, K] in the layout that the tensor-core product streams fastest: boxes of 128 rows
    x 64 columns, each stored as the 16 KB image that the 128-byte swizzle leaves in shared memory (the 16-byte
    chunk c of row r at chunk c ^ (r % 8)), box (row tile, k block) at index row_tile * ceil(K / 64) + k_block,
    zero-padded at the edges.  One box is one contiguous bulk copy."""

    def __init__(self, boxes: torch.Tensor, rows: int, cols: int):
        self.boxes, self.rows, self.cols = boxes, rows, cols

    @property
    def shape(self):
        return (self.rows, self.cols)

    @property
    def device(self):
        return self.boxes.device

    def row_major(self) -> torch.Tensor:
        """The matrix back in rows (for tests and for kernels that do not read boxes)."""
        row_tiles, k_blocks = self.boxes.shape[:2]
        chunks = self.boxes.view(row_tiles, k_blocks, 128, 8, 8)
        plain = chunks[:, :, torch.arange(128, device=self.device)[:, None], _swizzle_index(self.device), :]
        plain = plain.reshape(row_tiles, k_blocks, 128, 64).permute(0, 2, 1, 3).reshape(row_tiles * 128, k_blocks * 64)
        return plain[: self.rows, : self.cols].contiguous()


def _swizzle_index(device) -> torch.Tensor:
    """[128, 8]: where chunk c of row r lies under the 128-byte swizzle (an involution)."""
    rows = torch.arange(128, device=device)[:, None]
    return torch.arange(8, device=device)[None, :] ^ (rows % 8)


def tile_weight(weight: torch.Tensor) -> TiledWeight:
    """Re-packs a bf16 matrix [N, K] on the device into the tiled layout (done once, at load)."""
    _need_cuda(weight)
    assert weight.dim() == 2 and weight.dtype == torch.bfloat16
    n, k = weight.shape
    row_tiles, k_blocks = (n + 127) // 128, (k + 63) // 64
    if row_tiles * 128 != n or k_blocks * 64 != k:
        padded = torch.zeros((row_tiles * 128, k_blocks * 64), dtype=weight.dtype, device=weight.device)
        padded[:n, :k] = weight
    else:
        padded = weight
    boxes = padded.view(row_tiles, 128, k_blocks, 8, 8).permute(0, 2, 1, 3, 4)  # [row tile, k block, row, chunk, 8]
    boxes = boxes[:, :, torch.arange(128, device=weight.device)[:, None], _swizzle_index(weight.device), :]
    boxes = boxes.reshape(row_tiles, k_blocks, 128 * 64).contiguous()
    tiled_bytes = library().kirai_gemm_bf16_tiled_bytes
    tiled_bytes.restype = ctypes.c_long
    assert boxes.numel() * 2 == int(tiled_bytes(_i(n), _i(k)))
    return TiledWeight(boxes, n, k)


# ---- products held back and launched together
# A decode step of a few tokens runs product after product, each bound by its weight stream, and every launch pays a
# ramp of its own.  Inside ``chained_products()`` a product of at most 64 rows with tiled weights is not launched at
# once: it is put on a list, and the list goes out as ONE persistent kernel (csrc/gemm_chain.cu, whose weight stream
# runs on from product to product) as soon as anything else is launched or the block ends.  Results are therefore
# not computed when ``linear_tcgen05`` returns, only when the next kernel of another kind has been asked for: code
# inside such a block must touch activations through the functions of this module only (every one of them sends the
# list out first), never through torch arithmetic or a copy to the host.
chain_stamps = None     # a tensor of sms * 6 * 4 int64: the chain kernel writes its clock stamps there (measurements)
# Off by default: on the 8B layer sizes the chain measured slower than the products launched one by one (see the
# head of csrc/gemm_chain.cu for the figures and the reasons); True lets the model's steps use it.
chain_products = False
_chain_depth = 0
_pending: list = []
_chain_workspaces: dict = {}


class chained_products:
    """``with ops.chained_products(): ...`` holds products back as described above; ``enabled=False`` does nothing."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and chain_products

    def __enter__(self):
        global _chain_depth
        if self.enabled:
            _chain_depth += 1
        return self

    def __exit__(self, kind, value, traceback):
        global _chain_depth
        if self.enabled:
            _chain_depth -= 1
            if _chain_depth == 0:
                if kind is None:
                    flush_products()
                else:
                    _pending.clear()  # an error on the way: nothing half-described is launched
        return False


def chaining() -> bool:
    """Whether products are being held back right now."""
    return _chain_depth > 0 and chain_products


def _chain_workspace(device: torch.device) -> torch.Tensor:
    """One workspace per device (partial tiles and counters, 10 MB): chains on one device run one after the other, as
    everything of a step does; two streams that ran chains at the same time would need one each."""
    key = torch.device(device)
    if key.index is None:
        key = torch.device("cuda", torch.cuda.current_device())
    if key not in _chain_workspaces:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the workspace of chained products must exist before a stream capture begins: "
                              "run the step once outside the capture")
        size = library().kirai_gemm_chain_workspace_bytes
        size.restype = ctypes.c_long
        _chain_workspaces[key] = torch.zeros(int(size()), dtype=torch.uint8, device=device)
    return _chain_workspaces[key]


def _launch_product(item) -> None:
    x, weight, out, n, k, width, splits, form, row_scale, resid, norm_weight, sumsq_out = item
    tiled = isinstance(weight, TiledWeight)
    if row_scale is not None:
        sumsq, count, eps = row_scale
        scale_args = (_ptr(sumsq), _i(sumsq.shape[0]), _f(float(count)), _f(float(eps)))
    else:
        scale_args = (_ptr(None), _i(0), _f(1.0), _f(0.0))
    _launch("kirai_gemm_bf16_general", _ptr(x), _ptr(weight.boxes if tiled else weight), _i(tiled), _ptr(out), _i(x.shape[0]),
            _i(n), _i(k), _l(x.stride(0)), _l(width), _i(splits), _i(form), *scale_args,
            _ptr(resid), _ptr(norm_weight), _ptr(sumsq_out), _ptr(error_flag(x.device)), _stream(),
            detail=f" m={x.shape[0]} n={n} k={k} form={form}" if _timer is not None else "")


def flush_products() -> None:
    """Launches the products that were held back: one alone through the single-product kernel, several as one chain."""
    global _pending
    items, _pending = _pending, []
    if not items:
        return
    if len(items) > 1:
        count = len(items)
        pointers, longs, ints, floats = ctypes.c_void_p * count, ctypes.c_long * count, ctypes.c_int * count, ctypes.c_float * count

        def ptrs(values):
            return pointers(*[0 if v is None else v.data_ptr() for v in values])

        x0 = items[0][0]
        workspace = _chain_workspace(x0.device)
        scales = [item[8] for item in items]
        fn = library().kirai_gemm_chain_bf16
        fn.restype = ctypes.c_int
        status = fn(
            _i(count), _i(x0.shape[0]), ptrs([item[0] for item in items]), longs(*[item[0].stride(0) for item in items]),
            ptrs([item[1].boxes for item in items]), ptrs([item[2] for item in items]), longs(*[item[5] for item in items]),
            ints(*[item[3] for item in items]), ints(*[item[4] for item in items]), ints(*[item[7] for item in items]),
            ptrs([None if sc is None else sc[0] for sc in scales]), ints(*[0 if sc is None else sc[0].shape[0] for sc in scales]),
            floats(*[1.0 if sc is None else float(sc[1]) for sc in scales]), floats(*[0.0 if sc is None else float(sc[2]) for sc in scales]),
            ptrs([item[9] for item in items]), ptrs([item[10] for item in items]), ptrs([item[11] for item in items]),
            _ptr(workspace), _l(workspace.numel()), _ptr(error_flag(x0.device)), _ptr(chain_stamps), _stream())
        if status == 0:
            global launch_count
            launch_count += 1
            launch_counts["kirai_gemm_chain_bf16"] = launch_counts.get("kirai_gemm_chain_bf16", 0) + 1
            return
        if status not in _REFUSALS:
            _check(status, "kirai_gemm_chain_bf16")
        # refused (a shape the chain does not take): one by one
    for item in items:
        _launch_product(item)


def _gemm(x, weight, out, n: int, k: int, width: int, splits: int, form: int, row_scale, resid, norm_weight, sumsq_out):
    if row_scale is not None:
        sumsq = row_scale[0]
        assert sumsq.dtype == torch.float32 and sumsq.dim() == 2 and sumsq.shape[1] == x.shape[0] and sumsq.is_contiguous()
    item = (x, weight, out, n, k, width, splits, form, row_scale, resid, norm_weight, sumsq_out)
    if chaining() and isinstance(weight, TiledWeight) and x.shape[0] <= 64 and splits == 0 and form not in (4, 5):
        if _pending and _pending[0][0].shape[0] != x.shape[0]:
            flush_products()
        _pending.append(item)
        limit = library().kirai_gemm_chain_max_phases
        limit.restype = ctypes.c_int
        if len(_pending) >= int(limit()):
            flush_products()
        return
    if _pending:
        flush_products()
    _launch_product(item)


def _check_product(x, weight) -> tuple:
    if isinstance(weight, TiledWeight):
        _need_cuda(x, weight.boxes)
    else:
        _need_cuda(x, weight)
        assert weight.dim() == 2 and weight.is_contiguous() and weight.dtype == torch.bfloat16
    assert x.dim() == 2 and x.stride(1) == 1 and x.dtype == torch.bfloat16 and x.shape[1] == weight.shape[1]
    return x.shape[0], x.shape[1], weight.shape[0]


def linear_tcgen05(x: torch.Tensor, weight, out_dtype: Optional[torch.dtype] = None,
                   splits: int = 0, swiglu: bool = False, row_scale: Optional[tuple] = None,
                   gate_act: str = "silu", relu2: bool = False) -> torch.Tensor:
    """bf16 ``x`` [M, K] times ``weight`` [N, K] transposed on the tcgen05 tensor cores (32-bit accumulation).

    ``weight`` is a row-major tensor or a ``TiledWeight``.  K and the row stride of ``x`` must be multiples of 8
    (TMA reads rows in 16-byte units).  ``splits`` > 1 cuts K between the CTAs of a cluster (0: chosen from the
    shape, at most 4).  With ``swiglu`` the rows of ``weight`` are 8 gate rows, their 8 up rows, 8 gate rows, ...
    and the result is silu(gate) * up, [M, N / 2] (``gate_act`` "gelu_tanh": the tanh form of gelu in place of silu).
    ``row_scale`` = (sumsq [P, M] float32, count, eps) multiplies
    row m of the product by 1 / sqrt(sum_p sumsq[p, m] / count + eps): ``x`` then holds rows that an RMSNorm left
    unscaled.  ``relu2``: the result is relu(product)^2 (bfloat16).
    """
    m, k, n = _check_product(x, weight)
    out_dtype = out_dtype or torch.bfloat16
    if swiglu:
        assert out_dtype == torch.bfloat16 and n % 16 == 0 and not relu2
    if relu2:
        assert out_dtype == torch.bfloat16
    width = n // 2 if swiglu else n
    out = torch.empty((m, width), dtype=out_dtype, device=x.device)
    form = (5 if gate_act == "gelu_tanh" else 2) if swiglu else (4 if relu2 else (0 if out_dtype == torch.bfloat16 else 1))
    assert gate_act in GATED_ACTIVATIONS
    _gemm(x, weight, out, n, k, width, splits, form, row_scale, None, None, None)
    return out


def linear_residual_norm(x: torch.Tensor, weight, resid: torch.Tensor, norm_weight: torch.Tensor,
                         splits: int = 0) -> tuple:
    """``resid`` [M, N] (float32, in place) += ``x`` [M, K] times ``weight`` [N, K] transposed, on the tensor cores;
    returns (bf16(resid * norm_weight) [M, N], sumsq [P, M]): the rows of the next RMSNorm without their
    1 / rms factor, and the parts of each row's sum of squares, which ``linear_tcgen05(row_scale=...)`` applies."""
    m, k, n = _check_product(x, weight)
    _need_cuda(resid, norm_weight)
    assert resid.dtype == torch.float32 and resid.shape == (m, n) and resid.is_contiguous()
    assert norm_weight.dtype == torch.float32 and norm_weight.shape == (n,) and norm_weight.is_contiguous()
    parts = int(library().kirai_gemm_bf16_residual_parts(_i(m), _i(n)))
    rows = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty((parts, m), dtype=torch.float32, device=x.device)
    _gemm(x, weight, rows, n, k, n, splits, 3, None, resid, norm_weight, sumsq)
    return rows, sumsq


def linear_relu2_takes(x: torch.Tensor, weight) -> bool:
    """Whether ``linear_relu2`` runs for these operands: the tensor-core product with the activation in its epilogue."""
    n = weight.shape[0]
    return tcgen05_takes(x) and n % 8 == 0 and (isinstance(weight, TiledWeight) or weight.dtype == torch.bfloat16)


def linear_relu2(x: torch.Tensor, weight) -> torch.Tensor:
    """relu(``x`` ``weight``^T)^2 in bfloat16, the activation in the product's epilogue."""
    return linear_tcgen05(x, weight, torch.bfloat16, relu2=True)


def tcgen05_takes(x: torch.Tensor) -> bool:
    """Whether the tensor-core GEMM can read ``x`` [M, K] (bf16, 16-byte aligned rows)."""
    return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and x.stride(1) == 1
            and x.data_ptr() % 16 == 0)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stacks gate [I, K] and up [I, K] as 8 gate rows, their 8 up rows, ... (I a multiple of 8),
    the row order that the SwiGLU epilogue of the tensor-core GEMM reads."""
    inter, k = gate.shape
    assert up.shape == gate.shape and inter % 8 == 0
    return torch.stack([gate.view(inter // 8, 8, k), up.view(inter // 8, 8, k)], dim=1).reshape(2 * inter, k).contiguous()


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """The linear layer of the product path: 32-bit FMAs for float32; for bfloat16 the tcgen05
    kernel, or the CUDA-core kernel when K is not a multiple of 8 (TMA cannot read such rows)."""
    if isinstance(weight, TiledWeight):
        return linear_tcgen05(x if tcgen05_takes(x) else x.contiguous(), weight, out_dtype)
    if tcgen05_takes(x):
        return linear_tcgen05(x, weight, out_dtype)
    return linear_plain(x, weight, out_dtype)


# ------------------------------------------------------------------------ SwiGLU
def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """silu(gate) * up for ``gate_up`` [T, 2 I] (gate half first); returns [T, I]."""
    _need_cuda(gate_up)
    assert gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _call(f"kirai_swiglu_{_suffix(gate_up.dtype)}", _ptr(gate_up), _ptr(out), _i(rows), _i(inter), _stream())
    return out


def decode_advance(token_ids: torch.Tensor, sampled: torch.Tensor, positions: torch.Tensor, context_len: torch.Tensor) -> None:
    """token_ids <- sampled; positions += 1; context_len += 1 (all int32 [R], on the device)."""
    _need_cuda(token_ids, sampled, positions, context_len)
    for t in (token_ids, sampled, positions, context_len):
        assert t.dtype == torch.int32 and t.is_contiguous() and t.numel() == token_ids.numel()
    _call("kirai_decode_advance", _ptr(token_ids), _ptr(sampled), _ptr(positions), _ptr(context_len),
          _i(token_ids.numel()), _stream())


# ---------------------------------------------------------------------- sampling
def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """Index of the greatest logit of each row, the lowest index on ties."""
    _need_cuda(logits)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.is_contiguous()
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _call("kirai_argmax_rows", _ptr(logits), _ptr(out), _i(logits.shape[0]), _i(logits.shape[1]),
          _ptr(error_flag(logits.device)), _stream())
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, draw: torch.Tensor) -> torch.Tensor:
    """One token per row: greedy where temperature is 0, else nucleus sampling with the row's draw."""
    _need_cuda(logits, temperature, top_p, draw)
    assert logits.dim() == 2 and logits.dtype == torch.float32 and logits.is_contiguous()
    rows = logits.shape[0]
    for t in (temperature, top_p, draw):
        assert t.dtype == torch.float32 and t.numel() == rows and t.is_contiguous()
    needs_scratch = library().kirai_sample_rows_needs_scratch
    needs_scratch.restype = ctypes.c_int
    scratch = torch.empty_like(logits) if needs_scratch(_i(rows), _i(logits.shape[1])) else None
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    _call("kirai_sample_rows", _ptr(logits), _ptr(scratch), _ptr(temperature), _ptr(top_p), _ptr(draw), _ptr(out),
          _i(rows), _i(logits.shape[1]), _ptr(error_flag(logits.device)), _stream())
    return out
