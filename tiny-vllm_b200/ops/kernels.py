"""Python face of the CUDA kernels: tensors in, launch on the current stream.

Every function checks shapes and dtypes, refuses what its kernel does not take
with a clear error, and raises :class:`KernelError` if the launch fails.  There
is no other implementation behind these functions: without a GPU and a built
library they raise.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    """A kernel refused its arguments or its launch failed."""


def dtype_tag(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 and bfloat16, not {dtype}")


def _stream() -> int:
    # the raw handle of the current stream of the current device: the same value as
    # torch.cuda.current_stream().cuda_stream without building a Stream object (this runs once a launch)
    return torch._C._cuda_getCurrentRawStream(torch._C._cuda_getDevice())


_launches = 0

# Programmatic dependent launch for the kernels that wait for their predecessor themselves
# (griddepcontrol.wait): they may start, and fetch weights, while the kernel before them ends.
# TINYVLLM_B200_PDL=0 turns it off; a comma-separated list (gemm,norm,attention,attention_few,prefill,
# sample) keeps it for those kernels only (attention: the decode attention at every batch size;
# attention_few: with up to PDL_ATTENTION_ROWS rows and only where the launch runs as CTAs of eight
# warps that are all on the GPU at once, which find the SMs free: batch 1 to 3 gain 3 to 4 %, batch
# 4 is level and batch 6 loses 3 %, its clusters waiting for room beside the projection's CTAs; prefill: the prompt's q/k norm, rotation and cache write,
# and the tcgen05 attention).
_PDL_DEFAULT = ("gemm", "norm", "attention_few")
PDL_ATTENTION_ROWS = 3
_setting = os.environ.get("TINYVLLM_B200_PDL", "1")
PDL = frozenset() if _setting == "0" else frozenset(_PDL_DEFAULT if _setting == "1" else _setting.split(","))


def _pdl(kind: str) -> int:
    return 1 if kind in PDL else 0


def launch_count() -> int:
    """Kernels of this package launched so far by this process (graph replays not counted)."""
    return _launches


def _check(code: int, what: str, launches: int = 1) -> None:
    global _launches
    if code == 0:
        _launches += launches
        return
    if code < 0:
        raise KernelError(f"{what}: the kernel does not take these sizes")
    raise KernelError(f"{what}: CUDA error {code}")


def _need_cuda(*tensors: torch.Tensor) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU path")


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


_functions: dict[str, ctypes._CFuncPtr] = {}


def _fn(library: str, name: str, argtypes, restype=c_int):
    function = _functions.get(name)
    if function is None:
        function = getattr(load_library(library), name)
        function.argtypes = argtypes
        function.restype = restype
        _functions[name] = function
    return function


def _fn_of(library: str, name: str, argtypes, restype=c_int):
    """:func:`_fn` for a function that several libraries define (one per head size and weight type)."""
    key = f"{library}:{name}"
    function = _functions.get(key)
    if function is None:
        function = getattr(load_library(library), name)
        function.argtypes = argtypes
        function.restype = restype
        _functions[key] = function
    return function


DECODE_HEAD_DIMS = (64, 128, 256)
BF16_OR_F32 = {F32: torch.float32, BF16: torch.bfloat16}


def _decode_library(head_dim: int, weight_tag: int) -> str:
    """The fused decode attention is compiled per head size and type of norm weights."""
    if head_dim not in DECODE_HEAD_DIMS:
        raise KernelError(f"attention_decode takes head sizes {DECODE_HEAD_DIMS}, not {head_dim}")
    return f"attention_decode_{head_dim}_{'f32' if weight_tag == F32 else 'bf16'}"


# ------------------------------------------------------------------ embedding
def embed_rows(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]]; ids int32."""
    _need_cuda(table, ids)
    if ids.dtype != torch.int32 or ids.dim() != 1 or table.dim() != 2 or not table.is_contiguous():
        raise KernelError("embed_rows wants a contiguous [vocab, width] table and int32 ids [tokens]")
    rows, (vocab, width) = ids.shape[0], table.shape
    if out is None:
        out = torch.empty((rows, width), dtype=table.dtype, device=table.device)
    fn = _fn("pointwise", "tvb_embed_rows",
             [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(table.data_ptr(), ids.data_ptr(), out.data_ptr(), rows, width, vocab,
              dtype_tag(table.dtype), _stream()), "embed_rows")
    return out


# -------------------------------------------------------------------- RMSNorm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, *, residual: torch.Tensor | None = None,
             rows: torch.Tensor | None = None, out: torch.Tensor | None = None,
             residual_out: torch.Tensor | None = None, want_residual: bool = True):
    """RMSNorm over the last dimension of x [tokens, width].

    With ``residual`` the rounded sum x + residual is normalised and returned as
    the second result (the new residual stream).  With ``rows`` (int32) only
    those rows are produced, in that order, and no residual is returned.
    """
    _need_cuda(x, weight, residual, rows)
    if x.dim() != 2 or not x.is_contiguous() or weight.shape != (x.shape[1],):
        raise KernelError("rms_norm wants contiguous x [tokens, width] and weight [width]")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype
                                 or not residual.is_contiguous()):
        raise KernelError("rms_norm: residual must match x")
    width = x.shape[1]
    if width * 4 > 200 * 1024:
        raise KernelError(f"rms_norm: width {width} is larger than a row buffer of shared memory holds")
    count = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("rms_norm: rows must be int32")
    if out is None:
        out = torch.empty((count, width), dtype=x.dtype, device=x.device)
    if residual is not None and rows is None and want_residual and residual_out is None:
        residual_out = torch.empty_like(x)
    if rows is not None or residual is None:
        residual_out = None
    if x.dtype == torch.bfloat16 and width % 8 == 0 and width <= 8192:     # 16-byte accesses
        fn = _fn("pointwise_bf16", "tvb_rms_norm_bf16",
                 [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
                  c_int, c_int, c_void_p])
        _check(fn(x.data_ptr(), _ptr(residual), weight.data_ptr(), out.data_ptr(), _ptr(residual_out),
                  _ptr(rows), count, width, eps, dtype_tag(weight.dtype), _pdl("norm"), _stream()),
               "rms_norm")
        if residual is not None and rows is None:
            return out, residual_out
        return out
    fn = _fn("pointwise", "tvb_rms_norm",
             [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float,
              c_int, c_int, c_int, c_void_p])
    _check(fn(x.data_ptr(), _ptr(residual), weight.data_ptr(), out.data_ptr(), _ptr(residual_out),
              _ptr(rows), count, width, eps, dtype_tag(x.dtype), dtype_tag(weight.dtype), _pdl("norm"),
              _stream()), "rms_norm")
    if residual is not None and rows is None:
        return out, residual_out
    return out


# ------------------------------------------------------------- SiLU(gate) * up
def silu_mul(gate_up: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """round(round(silu(gate)) * up) of packed rows [tokens, 2 * inter]."""
    _need_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelError("silu_mul wants contiguous [tokens, 2 * inter]")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    if gate_up.dtype == torch.bfloat16 and inter % 8 == 0:
        fn = _fn("pointwise_bf16", "tvb_silu_mul_bf16", [c_void_p, c_void_p, c_int, c_int, c_void_p])
        _check(fn(gate_up.data_ptr(), out.data_ptr(), rows, inter, _stream()), "silu_mul")
        return out
    fn = _fn("pointwise", "tvb_silu_mul", [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(gate_up.data_ptr(), out.data_ptr(), rows, inter, dtype_tag(gate_up.dtype), _stream()),
           "silu_mul")
    return out


# -------------------------------------------------------------- rotary tables
def rope_tables(inv_freq: torch.Tensor, positions: int) -> tuple[torch.Tensor, torch.Tensor]:
    """float32 cos and sin of position * inv_freq[j], [positions, half]."""
    _need_cuda(inv_freq)
    if inv_freq.dtype != torch.float32 or inv_freq.dim() != 1:
        raise KernelError("rope_tables wants float32 inv_freq [half]")
    half = inv_freq.shape[0]
    cos = torch.empty((positions, half), dtype=torch.float32, device=inv_freq.device)
    sin = torch.empty_like(cos)
    fn = _fn("pointwise", "tvb_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(inv_freq.data_ptr(), cos.data_ptr(), sin.data_ptr(), positions, half, _stream()),
           "rope_tables")
    return cos, sin


# ------------------------------------ q/k norm + rotation + cache write, fused
def qk_norm_rope_store(qkv: torch.Tensor, *, num_q: int, num_kv: int, head_dim: int,
                       positions: torch.Tensor, q_weight: torch.Tensor | None,
                       k_weight: torch.Tensor | None, eps: float,
                       cos: torch.Tensor | None, sin: torch.Tensor | None,
                       slots: torch.Tensor | None, key_cache: torch.Tensor | None,
                       value_cache: torch.Tensor | None) -> None:
    """In place on the packed projection [tokens, (num_q + 2 num_kv) * head_dim]: q heads are
    normalised and rotated where they stand; k heads are normalised, rotated and written to
    ``key_cache`` at ``slots`` (page * page_size + offset); v heads are copied to
    ``value_cache``.  Caches are [pages, num_kv, page_size, head_dim]; without ``slots``
    nothing is written."""
    _need_cuda(qkv, positions, q_weight, k_weight, cos, sin, slots, key_cache, value_cache)
    tokens = qkv.shape[0]
    if qkv.dim() != 2 or not qkv.is_contiguous() or qkv.shape[1] != (num_q + 2 * num_kv) * head_dim:
        raise KernelError("qk_norm_rope_store: qkv must be contiguous [tokens, (q + 2 kv) * head_dim]")
    if head_dim % 2 or head_dim > 256:
        raise KernelError(f"qk_norm_rope_store takes even head sizes up to 256, not {head_dim}")
    if positions.dtype != torch.int32 or positions.shape != (tokens,):
        raise KernelError("qk_norm_rope_store: positions must be int32 [tokens]")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("qk_norm_rope_store: q and k norm weights come together")
    weight_tag = dtype_tag(qkv.dtype)
    if q_weight is not None:
        if q_weight.shape != (head_dim,) or k_weight.shape != (head_dim,) or q_weight.dtype != k_weight.dtype:
            raise KernelError("qk_norm_rope_store: norm weights must be [head_dim] of one dtype")
        weight_tag = dtype_tag(q_weight.dtype)
    table_positions = 0
    if cos is not None:
        if cos.dtype != torch.float32 or cos.shape != sin.shape or cos.shape[1] != head_dim // 2:
            raise KernelError("qk_norm_rope_store: tables must be float32 [positions, head_dim / 2]")
        table_positions = cos.shape[0]
    if slots is not None:
        if (slots.dtype != torch.int32 or slots.shape != (tokens,) or key_cache is None
                or value_cache is None or key_cache.dim() != 4
                or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim)
                or key_cache.dtype != qkv.dtype or value_cache.shape != key_cache.shape
                or not key_cache.is_contiguous() or not value_cache.is_contiguous()):
            raise KernelError("qk_norm_rope_store: slots int32 [tokens]; caches contiguous "
                              "[pages, num_kv, page_size, head_dim] of the dtype of qkv")
    page_size = key_cache.shape[2] if slots is not None else 0
    if qkv.dtype == torch.bfloat16 and head_dim in (16, 32, 64, 128, 256):
        fn = _fn("pointwise_bf16", "tvb_qk_norm_rope_store_bf16",
                 [c_void_p] * 9 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p])
        _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
                  positions.data_ptr(), _ptr(slots), _ptr(key_cache), _ptr(value_cache), tokens, num_q,
                  num_kv, head_dim, page_size, table_positions, eps, weight_tag, _pdl("prefill"), _stream()),
               "qk_norm_rope_store")
        return
    fn = _fn("pointwise", "tvb_qk_norm_rope_store",
             [c_void_p] * 9 + [c_int] * 6 + [c_float, c_int, c_int, c_void_p])
    _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
              positions.data_ptr(), _ptr(slots), _ptr(key_cache), _ptr(value_cache), tokens, num_q,
              num_kv, head_dim, page_size, table_positions, eps, dtype_tag(qkv.dtype), weight_tag,
              _stream()),
           "qk_norm_rope_store")


# ------------------------------------------------------------------ attention
_chunk_keys: int | None = None


def attention_chunk_keys() -> int:
    global _chunk_keys
    if _chunk_keys is None:
        _chunk_keys = _fn("attention_rows", "tvb_attention_chunk_keys", [])()
    return _chunk_keys


ATTENTION_ROWS_MAX_DIM = 640      # 32 lanes * ATTN_WIDE_DIMS of attention_rows.cu


def attention_rows_scratch_floats(tokens: int, num_q: int, head_dim: int, max_chunks: int) -> int:
    """``head_dim``: the size of a value."""
    return tokens * num_q * max_chunks * (head_dim + 2)


def attention_rows(q: torch.Tensor, q_token_stride: int, key_cache: torch.Tensor,
                   value_cache: torch.Tensor, block_tables: torch.Tensor, token_row: torch.Tensor,
                   positions: torch.Tensor, *, num_q: int, num_kv: int, head_dim: int,
                   window: int | None, scale: float, out: torch.Tensor | None = None,
                   scratch: torch.Tensor | None = None, max_chunks: int = 0,
                   value_dim: int | None = None, keep_first: int = 0,
                   gate: torch.Tensor | None = None, gate_per_head: bool = False,
                   slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                   value_offset: int | None = None, bias_table: torch.Tensor | None = None,
                   segment: int | None = None) -> torch.Tensor:
    """Paged causal attention, one warp per (token, head).

    ``q`` holds the query heads of token t at ``t * q_token_stride`` elements
    (the packed projection serves as it is).  ``max_chunks > 0`` spreads the
    chunks of every row over the grid and needs ``scratch`` (float32, at least
    :func:`attention_rows_scratch_floats` long); 0 walks them in one warp.
    ``value_dim``: size of a value if it is not ``head_dim``; ``keep_first``: with a window, the
    first so many keys stay visible; ``gate`` [tokens, num_q * value_dim] (rows may be strided):
    the output is multiplied by sigmoid(gate); with ``gate_per_head`` the gate is [tokens, num_q],
    one number a head; ``out`` may have strided rows too.  ``slopes`` (float32 [num_q]): slope *
    (position - j) is taken off the score of key j; ``sinks`` (float32 [num_q]): exp(sink) joins the
    softmax's denominator once.  ``value_offset``: the values are the ``value_dim`` elements from
    there on of every key row (``value_cache`` is then None).  ``bias_table`` (float32 [rows, num_q]):
    table[min(position - j, rows - 1), head] is added to the score of key j; ``segment``: the query at
    position p sees only the keys from p - p % segment on."""
    _need_cuda(q, key_cache, value_cache, block_tables, token_row, positions, scratch, gate, slopes, sinks,
               bias_table)
    if bias_table is not None and (bias_table.dtype != torch.float32 or bias_table.dim() != 2
                                   or bias_table.shape[1] != num_q or bias_table.shape[0] < 1
                                   or not bias_table.is_contiguous()):
        raise KernelError("attention_rows: the bias table must be contiguous float32 [distances, num_q]")
    if segment is not None and segment <= 0:
        raise KernelError("attention_rows: a segment holds at least one position")
    tokens = positions.shape[0]
    value_dim = head_dim if value_dim is None else value_dim
    if head_dim > ATTENTION_ROWS_MAX_DIM or value_dim > ATTENTION_ROWS_MAX_DIM or num_q % num_kv:
        raise KernelError(f"attention_rows takes head sizes up to {ATTENTION_ROWS_MAX_DIM} and whole groups "
                          f"(head_dim {head_dim}, {num_q} / {num_kv} heads)")
    if key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            key_cache.dtype != q.dtype or not key_cache.is_contiguous():
        raise KernelError("attention_rows: caches must be contiguous [pages, num_kv, page_size, head_dim]")
    if value_offset is not None:
        if value_cache is not None or not 0 <= value_offset <= head_dim - value_dim:
            raise KernelError("attention_rows: values inside the key rows must fit them, and come without a "
                              "value cache")
        value_ptr, value_stride = key_cache.data_ptr() + value_offset * key_cache.element_size(), head_dim
    else:
        if value_cache.shape != key_cache.shape[:3] + (value_dim,) or not value_cache.is_contiguous() or \
                value_cache.dtype != q.dtype:
            raise KernelError("attention_rows: values must be contiguous [pages, num_kv, page_size, value_dim]")
        value_ptr, value_stride = value_cache.data_ptr(), 0
    gate_shape = (tokens, num_q) if gate_per_head else (tokens, num_q * value_dim)
    for name, t, shape in (("out", out, (tokens, num_q * value_dim)), ("gate", gate, gate_shape)):
        if t is not None and (t.dim() != 2 or t.shape != shape or t.stride(1) != 1 or t.dtype != q.dtype):
            raise KernelError(f"attention_rows: {name} must be {list(shape)} of the dtype of q "
                              "with contiguous rows")
    for name, t in (("slopes", slopes), ("sinks", sinks)):
        if t is not None and (t.dtype != torch.float32 or t.shape != (num_q,) or not t.is_contiguous()):
            raise KernelError(f"attention_rows: {name} must be contiguous float32 [num_q]")
    for name, t in (("block_tables", block_tables), ("token_row", token_row), ("positions", positions)):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError(f"attention_rows: {name} must be contiguous int32")
    if block_tables.dim() != 2 or token_row.shape != (tokens,):
        raise KernelError("attention_rows: block_tables [requests, blocks], token_row [tokens]")
    if out is None:
        out = torch.empty((tokens, num_q * value_dim), dtype=q.dtype, device=q.device)
    if max_chunks > 0:
        need = attention_rows_scratch_floats(tokens, num_q, value_dim, max_chunks)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention_rows: split mode needs {need} float32 of scratch")
    fn = _fn("attention_rows", "tvb_attention_rows_masked",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int,
              c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(q.data_ptr(), q_token_stride, key_cache.data_ptr(), value_ptr, value_stride,
              block_tables.data_ptr(), block_tables.shape[1], token_row.data_ptr(),
              positions.data_ptr(), out.data_ptr(), out.stride(0), _ptr(gate),
              0 if gate is None else gate.stride(0), 1 if gate_per_head else 0, _ptr(slopes), _ptr(sinks),
              _ptr(bias_table), 0 if bias_table is None else bias_table.shape[0], segment or 0,
              _ptr(scratch), max_chunks, tokens, num_q, num_kv,
              head_dim, value_dim, key_cache.shape[2], window or 0, keep_first if window else 0, scale,
              dtype_tag(q.dtype), _stream()),
           "attention_rows", 2 if max_chunks > 0 else 1)
    return out



# ------------------------------------------------ a float32 residual stream
def stream_norm(stream: torch.Tensor | None, weight: torch.Tensor | None, eps: float, *,
                add: torch.Tensor | None = None, add2: torch.Tensor | None = None,
                rows: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
                want_output: bool = True):
    """The pre-norm of a model whose residual stream is float32 whatever its storage type.

    s' = stream + (add + add2) in float32 (any of the three may be missing, not all), written back
    into ``stream`` (a new tensor without one); y = s' * rsqrt(mean(s'^2) + eps) * weight, rounded
    once, in ``out_dtype``.  Returns (y, s').  With ``rows`` (int32) only those rows of y are
    produced and nothing is written back: (y, None).  ``want_output=False``: only the sum."""
    _need_cuda(stream, weight, add, add2, rows)
    first = stream if stream is not None else add
    if first is None or first.dim() != 2 or not first.is_contiguous():
        raise KernelError("stream_norm wants a contiguous [tokens, width] stream or addend")
    tokens, width = first.shape
    if stream is not None and stream.dtype != torch.float32:
        raise KernelError("stream_norm: the stream is float32")
    if add2 is not None and add is None:
        raise KernelError("stream_norm: a second addend needs a first")
    for t in (add, add2):
        if t is not None and (t.shape != (tokens, width) or not t.is_contiguous() or t.dtype != add.dtype):
            raise KernelError("stream_norm: addends must match the stream's shape and each other's dtype")
    if width * 4 > 200 * 1024:
        raise KernelError(f"stream_norm: width {width} is larger than a row buffer of shared memory holds")
    if want_output and (weight is None or weight.shape != (width,)):
        raise KernelError("stream_norm wants a weight [width]")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("stream_norm: rows must be int32")
    count = tokens if rows is None else rows.shape[0]
    out_dtype = out_dtype or (add.dtype if add is not None and add.dtype != torch.float32 else
                              weight.dtype if weight is not None else torch.float32)
    y = torch.empty((count, width), dtype=out_dtype, device=first.device) if want_output else None
    stream_out = None
    if rows is None:
        stream_out = stream if stream is not None else torch.empty((tokens, width), dtype=torch.float32,
                                                                   device=first.device)
    fn = _fn("stream_norm", "tvb_stream_norm",
             [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_float, c_int, c_void_p])
    _check(fn(_ptr(stream), _ptr(add), _ptr(add2), dtype_tag(add.dtype) if add is not None else F32,
              _ptr(weight) if want_output else None,
              dtype_tag(weight.dtype) if weight is not None else dtype_tag(out_dtype), _ptr(y),
              dtype_tag(out_dtype), _ptr(stream_out), _ptr(rows), count, width, eps, _pdl("norm"), _stream()),
           "stream_norm")
    return y, stream_out


def sandwich_norm(stream: torch.Tensor, y: torch.Tensor | None, *, post_weight: torch.Tensor | None = None,
                  pre_weight: torch.Tensor | None = None, post_eps: float = 0.0, pre_eps: float = 0.0,
                  row_scale: torch.Tensor | None = None, x: torch.Tensor | None = None,
                  rows: torch.Tensor | None = None, out_dtype: torch.dtype | None = None):
    """A norm behind a sublayer and the norm in front of the next, in one pass over a float32 residual stream.

    t = y + row_scale[:, None] * x (the second term with ``row_scale`` float32 [tokens] and ``x`` [tokens, width]
    of the storage type); s' = stream + t * rsqrt(mean(t^2) + post_eps) * post_weight, written back into
    ``stream`` (without ``post_weight``: s' = stream + t; without ``y``: s' = stream); out = s' * rsqrt(mean(s'^2)
    + pre_eps) * pre_weight, rounded once to ``out_dtype`` (without ``pre_weight`` no out).  All float32.
    Returns (out, stream).  With ``rows`` (int32) only those rows of out are produced and nothing is written
    back: (out, None)."""
    _need_cuda(stream, y, post_weight, pre_weight, row_scale, x, rows)
    if stream.dim() != 2 or stream.dtype != torch.float32 or not stream.is_contiguous():
        raise KernelError("sandwich_norm wants a contiguous float32 [tokens, width] stream")
    tokens, width = stream.shape
    if y is not None and (y.shape != (tokens, width) or not y.is_contiguous()):
        raise KernelError("sandwich_norm: y must match the stream")
    if post_weight is not None and y is None:
        raise KernelError("sandwich_norm: a norm behind the sublayer needs the sublayer's output")
    weights = [w for w in (post_weight, pre_weight) if w is not None]
    for w in weights:
        if w.shape != (width,) or w.dtype != weights[0].dtype or not w.is_contiguous():
            raise KernelError("sandwich_norm: norm weights are contiguous [width] of one dtype")
    out_dtype = out_dtype or (weights[0].dtype if weights else torch.float32)
    if (row_scale is None) != (x is None) or (x is not None and (
            y is None or x.shape != (tokens, width) or x.dtype != out_dtype or not x.is_contiguous()
            or row_scale.shape != (tokens,) or row_scale.dtype != torch.float32 or not row_scale.is_contiguous())):
        raise KernelError("sandwich_norm: a scaled addend is float32 row_scale [tokens] and x [tokens, width] of "
                          "the output's dtype, beside y")
    if width * 4 > 200 * 1024:
        raise KernelError(f"sandwich_norm: width {width} is larger than a row buffer of shared memory holds")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("sandwich_norm: rows must be int32")
    count = tokens if rows is None else rows.shape[0]
    out = torch.empty((count, width), dtype=out_dtype, device=stream.device) if pre_weight is not None else None
    fn = _fn("stream_norm", "tvb_sandwich_norm",
             [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
              c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p])
    _check(fn(stream.data_ptr(), _ptr(y), dtype_tag(y.dtype) if y is not None else F32, _ptr(row_scale), _ptr(x),
              _ptr(post_weight), _ptr(pre_weight), dtype_tag(weights[0].dtype) if weights else dtype_tag(out_dtype),
              _ptr(out), dtype_tag(out_dtype), stream.data_ptr() if rows is None else None, _ptr(rows), count, width,
              post_eps, pre_eps, _pdl("norm"), _stream()), "sandwich_norm")
    return out, (stream if rows is None else None)


def add_scaled_rows(y: torch.Tensor, x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """y[t] += scale[t] * x[t] in place: contiguous float32 y [tokens, width], x of any storage type, float32
    scale [tokens]."""
    _need_cuda(y, x, scale)
    if y.dim() != 2 or y.dtype != torch.float32 or not y.is_contiguous() or x.shape != y.shape \
            or not x.is_contiguous() or scale.shape != (y.shape[0],) or scale.dtype != torch.float32 \
            or not scale.is_contiguous():
        raise KernelError("add_scaled_rows wants float32 y [tokens, width], x of its shape and float32 scale [tokens]")
    fn = _fn("stream_norm", "tvb_add_scaled_rows", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(y.data_ptr(), x.data_ptr(), scale.data_ptr(), y.shape[0], y.shape[1], dtype_tag(x.dtype), _stream()),
           "add_scaled_rows")
    return y


ACT_SILU, ACT_GELU_TANH = 0, 1
ACTIVATIONS = {"silu": ACT_SILU, "gelu_tanh": ACT_GELU_TANH}


def gated_act(packed: torch.Tensor, gate_at: int, up_at: int, inter: int, activation: str, *,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """round(round(act(gate)) * up) where gate and up are the ``inter`` columns of ``packed``
    [tokens, any] from ``gate_at`` and ``up_at`` on; ``out`` [tokens, inter] may have strided rows."""
    _need_cuda(packed, out)
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act knows {', '.join(ACTIVATIONS)}, not {activation!r}")
    if packed.dim() != 2 or packed.stride(1) != 1 or min(gate_at, up_at) < 0 or \
            max(gate_at, up_at) + inter > packed.shape[1]:
        raise KernelError("gated_act wants [tokens, columns] with contiguous rows that hold gate and up")
    tokens = packed.shape[0]
    if out is None:
        out = torch.empty((tokens, inter), dtype=packed.dtype, device=packed.device)
    elif out.shape != (tokens, inter) or out.dtype != packed.dtype or out.stride(1) != 1:
        raise KernelError("gated_act: out must be [tokens, inter] of the input's dtype with contiguous rows")
    fn = _fn("stream_norm", "tvb_gated_act",
             [c_void_p, c_longlong, c_int, c_int, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(packed.data_ptr(), packed.stride(0), gate_at, up_at, out.data_ptr(), out.stride(0), tokens, inter,
              ACTIVATIONS[activation], dtype_tag(packed.dtype), _stream()), "gated_act")
    return out


def sum_pair(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """float32 a + b of two contiguous tensors of one shape and dtype."""
    _need_cuda(a, b)
    if a.shape != b.shape or a.dtype != b.dtype or not a.is_contiguous() or not b.is_contiguous():
        raise KernelError("sum_pair wants two contiguous tensors of one shape and dtype")
    out = torch.empty(a.shape, dtype=torch.float32, device=a.device)
    fn = _fn("stream_norm", "tvb_sum_pair", [c_void_p, c_void_p, c_void_p, c_longlong, c_int, c_void_p])
    _check(fn(a.data_ptr(), b.data_ptr(), out.data_ptr(), a.numel(), dtype_tag(a.dtype), _stream()), "sum_pair")
    return out



# ------------------------------------ layer norm behind the residual sum, over a float32 stream
def post_layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, *, alpha: float = 1.0,
                    add: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                    out_dtype: torch.dtype | None = None, want_stream: bool = True):
    """out = LN(alpha * x + add) * weight, with mean, variance and the sum in float32.

    ``x`` [tokens, width] is the residual stream (float32, or of the storage type where a model
    starts it); ``add`` a sublayer's output (float32 or storage type) or None.  Returns (y, stream):
    ``stream`` is ``out`` in float32 (a new tensor), ``y`` the same values rounded once to
    ``out_dtype``; where ``out_dtype`` is float32 the two are one tensor.  With ``rows`` (int32) only
    those rows are produced, and only y."""
    _need_cuda(x, weight, add, rows)
    if x.dim() != 2 or not x.is_contiguous():
        raise KernelError("post_layer_norm wants a contiguous [tokens, width] stream")
    tokens, width = x.shape
    if add is not None and (add.shape != x.shape or not add.is_contiguous()):
        raise KernelError("post_layer_norm: the addend must match the stream")
    if weight.shape != (width,) or width * 4 > 200 * 1024:
        raise KernelError("post_layer_norm wants a weight [width] and a row that fits shared memory")
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("post_layer_norm: rows must be int32")
    out_dtype = out_dtype or (x.dtype if x.dtype != torch.float32 or weight.dtype == torch.float32 else weight.dtype)
    count = tokens if rows is None else rows.shape[0]
    want_stream = want_stream and rows is None
    stream = torch.empty((count, width), dtype=torch.float32, device=x.device) \
        if want_stream or out_dtype == torch.float32 else None
    y = None if out_dtype == torch.float32 else torch.empty((count, width), dtype=out_dtype, device=x.device)
    fn = _fn("post_norm", "tvb_post_layer_norm",
             [c_void_p, c_int, c_float, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_int, c_int, c_float, c_void_p])
    _check(fn(x.data_ptr(), dtype_tag(x.dtype), alpha, _ptr(add), dtype_tag(add.dtype) if add is not None else F32,
              weight.data_ptr(), dtype_tag(weight.dtype), _ptr(y), dtype_tag(out_dtype), _ptr(stream), _ptr(rows),
              count, width, eps, _stream()), "post_layer_norm")
    return (stream if y is None else y), stream


def scale_float32(x: torch.Tensor, factor: float) -> torch.Tensor:
    """x * factor in place, for a contiguous float32 tensor (logits that a model scales)."""
    _need_cuda(x)
    if x.dtype != torch.float32 or not x.is_contiguous():
        raise KernelError("scale_float32 wants a contiguous float32 tensor")
    fn = _fn("post_norm", "tvb_scale_float32", [c_void_p, c_longlong, c_float, c_void_p])
    _check(fn(x.data_ptr(), x.numel(), factor, _stream()), "scale_float32")
    return x


# ------------------------------------------- norms over whole projections, latents, head products
def projection_norm(proj: torch.Tensor, segments, positions: torch.Tensor | None, eps: float, *,
                    temperature: tuple[float, int] | None = None, store: dict | None = None,
                    rotation: dict | None = None) -> None:
    """In place on a packed projection [tokens, columns]: every segment (first column, columns, weight
    [columns], tempered) becomes v * rsqrt(mean(v^2) + eps) * weight over the whole segment; a tempered
    segment is also multiplied by 1 + coef * ln(floor((p + 1) / every) + 1) of the token's position p
    (``temperature`` = (coef, every)).  One or two segments.  ``store`` (slots int32 [tokens], key_cache
    [pages, num_kv, page, key_dim], value_cache [pages, num_kv, page, value_dim], v_at): the second segment
    is the token's keys, which go, normalised, to its cache rows, together with the values from column
    ``v_at`` on.  ``rotation`` (inv_freq float32 [rot_dims / 2], rot_dims, pairing, head_dim): behind the norm the
    first ``rot_dims`` elements of every head of ``head_dim`` elements, in every segment, turn by position *
    inv_freq (float32), so that the keys reach the cache turned and no other kernel has to prepare q and k."""
    _need_cuda(proj, positions, *[seg[2] for seg in segments])
    inv_freq, rot_dims, halves, head_dim = None, 0, 0, 0
    if rotation is not None:
        inv_freq, rot_dims, head_dim = rotation["inv_freq"], int(rotation["rot_dims"]), int(rotation["head_dim"])
        _need_cuda(inv_freq)
        if rotation["pairing"] not in PAIRINGS or inv_freq.dtype != torch.float32 or rot_dims % 2 or \
                inv_freq.shape != (rot_dims // 2,) or not inv_freq.is_contiguous() or not 0 < rot_dims <= head_dim or \
                any(seg[1] % head_dim for seg in segments) or positions is None or positions.dtype != torch.int32 or \
                positions.shape != (proj.shape[0],):
            raise KernelError("projection_norm: a rotation wants float32 inv_freq [rot_dims / 2], rot_dims <= head_dim, "
                              "segments of whole heads and int32 positions [tokens]")
        halves = PAIRINGS[rotation["pairing"]]
    if proj.dim() != 2 or proj.stride(1) != 1 or not 1 <= len(segments) <= 2:
        raise KernelError("projection_norm wants [tokens, columns] with contiguous rows and one or two segments")
    tokens = proj.shape[0]
    for at, cols, weight, _ in segments:
        if at < 0 or cols <= 0 or at + cols > proj.shape[1] or weight.shape != (cols,) or \
                weight.dtype != segments[0][2].dtype or not weight.is_contiguous():
            raise KernelError("projection_norm: a segment lies inside the row and has a weight of its size")
    coef, every = temperature if temperature is not None else (0.0, 0)
    if any(seg[3] for seg in segments) and every > 0 and (
            positions is None or positions.dtype != torch.int32 or positions.shape != (tokens,)):
        raise KernelError("projection_norm: a temperature needs int32 positions [tokens]")
    first = segments[0]
    second = segments[1] if len(segments) > 1 else (0, 0, None, False)
    slots = key_cache = value_cache = None
    num_kv = key_dim = value_dim = page_size = v_at = 0
    if store is not None:
        slots, key_cache, value_cache, v_at = store["slots"], store["key_cache"], store["value_cache"], store["v_at"]
        _need_cuda(slots, key_cache, value_cache)
        if len(segments) != 2 or key_cache.dim() != 4 or value_cache.dim() != 4 or \
                key_cache.shape[:3] != value_cache.shape[:3] or not key_cache.is_contiguous() or \
                not value_cache.is_contiguous() or key_cache.dtype != proj.dtype or value_cache.dtype != proj.dtype or \
                slots.dtype != torch.int32 or slots.shape != (tokens,):
            raise KernelError("projection_norm: storing needs two segments, int32 slots [tokens] and contiguous caches "
                              "[pages, num_kv, page_size, key / value size] of the projection's dtype")
        _, num_kv, page_size, key_dim = key_cache.shape
        value_dim = value_cache.shape[3]
        if second[1] != num_kv * key_dim or v_at < 0 or v_at + num_kv * value_dim > proj.shape[1]:
            raise KernelError("projection_norm: the second segment is the keys of all kv heads, the values lie inside the row")
    fn = _fn("latent_prepare", "tvb_projection_norm_rotate_store",
             [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
              c_float, c_float, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
              c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(proj.data_ptr(), proj.stride(0), first[0], first[1], first[2].data_ptr(), int(bool(first[3])),
              second[0], second[1], _ptr(second[2]), int(bool(second[3])), dtype_tag(first[2].dtype),
              _ptr(positions), eps, float(coef), int(every), _ptr(slots), _ptr(key_cache), _ptr(value_cache), num_kv,
              key_dim, value_dim, page_size, v_at, tokens, dtype_tag(proj.dtype), _ptr(inv_freq), rot_dims, halves,
              head_dim, _stream()),
           "projection_norm")


def latent_prepare(proj: torch.Tensor, *, dq_at: int, q_rank: int, q_weight: torch.Tensor | None,
                   dkv_at: int, kv_rank: int, kv_weight: torch.Tensor, rot_dim: int,
                   inv_freq: torch.Tensor | None, magnitude: float, positions: torch.Tensor,
                   slots: torch.Tensor | None, key_cache: torch.Tensor | None, eps: float,
                   pairing: str = "interleaved") -> torch.Tensor | None:
    """From a packed projection [tokens, columns] that holds a query latent (``q_rank`` columns from
    ``dq_at``) and a key/value latent with a part to rotate (``kv_rank + rot_dim`` columns from
    ``dkv_at``): returns RMSnorm(query latent) * q_weight [tokens, q_rank]; writes [RMSnorm(latent) *
    kv_weight | rotated part] to ``key_cache`` [pages, 1, page, kv_rank + rot_dim] at ``slots``.  The
    pair (2i, 2i + 1) (``pairing`` "half_split": (i, i + rot_dim / 2)) turns by position * inv_freq[i]
    (float32), cosine and sine times ``magnitude``."""
    _need_cuda(proj, q_weight, kv_weight, inv_freq, positions, slots, key_cache)
    if pairing not in PAIRINGS:
        raise KernelError(f"latent_prepare: pairing {pairing!r} is not known")
    tokens = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1 or min(dq_at, dkv_at) < 0 or \
            max(dq_at + q_rank, dkv_at + kv_rank + rot_dim) > proj.shape[1]:
        raise KernelError("latent_prepare: the latents do not fit the projection's rows")
    if kv_weight.shape != (kv_rank,) or (q_rank > 0 and (q_weight is None or q_weight.shape != (q_rank,)
                                                        or q_weight.dtype != kv_weight.dtype)):
        raise KernelError("latent_prepare: norm weights of the latents' sizes and of one dtype")
    if rot_dim % 2 or (rot_dim > 0 and (inv_freq is None or inv_freq.dtype != torch.float32
                                        or inv_freq.shape != (rot_dim // 2,) or not inv_freq.is_contiguous())):
        raise KernelError("latent_prepare: inv_freq must be float32 [rot_dim / 2]")
    if positions.dtype != torch.int32 or positions.shape != (tokens,):
        raise KernelError("latent_prepare: positions must be int32 [tokens]")
    if slots is not None and (slots.dtype != torch.int32 or slots.shape != (tokens,) or key_cache is None
                              or key_cache.dim() != 4 or key_cache.shape[1] != 1
                              or key_cache.shape[3] != kv_rank + rot_dim or key_cache.dtype != proj.dtype
                              or not key_cache.is_contiguous()):
        raise KernelError("latent_prepare: slots int32 [tokens]; cache contiguous [pages, 1, page_size, "
                          "kv_rank + rot_dim] of the projection's dtype")
    q_latent = torch.empty((tokens, q_rank), dtype=proj.dtype, device=proj.device) if q_rank > 0 else None
    fn = _fn("latent_prepare", "tvb_latent_prepare",
             [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_longlong, c_int, c_int, c_void_p, c_int,
              c_int, c_void_p, c_float, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_void_p])
    _check(fn(proj.data_ptr(), proj.stride(0), dq_at, q_rank, _ptr(q_weight), _ptr(q_latent), q_rank, dkv_at,
              kv_rank, kv_weight.data_ptr(), dtype_tag(kv_weight.dtype), rot_dim, _ptr(inv_freq), magnitude,
              positions.data_ptr(), _ptr(slots), _ptr(key_cache) if slots is not None else None, eps, tokens,
              dtype_tag(proj.dtype), PAIRINGS[pairing], _stream()), "latent_prepare")
    return q_latent


def _heads_view(t: torch.Tensor, heads: int, size: int, what: str) -> tuple[int, int]:
    if t.dim() != 3 or t.shape[1:] != (heads, size) or t.stride(2) != 1:
        raise KernelError(f"{what} must be [tokens, {heads}, {size}] with contiguous innermost elements")
    return t.stride(0), t.stride(1)


def rotate_heads(src: torch.Tensor, dst: torch.Tensor, inv_freq: torch.Tensor, magnitude: float,
                 positions: torch.Tensor, pairing: str = "interleaved") -> None:
    """dst[t, h, :] = src[t, h, :] with every pair (2i, 2i + 1) (``pairing`` "half_split": (i, i + rot_dim / 2))
    turned by position * inv_freq[i] and cosine and sine multiplied by ``magnitude``; both [tokens, heads,
    rot_dim], any strides."""
    _need_cuda(src, dst, inv_freq, positions)
    if pairing not in PAIRINGS:
        raise KernelError(f"rotate_heads: pairing {pairing!r} is not known")
    tokens, heads, rot_dim = src.shape
    s_strides = _heads_view(src, heads, rot_dim, "rotate_heads: src")
    d_strides = _heads_view(dst, heads, rot_dim, "rotate_heads: dst")
    if dst.shape != src.shape or dst.dtype != src.dtype or rot_dim % 2 or inv_freq.dtype != torch.float32 or \
            inv_freq.shape != (rot_dim // 2,) or positions.dtype != torch.int32 or positions.shape != (tokens,):
        raise KernelError("rotate_heads: equal shapes, float32 inv_freq [rot_dim / 2], int32 positions [tokens]")
    fn = _fn("latent_prepare", "tvb_rotate_heads",
             [c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_longlong, c_int, c_int, c_void_p, c_float,
              c_void_p, c_int, c_int, c_int, c_void_p])
    _check(fn(src.data_ptr(), *s_strides, dst.data_ptr(), *d_strides, heads, rot_dim, inv_freq.data_ptr(),
              magnitude, positions.data_ptr(), tokens, dtype_tag(src.dtype), PAIRINGS[pairing], _stream()),
           "rotate_heads")


HEAD_PRODUCT_MAX_K = 1536        # eight float32 rows of x wait in 48 KB of shared memory
HEAD_PRODUCT_LIBRARY_TOKENS = 64   # bfloat16 tokens from which the products go to the batched library product


def head_product(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, gate: torch.Tensor | None = None) -> None:
    """out[t, h, j] = sum_k x[t, h, k] * w[h, j, k] for x [tokens, heads, k] and out [tokens, heads, n] with
    strides of their own and contiguous w [heads, n, k]; with ``gate`` [tokens, heads * n] the result is
    multiplied by sigmoid(gate) before it is rounded.  float32 sums in an order that k alone fixes."""
    _need_cuda(x, w, out, gate)
    if w.dim() != 3 or not w.is_contiguous():
        raise KernelError("head_product wants contiguous weights [heads, n, k]")
    heads, n, k = w.shape
    tokens = x.shape[0]
    x_strides = _heads_view(x, heads, k, "head_product: x")
    o_strides = _heads_view(out, heads, n, "head_product: out")
    if out.shape[0] != tokens or not (x.dtype == w.dtype == out.dtype) or k > HEAD_PRODUCT_MAX_K:
        raise KernelError(f"head_product: one dtype, equal token counts, k up to {HEAD_PRODUCT_MAX_K}")
    if gate is not None and (gate.shape != (tokens, heads * n) or gate.stride(1) != 1 or gate.dtype != x.dtype):
        raise KernelError("head_product: gate must be [tokens, heads * n] of the same dtype with contiguous rows")
    if x.dtype == torch.bfloat16 and tokens >= HEAD_PRODUCT_LIBRARY_TOKENS:
        # many tokens: one batched library product (a batch a head) on the tensor cores, then the result goes
        # to its place, with the gate on the way
        by_head = torch.bmm(x.transpose(0, 1), w.transpose(1, 2))            # [heads, tokens, n]
        fn = _fn("latent_prepare", "tvb_heads_place",
                 [c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                  c_void_p])
        _check(fn(by_head.data_ptr(), out.data_ptr(), *o_strides, _ptr(gate), 0 if gate is None else gate.stride(0),
                  tokens, heads, n, dtype_tag(x.dtype), _stream()), "heads_place")
        return
    fn = _fn("latent_prepare", "tvb_head_product",
             [c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_longlong, c_void_p, c_longlong,
              c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(x.data_ptr(), *x_strides, w.data_ptr(), out.data_ptr(), *o_strides, _ptr(gate),
              0 if gate is None else gate.stride(0), tokens, heads, n, k, dtype_tag(x.dtype), _stream()),
           "head_product")


# ----------------------------------------------------------- routing of a mixture of experts
EXPERT_ACTIVATIONS = {"relu_squared": 0, "silu": 1}
ROUTE_MAX_EXPERTS = 1024


def route_act(logits: torch.Tensor, up: torch.Tensor, *, experts: int, top: int, ff: int, shared_ff: int,
              activation: str = "relu_squared", out: torch.Tensor | None = None,
              weights_out: torch.Tensor | None = None) -> torch.Tensor:
    """From router logits (float32 [tokens, experts]) and the packed up-projection [tokens, experts * ff
    + shared_ff] to the input of the packed down-projection: act(up) times the expert's weight (the softmax
    over the ``top`` largest logits; 0 for every other expert), the shared expert's columns unweighted."""
    _need_cuda(logits, up, out, weights_out)
    tokens = up.shape[0]
    columns = experts * ff + shared_ff
    if activation not in EXPERT_ACTIVATIONS:
        raise KernelError(f"route_act knows {', '.join(EXPERT_ACTIVATIONS)}, not {activation!r}")
    if logits.dtype != torch.float32 or logits.shape != (tokens, experts) or logits.stride(1) != 1:
        raise KernelError("route_act: router logits are float32 [tokens, experts]")
    if up.dim() != 2 or up.shape[1] != columns or up.stride(1) != 1 or not 0 < experts <= ROUTE_MAX_EXPERTS \
            or top <= 0:
        raise KernelError("route_act: up must be [tokens, experts * ff + shared_ff] with contiguous rows")
    if out is None:
        out = torch.empty((tokens, columns), dtype=up.dtype, device=up.device)
    elif out.shape != (tokens, columns) or out.dtype != up.dtype or out.stride(1) != 1:
        raise KernelError("route_act: out must match up")
    if weights_out is not None and (weights_out.dtype != torch.float32 or weights_out.shape != (tokens, experts)
                                    or not weights_out.is_contiguous()):
        raise KernelError("route_act: weights_out must be contiguous float32 [tokens, experts]")
    fn = _fn("routed_act", "tvb_route_act",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int, c_int,
              c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), up.data_ptr(), up.stride(0), out.data_ptr(), out.stride(0),
              _ptr(weights_out), tokens, experts, top, ff, shared_ff, EXPERT_ACTIVATIONS[activation],
              dtype_tag(up.dtype), _stream()), "route_act")
    return out

def route_gated_act(logits: torch.Tensor, proj: torch.Tensor, *, experts: int, top: int, ff: int, shared_ff: int,
                    limit: float, shared_limit: float, alpha: float, route_scale: float = 1.0,
                    correction: torch.Tensor | None = None, groups: int = 1, keep: int = 1,
                    shared_gated: bool = False, out: torch.Tensor | None = None,
                    weights_out: torch.Tensor | None = None) -> torch.Tensor:
    """Sigmoid routing and gated experts with limits between the packed input and output products.

    ``logits`` float32 [tokens, experts (+ 1 with ``shared_gated``: the shared expert's gate logit)];
    ``proj`` [tokens, 2 * (experts * ff + shared_ff)] holds [gate | up] of every expert, then of the shared
    one.  Scores are sigmoid(logits); the ``top`` experts with the largest score + ``correction`` among
    the ``keep`` best of ``groups`` groups (a group's score: the sum of its two largest) are chosen and
    weighted score / (sum of the chosen scores + 1e-20) * ``route_scale``.  The result [tokens, experts * ff
    + shared_ff] holds min(gate, limit) * sigmoid(alpha * that) * (clamp(up, -limit, limit) + 1) times the
    expert's weight (0 if not chosen); the shared expert's columns use ``shared_limit`` and the weight
    sigmoid(its gate logit), or 1."""
    _need_cuda(logits, proj, correction, out, weights_out)
    tokens = proj.shape[0]
    columns = experts * ff + shared_ff
    if logits.dtype != torch.float32 or logits.shape != (tokens, experts + (1 if shared_gated else 0)) \
            or logits.stride(1) != 1:
        raise KernelError("route_gated_act: router logits are float32 [tokens, experts (+ 1)]")
    if proj.dim() != 2 or proj.shape[1] != 2 * columns or proj.stride(1) != 1 \
            or not 0 < experts <= ROUTE_MAX_EXPERTS or top <= 0:
        raise KernelError("route_gated_act: the projection must be [tokens, 2 * (experts * ff + shared_ff)]")
    if groups <= 0 or experts % groups or not 0 < keep <= groups:
        raise KernelError("route_gated_act: experts form equal groups of which some are kept")
    if correction is not None and (correction.dtype != torch.float32 or correction.shape != (experts,)
                                   or not correction.is_contiguous()):
        raise KernelError("route_gated_act: the correction is contiguous float32 [experts]")
    if out is None:
        out = torch.empty((tokens, columns), dtype=proj.dtype, device=proj.device)
    elif out.shape != (tokens, columns) or out.dtype != proj.dtype or out.stride(1) != 1:
        raise KernelError("route_gated_act: out must be [tokens, experts * ff + shared_ff] of the projection's dtype")
    if weights_out is not None and (weights_out.dtype != torch.float32 or weights_out.shape != (tokens, experts)
                                    or not weights_out.is_contiguous()):
        raise KernelError("route_gated_act: weights_out must be contiguous float32 [tokens, experts]")
    fn = _fn("routed_act", "tvb_route_gated_act",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_int, c_int,
              c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_float, c_float, c_float, c_int, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), _ptr(correction), proj.data_ptr(), proj.stride(0),
              out.data_ptr(), out.stride(0), _ptr(weights_out), tokens, experts, top, groups, keep, route_scale,
              ff, shared_ff, 1 if shared_gated else 0, limit, shared_limit, alpha, dtype_tag(proj.dtype),
              _stream()), "route_gated_act")
    return out


def route_softmax_gated(logits: torch.Tensor, proj: torch.Tensor, *, experts: int, identity: int, top: int, ff: int,
                        correction: torch.Tensor | None = None, renormalise: bool = False,
                        out: torch.Tensor | None = None, weights_out: torch.Tensor | None = None):
    """Softmax routing over experts and pass-through slots, and gated experts, between the packed input and
    output products.

    ``logits`` float32 [tokens, experts + identity]; the scores are their softmax over all slots, the ``top``
    slots with the largest score + ``correction`` (float32 [experts + identity]) are chosen, and a chosen
    slot's weight is its score (``renormalise``: over the sum of the chosen scores).  ``proj`` [tokens, 2 *
    experts * ff] holds [gate | up] of every expert; the result [tokens, experts * ff] holds silu(gate) * up
    times the expert's weight (0 if not chosen).  The last ``identity`` slots have no columns: the sum of their
    weights comes back as float32 [tokens] (None without such slots), and the caller adds that many times the
    experts' input to the down-projection's result.  Returns (inner, identity weights)."""
    _need_cuda(logits, proj, correction, out, weights_out)
    tokens = proj.shape[0]
    slots = experts + identity
    columns = experts * ff
    if logits.dtype != torch.float32 or logits.shape != (tokens, slots) or logits.stride(1) != 1:
        raise KernelError("route_softmax_gated: router logits are float32 [tokens, experts + identity]")
    if proj.dim() != 2 or proj.shape[1] != 2 * columns or proj.stride(1) != 1 or experts <= 0 or identity < 0 \
            or slots > ROUTE_MAX_EXPERTS or top <= 0:
        raise KernelError("route_softmax_gated: the projection must be [tokens, 2 * experts * ff]")
    if correction is not None and (correction.dtype != torch.float32 or correction.shape != (slots,)
                                   or not correction.is_contiguous()):
        raise KernelError("route_softmax_gated: the correction is contiguous float32 [experts + identity]")
    if out is None:
        out = torch.empty((tokens, columns), dtype=proj.dtype, device=proj.device)
    elif out.shape != (tokens, columns) or out.dtype != proj.dtype or out.stride(1) != 1:
        raise KernelError("route_softmax_gated: out must be [tokens, experts * ff] of the projection's dtype")
    if weights_out is not None and (weights_out.dtype != torch.float32 or weights_out.shape != (tokens, slots)
                                    or not weights_out.is_contiguous()):
        raise KernelError("route_softmax_gated: weights_out must be contiguous float32 [tokens, experts + identity]")
    passed = torch.empty((tokens,), dtype=torch.float32, device=proj.device) if identity else None
    fn = _fn("routed_act", "tvb_route_softmax_gated",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_void_p, c_int,
              c_int, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), _ptr(correction), proj.data_ptr(), proj.stride(0),
              out.data_ptr(), out.stride(0), _ptr(weights_out), _ptr(passed), tokens, experts, identity, top,
              1 if renormalise else 0, ff, dtype_tag(proj.dtype), _stream()), "route_softmax_gated")
    return out, passed


# --------------------------------------------------- retention: linear attention with a decay a head
RETENTION_MAX_DIM = 256
RETENTION_ACTS = {None: 0, "silu": 1, "sigmoid": 2}
SM_COUNT = 148                    # a B200's SMs: what the choice of a piece's size fills


_RETENTION_SCAN_ARGS = [c_void_p, c_void_p, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p,
                        c_void_p, c_void_p]
_RETENTION_FINISH_ARGS = [c_void_p, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_float,
                          c_int, c_void_p, c_int, c_void_p]


def retention_lanes(dim: int) -> int:
    """Lanes that share a tile of eight columns of the state: the fewest of 4, 8, 16 and 32 that hold the key
    with at most eight rows a lane."""
    return next((lanes for lanes in (4, 8, 16) if lanes * 8 >= dim), 32)


def retention_segment(tokens: int, rows: int, heads: int, dim: int, vdim: int) -> int:
    """Tokens a piece of the scan.  0 (whole entries) for steps of short entries, and where the entries'
    (head, 32 columns) CTAs, the narrowest there are, already give three SMs in two one.  Else, for
    prompts, the longest of 256, 128 and 64 tokens that gives the SMs four CTAs each: the pieces cost a
    correcting pass, a third of the scan's arithmetic, and fill SMs that whole entries leave idle (measured
    at 2,048 tokens with heads of 128: 16 heads 2.2 times and 32 heads 1.3 times as fast, 64 heads slower)."""
    if 2 * rows * heads * -(-vdim // 32) >= 3 * SM_COUNT or tokens < 4 * max(rows, 1) or tokens < 256:
        return 0
    per_piece = heads * -(-vdim // (128 // retention_lanes(dim) * 8))
    segment = 256
    while segment > 64 and (tokens // segment) * per_piece < 4 * SM_COUNT:
        segment //= 2
    return segment


def retention(proj: torch.Tensor, *, q_at: int, k_at: int, v_at: int, g_at: int | None, heads: int, dim: int,
              vdim: int, decay: torch.Tensor, state: torch.Tensor, row_starts: torch.Tensor,
              state_slots: torch.Tensor, token_row: torch.Tensor, positions: torch.Tensor,
              inv_freq: torch.Tensor | None = None, rot_dims: int = 0, pairing: str = "half_split",
              key_scale: float = 1.0, unit_norm: bool = True, eps: float = 0.0, gate_act: str | None = "silu",
              out: torch.Tensor | None = None, raw_out: torch.Tensor | None = None, lanes: int = 0,
              segment: int | None = None) -> torch.Tensor:
    """Retention between a mixer's packed input projection and its output projection.

    ``proj`` [tokens, columns] holds q heads (``dim`` wide) from column ``q_at``, k heads from ``k_at``,
    v heads (``vdim``) from ``v_at`` and, with ``g_at``, a gate of heads * vdim columns.  Per request
    (``row_starts`` [rows + 1] first flat token of every entry, ``state_slots`` [rows]) and head, token by
    token: S <- decay_h S + k v^T, o = S^T q, from the float32 ``state`` [slots, heads, dim, vdim] of the
    request's slot, which is left as the state after the step's last token.  q and k are turned by
    position * ``inv_freq`` on their first ``rot_dims`` dimensions and k is multiplied by ``key_scale``,
    all in float32.  Every head's o is divided by its root mean square (``unit_norm``, with ``eps``),
    multiplied by act(gate) and rounded to the projection's type: [tokens, heads * vdim].  ``raw_out``
    (float32 [tokens, heads * vdim]) receives o itself.  ``lanes`` (4, 8, 16 or 32, at least an eighth of
    ``dim``; 0: the fewest, or more where SMs would idle) is the number of lanes that share a tile of eight columns of the state.

    ``segment``: 0 walks every entry token by token in one CTA a (head, block of columns); n > 0 cuts the
    entries into pieces of n tokens that run side by side from a state of zero, joins the pieces' states
    along each entry and adds to every token what the state before its piece gives it (S_0 reaches token t
    of a piece as decay^(t + 1) S_0^T q_t).  None chooses: whole entries for steps of few tokens, pieces of
    64 to 256 tokens, enough of them to fill the SMs, for prompts."""
    _need_cuda(proj, decay, state, row_starts, state_slots, token_row, positions, inv_freq, out, raw_out)
    tokens = proj.shape[0]
    rows = state_slots.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("retention: the projection must be [tokens, columns] with contiguous rows")
    ends = [q_at + heads * dim, k_at + heads * dim, v_at + heads * vdim] + ([] if g_at is None else [g_at + heads * vdim])
    if min(q_at, k_at, v_at, 0 if g_at is None else g_at) < 0 or max(ends) > proj.shape[1]:
        raise KernelError("retention: the heads do not fit the projection's rows")
    if not 0 < dim <= RETENTION_MAX_DIM or vdim <= 0:
        raise KernelError(f"retention takes key sizes up to {RETENTION_MAX_DIM}, not {dim}")
    if state.dtype != torch.float32 or state.dim() != 4 or state.shape[1:] != (heads, dim, vdim) \
            or not state.is_contiguous():
        raise KernelError("retention: the state is contiguous float32 [slots, heads, dim, vdim]")
    if decay.dtype != torch.float32 or decay.shape != (heads,) or not decay.is_contiguous():
        raise KernelError("retention: decay is contiguous float32 [heads]")
    for name, t, shape in (("row_starts", row_starts, (rows + 1,)), ("state_slots", state_slots, (rows,)),
                           ("token_row", token_row, (tokens,)), ("positions", positions, (tokens,))):
        if t.dtype != torch.int32 or t.shape != shape or not t.is_contiguous():
            raise KernelError(f"retention: {name} must be contiguous int32 {list(shape)}")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (rot_dims // 2,) or rot_dims % 2
                                 or not 0 < rot_dims <= dim or not inv_freq.is_contiguous()):
        raise KernelError("retention: inv_freq must be float32 [rot_dims / 2] with rot_dims <= dim")
    if pairing not in PAIRINGS or gate_act not in RETENTION_ACTS:
        raise KernelError(f"retention: pairing {pairing!r} or gate activation {gate_act!r} is not known")
    if out is None:
        out = torch.empty((tokens, heads * vdim), dtype=proj.dtype, device=proj.device)
    elif out.shape != (tokens, heads * vdim) or out.dtype != proj.dtype or out.stride(1) != 1:
        raise KernelError("retention: out must be [tokens, heads * vdim] of the projection's dtype")
    if raw_out is None:
        raw_out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=proj.device)
    elif raw_out.shape != (tokens, heads * vdim) or raw_out.dtype != torch.float32 or not raw_out.is_contiguous():
        raise KernelError("retention: raw_out must be contiguous float32 [tokens, heads * vdim]")
    turned = torch.empty((2, tokens, heads * dim), dtype=torch.float32, device=proj.device)
    if segment is None:
        segment = retention_segment(tokens, rows, heads, dim, vdim)
    if segment < 0:
        raise KernelError("retention: a piece has at least one token")
    pieces = tokens // segment + rows if segment else 0
    parts = torch.empty((pieces, heads, dim, vdim), dtype=torch.float32, device=proj.device) if segment else None
    tag = dtype_tag(proj.dtype)
    prepare = _fn("retention", "tvb_retention_prepare",
                  [c_void_p, c_longlong, c_int, c_int, c_int, c_int, c_void_p, c_int, c_int, c_float, c_void_p,
                   c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(prepare(proj.data_ptr(), proj.stride(0), q_at, k_at, heads, dim, _ptr(inv_freq), rot_dims,
                   PAIRINGS[pairing], key_scale, positions.data_ptr(), turned[0].data_ptr(), turned[1].data_ptr(),
                   tokens, tag, _stream()), "retention_prepare")
    scan = _fn_of("retention", "tvb_retention_scan", _RETENTION_SCAN_ARGS)
    _check(scan(turned[0].data_ptr(), turned[1].data_ptr(), proj.data_ptr() + v_at * proj.element_size(),
                proj.stride(0), state.data_ptr(), decay.data_ptr(), row_starts.data_ptr(), state_slots.data_ptr(),
                token_row.data_ptr(), raw_out.data_ptr(), rows, heads, dim, vdim, lanes, _ptr(parts), segment, pieces, tag,
                None, None, None, _stream()), "retention_scan", launches=3 if segment else 1)
    finish = _fn_of("retention", "tvb_retention_finish", _RETENTION_FINISH_ARGS)
    gate_ptr = None if g_at is None else proj.data_ptr() + g_at * proj.element_size()
    _check(finish(raw_out.data_ptr(), gate_ptr, proj.stride(0), out.data_ptr(), out.stride(0), tokens, heads, vdim,
                  1 if unit_norm else 0, eps, RETENTION_ACTS[gate_act if g_at is not None else None], None, tag,
                  _stream()), "retention_finish")
    return out


GATED_QUERY_ACTS = {None: 0, "silu": 1}
GATED_STEP_MAX_PLAIN_COLUMNS = 256     # STEP_THREADS of retention.cu: a column a thread where float4s do not fit


def gated_recurrence(proj: torch.Tensor, *, q_at: int, g_at: int, v_at: int, heads: int, dim: int, vdim: int,
                     state: torch.Tensor, row_starts: torch.Tensor, state_slots: torch.Tensor,
                     token_row: torch.Tensor, bias: torch.Tensor | None = None, lower: torch.Tensor | None = None,
                     query_act: str | None = "silu", k_at: int | None = None, unit_norm: bool = True,
                     norm_weight: torch.Tensor | None = None, eps: float = 0.0, out: torch.Tensor | None = None,
                     raw_out: torch.Tensor | None = None, lanes: int = 0, segment: int | None = None) -> torch.Tensor:
    """A linear recurrence whose decay is a gate a token and key channel, between a mixer's packed input
    projection and its output projection.

    ``proj`` [tokens, columns] holds q heads (``dim`` wide) from column ``q_at``, the gates' pre-activations
    (heads of ``dim``) from ``g_at`` and v heads (``vdim``) from ``v_at``.  q = act(q) (``query_act``: None or
    "silu"); g = lower + (1 - lower) * sigmoid(pre-activation + bias) with float32 ``bias`` and ``lower``
    [heads * dim] (either may be None: 0).  Per request and head, token by token, S <- diag(g) S + k v^T and
    o = S^T q from the float32 ``state`` [slots, heads, dim, vdim] of the request's slot, which is left as the
    state after the step's last token.  The keys are what the gate lets go, k = 1 - g, unless ``k_at`` names
    columns with keys of their own.  Every head's o is divided by its root mean square (``unit_norm``, with
    ``eps``) and multiplied by ``norm_weight`` (float32 [vdim], one for all heads), then rounded to the
    projection's type: [tokens, heads * vdim].  Gates, products, state and sums are float32.

    ``segment`` as in :func:`retention`: 0 walks whole entries, n > 0 cuts them into pieces of n tokens that
    run side by side (a piece's decay is the product of its gates, channel by channel), None chooses.

    A step in which every entry is one token (as many tokens as entries) runs as one launch, a CTA a (request,
    head), unless ``raw_out``, ``lanes`` or a ``segment`` ask for the scan."""
    _need_cuda(proj, state, row_starts, state_slots, token_row, bias, lower, norm_weight, out, raw_out)
    tokens = proj.shape[0]
    rows = state_slots.shape[0]
    per = heads * dim
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("gated_recurrence: the projection must be [tokens, columns] with contiguous rows")
    ends = [q_at + per, g_at + per, v_at + heads * vdim] + ([] if k_at is None else [k_at + per])
    if min(q_at, g_at, v_at, 0 if k_at is None else k_at) < 0 or max(ends) > proj.shape[1]:
        raise KernelError("gated_recurrence: the heads do not fit the projection's rows")
    if not 0 < dim <= RETENTION_MAX_DIM or vdim <= 0:
        raise KernelError(f"gated_recurrence takes key sizes up to {RETENTION_MAX_DIM}, not {dim}")
    if state.dtype != torch.float32 or state.dim() != 4 or state.shape[1:] != (heads, dim, vdim) \
            or not state.is_contiguous():
        raise KernelError("gated_recurrence: the state is contiguous float32 [slots, heads, dim, vdim]")
    for name, t, shape in (("row_starts", row_starts, (rows + 1,)), ("state_slots", state_slots, (rows,)),
                           ("token_row", token_row, (tokens,))):
        if t.dtype != torch.int32 or t.shape != shape or not t.is_contiguous():
            raise KernelError(f"gated_recurrence: {name} must be contiguous int32 {list(shape)}")
    for name, t, shape in (("bias", bias, (per,)), ("lower", lower, (per,)), ("norm_weight", norm_weight, (vdim,))):
        if t is not None and (t.dtype != torch.float32 or t.shape != shape or not t.is_contiguous()):
            raise KernelError(f"gated_recurrence: {name} must be contiguous float32 {list(shape)}")
    if query_act not in GATED_QUERY_ACTS:
        raise KernelError(f"gated_recurrence: the queries' activation is None or 'silu', not {query_act!r}")
    if out is None:
        out = torch.empty((tokens, heads * vdim), dtype=proj.dtype, device=proj.device)
    elif out.shape != (tokens, heads * vdim) or out.dtype != proj.dtype or out.stride(1) != 1:
        raise KernelError("gated_recurrence: out must be [tokens, heads * vdim] of the projection's dtype")
    if raw_out is not None and (raw_out.shape != (tokens, heads * vdim) or raw_out.dtype != torch.float32
                                or not raw_out.is_contiguous()):
        raise KernelError("gated_recurrence: raw_out must be contiguous float32 [tokens, heads * vdim]")
    if segment is None:
        segment = retention_segment(tokens, rows, heads, dim, vdim)
    if segment < 0:
        raise KernelError("gated_recurrence: a piece has at least one token")
    from .build import variant
    library = variant("retention", RET_GATED=1 if k_at is None else 2)
    tag = dtype_tag(proj.dtype)
    if tokens == rows and k_at is None and raw_out is None and not segment and lanes == 0 and (
            vdim % 4 == 0 or vdim <= GATED_STEP_MAX_PLAIN_COLUMNS) and vdim <= 4 * GATED_STEP_MAX_PLAIN_COLUMNS:
        # every entry is one token (a decode step): preparation, the state's one move and the norm in one launch
        step = _fn_of(library, "tvb_gated_step",
                      [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_int, c_float, c_void_p, c_longlong, c_int, c_int, c_int, c_int,
                       c_int, c_void_p])
        _check(step(proj.data_ptr(), proj.stride(0), q_at, g_at, v_at, _ptr(bias), _ptr(lower),
                    GATED_QUERY_ACTS[query_act], state.data_ptr(), row_starts.data_ptr(), state_slots.data_ptr(),
                    token_row.data_ptr(), _ptr(norm_weight), 1 if unit_norm else 0, eps, out.data_ptr(), out.stride(0),
                    rows, heads, dim, vdim, tag, _stream()), "gated_step")
        return out
    if raw_out is None:
        raw_out = torch.empty((tokens, heads * vdim), dtype=torch.float32, device=proj.device)
    pieces = tokens // segment + rows if segment else 0
    # float32 rows: q, gates, (keys), and for pieces the queries times the running products of the gates
    work = torch.empty((4, tokens, per), dtype=torch.float32, device=proj.device)
    parts = torch.empty((pieces, heads, dim, vdim), dtype=torch.float32, device=proj.device) if segment else None
    piece_gates = torch.empty((pieces, heads, dim), dtype=torch.float32, device=proj.device) if segment else None
    prepare = _fn_of(library, "tvb_gated_prepare",
                     [c_void_p, c_longlong, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
                      c_int, c_void_p])
    _check(prepare(proj.data_ptr(), proj.stride(0), q_at, g_at, per, _ptr(bias), _ptr(lower),
                   GATED_QUERY_ACTS[query_act], work[0].data_ptr(), work[1].data_ptr(), tokens, tag, _stream()),
           "gated_prepare")
    keys = None
    if k_at is not None:
        keys = work[2]
        keys.copy_(proj[:, k_at:k_at + per])
    scan = _fn_of(library, "tvb_retention_scan", _RETENTION_SCAN_ARGS)
    _check(scan(work[0].data_ptr(), _ptr(keys), proj.data_ptr() + v_at * proj.element_size(), proj.stride(0),
                state.data_ptr(), None, row_starts.data_ptr(), state_slots.data_ptr(), token_row.data_ptr(),
                raw_out.data_ptr(), rows, heads, dim, vdim, lanes, _ptr(parts), segment, pieces, tag,
                work[1].data_ptr(), work[3].data_ptr() if segment else None, _ptr(piece_gates), _stream()),
           "gated_recurrence_scan", launches=4 if segment else 1)
    finish = _fn_of(library, "tvb_retention_finish", _RETENTION_FINISH_ARGS)
    _check(finish(raw_out.data_ptr(), None, proj.stride(0), out.data_ptr(), out.stride(0), tokens, heads, vdim,
                  1 if unit_norm else 0, eps, 0, _ptr(norm_weight), tag, _stream()), "gated_recurrence_finish")
    return out


# ------------------- q/k norm, rotation, value blend and cache write with every size a parameter
NORM_MODES = {None: 0, "unit": 1, "weight": 2}
PAIRINGS = {"interleaved": 0, "half_split": 1}


def qkv_prepare(proj: torch.Tensor, *, q_at: int, k_at: int, v_at: int, num_q: int, num_kv: int,
                key_dim: int, value_dim: int, positions: torch.Tensor, norm: str | None = None,
                q_weight: torch.Tensor | None = None, k_weight: torch.Tensor | None = None, eps: float = 0.0,
                inv_freq: torch.Tensor | None = None, rot_dims: int = 0, pairing: str = "interleaved",
                slots: torch.Tensor | None, key_cache: torch.Tensor | None, value_cache: torch.Tensor | None,
                v_first: torch.Tensor | None = None, blend: torch.Tensor | None = None,
                q_bias: torch.Tensor | None = None, k_bias: torch.Tensor | None = None,
                v_bias: torch.Tensor | None = None) -> None:
    """In place on a packed projection [tokens, columns] that holds the q heads from column
    ``q_at``, the k heads from ``k_at`` and the v heads from ``v_at``: q and k heads are normalised
    over the head (``norm`` None, "unit" or "weight") and rotated (``inv_freq`` float32
    [rot_dims / 2]; the angle is position * inv_freq in float32), q where it stands, k into
    ``key_cache`` [pages, num_kv, page, key_dim] at ``slots``; v heads go to ``value_cache``
    [pages, num_kv, page, value_dim], blended as (1 - blend) v + blend v_first when ``v_first``
    [tokens, num_kv * value_dim] (rows may be strided) and the one-element ``blend`` are given.
    ``q_bias`` [num_q * key_dim], ``k_bias`` [num_kv * key_dim], ``v_bias`` [num_kv * value_dim] (float32):
    added to the projection's columns before anything else.  ``v_at`` may equal ``k_at``: the values are
    then the keys as projected (k is not changed where it stands)."""
    _need_cuda(proj, positions, q_weight, k_weight, inv_freq, slots, key_cache, value_cache, v_first, blend,
               q_bias, k_bias, v_bias)
    for name, t, size in (("q_bias", q_bias, num_q * key_dim), ("k_bias", k_bias, num_kv * key_dim),
                          ("v_bias", v_bias, num_kv * value_dim)):
        if t is not None and (t.dtype != torch.float32 or t.shape != (size,) or not t.is_contiguous()):
            raise KernelError(f"qkv_prepare: {name} must be contiguous float32 [{size}]")
    if v_bias is not None and v_first is not None:
        raise KernelError("qkv_prepare: blended values take no bias")
    tokens = proj.shape[0]
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelError("qkv_prepare: the projection must be [tokens, columns] with contiguous rows")
    if min(q_at, k_at, v_at) < 0 or max(q_at + num_q * key_dim, k_at + num_kv * key_dim,
                                        v_at + num_kv * value_dim) > proj.shape[1]:
        raise KernelError("qkv_prepare: the heads do not fit the projection's rows")
    if key_dim > 256 or value_dim > 256:
        raise KernelError(f"qkv_prepare takes key and value sizes up to 256, not {key_dim} / {value_dim}")
    if positions.dtype != torch.int32 or positions.shape != (tokens,):
        raise KernelError("qkv_prepare: positions must be int32 [tokens]")
    if norm not in NORM_MODES or pairing not in PAIRINGS:
        raise KernelError(f"qkv_prepare: norm {norm!r} or pairing {pairing!r} is not known")
    weight_tag = dtype_tag(proj.dtype)
    if norm == "weight":
        if q_weight is None or k_weight is None or q_weight.shape != (key_dim,) or k_weight.shape != (key_dim,) \
                or q_weight.dtype != k_weight.dtype:
            raise KernelError("qkv_prepare: norm weights must be [key_dim] of one dtype")
        weight_tag = dtype_tag(q_weight.dtype)
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.shape != (rot_dims // 2,)
                                 or rot_dims % 2 or not 0 < rot_dims <= key_dim or not inv_freq.is_contiguous()):
        raise KernelError("qkv_prepare: inv_freq must be float32 [rot_dims / 2] with rot_dims <= key_dim")
    if slots is not None:
        if (slots.dtype != torch.int32 or slots.shape != (tokens,) or key_cache is None or value_cache is None
                or key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, key_dim)
                or value_cache.shape != key_cache.shape[:3] + (value_dim,) or key_cache.dtype != proj.dtype
                or value_cache.dtype != proj.dtype or not key_cache.is_contiguous()
                or not value_cache.is_contiguous()):
            raise KernelError("qkv_prepare: slots int32 [tokens]; caches contiguous [pages, num_kv, page_size, "
                              "key_dim / value_dim] of the projection's dtype")
    if v_first is not None:
        if (blend is None or blend.numel() != 1 or blend.dtype != proj.dtype or v_first.dtype != proj.dtype
                or v_first.shape != (tokens, num_kv * value_dim) or v_first.stride(1) != 1):
            raise KernelError("qkv_prepare: v_first [tokens, num_kv * value_dim] and a one-element blend, both "
                              "of the projection's dtype")
    fn = _fn("qkv_prepare", "tvb_qkv_prepare_biased",
             [c_void_p, c_longlong] + [c_int] * 8 + [c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int,
                                                    c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                                    c_longlong, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                    c_void_p, c_void_p])
    _check(fn(proj.data_ptr(), proj.stride(0), q_at, k_at, v_at, num_q, num_kv, key_dim, value_dim,
              NORM_MODES[norm], _ptr(q_weight), _ptr(k_weight), weight_tag, eps, _ptr(inv_freq), rot_dims,
              PAIRINGS[pairing], positions.data_ptr(), _ptr(slots), _ptr(key_cache), _ptr(value_cache),
              key_cache.shape[2] if slots is not None else 0, _ptr(v_first),
              0 if v_first is None else v_first.stride(0), _ptr(blend), tokens, dtype_tag(proj.dtype),
              _ptr(q_bias), _ptr(k_bias), _ptr(v_bias), _stream()), "qkv_prepare")



# ----------------- windowed attention on the tensor cores, compiled per (key size, value size)
TILES_CHUNK_KEYS = 128


def _tiles_library(key_dim: int, value_dim: int, value_in_key: bool = False) -> str:
    from .build import variant
    if value_in_key:
        return variant("attention_tiles", TILES_KEY_DIM=key_dim, TILES_VALUE_DIM=value_dim, TILES_VALUE_IN_KEY=1)
    return variant("attention_tiles", TILES_KEY_DIM=key_dim, TILES_VALUE_DIM=value_dim)


# largest key size with values inside the key rows: the value tile is the key tile, so shared memory holds one
TILES_MAX_DIM, TILES_MAX_DIM_VALUE_IN_KEY = 256, 320


def attention_tiles_supports(key_dim: int, value_dim: int, num_q: int, num_kv: int, *,
                             value_in_key: bool = False) -> bool:
    """Key and value sizes that are multiples of 16 (up to 256; keys up to 320 where the values lie inside
    the key rows), whole groups of up to 64 q heads."""
    key_limit = TILES_MAX_DIM_VALUE_IN_KEY if value_in_key else TILES_MAX_DIM
    return (key_dim % 16 == 0 and value_dim % 16 == 0 and 0 < key_dim <= key_limit and 0 < value_dim <= TILES_MAX_DIM
            and (not value_in_key or value_dim <= key_dim)
            and num_kv > 0 and num_q % num_kv == 0 and num_q // num_kv <= PREFILL_TILE_TOKENS)


def _tiles_window_chunks(window: int | None, keep_first: int, max_context: int) -> int:
    every = max(1, -(-max_context // TILES_CHUNK_KEYS))
    if not window:
        return every
    return min((window + TILES_CHUNK_KEYS - 2) // TILES_CHUNK_KEYS + 1, every) + -(-keep_first // TILES_CHUNK_KEYS)


def attention_tiles_singles_floats(tokens: int, num_q: int, value_dim: int, window: int | None,
                                   keep_first: int, max_context: int) -> int:
    """float32 scratch :func:`attention_tiles_singles` needs for ``tokens`` tokens."""
    return tokens * num_q * _tiles_window_chunks(window, keep_first if window else 0, max_context) * (value_dim + 2)


def _tiles_common(name, q, key_cache, value_cache, out, gate, num_q, num_kv, key_dim, value_dim, tokens,
                  gate_per_head=False, slopes=None, sinks=None):
    """Checks of both tile kernels; returns whether the values lie inside the key rows (no value cache)."""
    value_in_key = value_cache is None
    if q.dtype != torch.bfloat16 or key_cache.dtype != torch.bfloat16 or \
            (value_cache is not None and value_cache.dtype != torch.bfloat16):
        raise KernelError(f"{name} is a bfloat16 kernel")
    if not attention_tiles_supports(key_dim, value_dim, num_q, num_kv, value_in_key=value_in_key):
        raise KernelError(f"{name} does not take key size {key_dim}, value size {value_dim}, {num_q}/{num_kv} heads")
    if key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, key_dim) or \
            not key_cache.is_contiguous() or (value_cache is not None and (
                value_cache.shape != key_cache.shape[:3] + (value_dim,) or not value_cache.is_contiguous())):
        raise KernelError(f"{name}: caches must be contiguous [pages, num_kv, page_size, key / value size]")
    if q.dim() != 2 or q.stride(1) != 1 or q.stride(0) % 8 or q.data_ptr() % 16 or q.shape[1] < num_q * key_dim:
        raise KernelError(f"{name}: q must be [tokens, >= num_q * key_dim] with 16-byte aligned rows")
    if out is None or out.shape != (tokens, num_q * value_dim) or out.dtype != torch.bfloat16 or out.stride(1) != 1 \
            or out.stride(0) % 2 or out.data_ptr() % 4:
        raise KernelError(f"{name}: out must be bfloat16 [tokens, num_q * value_dim] with rows of an even stride")
    if gate is not None and gate_per_head:
        if gate.shape != (tokens, num_q) or gate.dtype != torch.bfloat16 or gate.stride(1) != 1:
            raise KernelError(f"{name}: a gate of one number a head is bfloat16 [tokens, num_q]")
    elif gate is not None and (gate.shape != (tokens, num_q * value_dim) or gate.dtype != torch.bfloat16
                               or gate.stride(1) != 1 or gate.stride(0) % 2 or gate.data_ptr() % 4):
        raise KernelError(f"{name}: gate must be bfloat16 [tokens, num_q * value_dim] with rows of an even stride")
    for label, t in (("slopes", slopes), ("sinks", sinks)):
        if t is not None and (t.dtype != torch.float32 or t.shape != (num_q,) or not t.is_contiguous()):
            raise KernelError(f"{name}: {label} must be contiguous float32 [num_q]")
    return value_in_key


def _tiles_table(who: str, bias_table, segment, window, num_q: int) -> None:
    if bias_table is not None and (bias_table.dtype != torch.float32 or bias_table.dim() != 2
                                   or bias_table.shape[1] != num_q or bias_table.shape[0] < 1
                                   or not bias_table.is_contiguous()):
        raise KernelError(f"{who}: the bias table must be contiguous float32 [distances, num_q]")
    if segment is not None and (segment <= 0 or window):
        raise KernelError(f"{who}: a segment holds at least one position and comes without a window")


def attention_tiles(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor | None,
                    block_tables: torch.Tensor, positions: torch.Tensor, tile_row: torch.Tensor,
                    tile_first: torch.Tensor, tile_count: torch.Tensor, *, num_q: int, num_kv: int,
                    key_dim: int, value_dim: int, window: int | None, keep_first: int, scale: float,
                    out: torch.Tensor, gate: torch.Tensor | None = None, gate_per_head: bool = False,
                    slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                    bias_table: torch.Tensor | None = None, segment: int | None = None) -> torch.Tensor:
    """Windowed paged attention on the tensor cores for tiles of up to 64 consecutive query tokens of
    one request (bfloat16; float32 scores, weights and sums).  ``q`` [tokens, >= num_q * key_dim]
    (rows may be strided) holds prepared queries; tile i holds ``tile_count[i]`` tokens from flat
    index ``tile_first[i]`` on of request row ``tile_row[i]``.  With a window the first
    ``keep_first`` keys stay visible.  ``gate``: the output is multiplied by sigmoid(gate), one number a
    value or (``gate_per_head``, [tokens, num_q]) one a head.  ``slopes`` (float32 [num_q]): slope *
    (position - j) is taken off the score of key j; ``sinks`` (float32 [num_q]): exp(sink) joins the
    denominator once.  ``bias_table`` (float32 [rows, num_q]): table[min(position - j, rows - 1), head] is
    added to the score of key j; ``segment`` (not with a window): the query at position p sees only the keys
    from p - p % segment on.  ``value_cache=None``: the values are the first ``value_dim`` elements of the key
    rows."""
    _need_cuda(q, key_cache, value_cache, block_tables, positions, tile_row, tile_first, tile_count, out, gate,
               slopes, sinks, bias_table)
    _tiles_table("attention_tiles", bias_table, segment, window, num_q)
    tokens, tiles = positions.shape[0], tile_row.shape[0]
    value_in_key = _tiles_common("attention_tiles", q, key_cache, value_cache, out, gate, num_q, num_kv, key_dim,
                                 value_dim, tokens, gate_per_head, slopes, sinks)
    for t in (block_tables, positions, tile_row, tile_first, tile_count):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_tiles: index tensors must be contiguous int32")
    library = _tiles_library(key_dim, value_dim, value_in_key)
    if _fn_of(library, "tvb_attention_tiles_tile_tokens", [])() != PREFILL_TILE_TOKENS:
        raise KernelError("attention_tiles: the library's tile size is not the one steps are cut for")
    fn = _fn_of(library, "tvb_attention_tiles_table",
                [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                 c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p] + [c_int] * 10
                + [c_float, c_void_p])
    _check(fn(q.data_ptr(), q.stride(0), key_cache.data_ptr(), _ptr(value_cache), block_tables.data_ptr(),
              block_tables.shape[1], positions.data_ptr(), tile_row.data_ptr(), tile_first.data_ptr(),
              tile_count.data_ptr(), out.data_ptr(), out.stride(0), _ptr(gate), 0 if gate is None else gate.stride(0),
              1 if gate_per_head else 0, _ptr(slopes), _ptr(sinks), _ptr(bias_table),
              0 if bias_table is None else bias_table.shape[0], segment or 0, tiles, num_q, num_kv, key_dim, value_dim, key_cache.shape[2], window or 0, keep_first if window else 0,
              scale, _stream()), "attention_tiles")
    return out


def attention_tiles_singles(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor | None,
                            block_tables: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor, *,
                            num_q: int, num_kv: int, key_dim: int, value_dim: int, window: int | None,
                            keep_first: int, scale: float, max_context: int, scratch: torch.Tensor,
                            out: torch.Tensor, gate: torch.Tensor | None = None, gate_per_head: bool = False,
                            slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None,
                            bias_table: torch.Tensor | None = None, segment: int | None = None) -> torch.Tensor:
    """The same attention for single tokens whose keys and values are in the cache already (decoded
    tokens): a CTA serves the q heads of one kv head over one chunk of 128 keys, a second launch
    merges a row's chunks.  Token i is of request row ``token_row[i]`` (-1: padding, zeros come out)
    at ``positions[i]`` < ``max_context``; ``scratch``: float32, :func:`attention_tiles_singles_floats`."""
    _need_cuda(q, key_cache, value_cache, block_tables, positions, token_row, out, gate, scratch, slopes, sinks,
               bias_table)
    _tiles_table("attention_tiles_singles", bias_table, segment, window, num_q)
    tokens = positions.shape[0]
    value_in_key = _tiles_common("attention_tiles_singles", q, key_cache, value_cache, out, gate, num_q, num_kv,
                                 key_dim, value_dim, tokens, gate_per_head, slopes, sinks)
    for t in (block_tables, positions, token_row):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_tiles_singles: index tensors must be contiguous int32")
    need = attention_tiles_singles_floats(tokens, num_q, value_dim, segment or window, keep_first, max_context)
    if scratch.dtype != torch.float32 or scratch.numel() < need:
        raise KernelError(f"attention_tiles_singles needs {need} float32 of scratch")
    fn = _fn_of(_tiles_library(key_dim, value_dim, value_in_key), "tvb_attention_tiles_singles_table",
                [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_longlong,
                 c_void_p, c_longlong, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p] + [c_int] * 8
                + [c_float, c_int, c_void_p])
    _check(fn(q.data_ptr(), q.stride(0), key_cache.data_ptr(), _ptr(value_cache), block_tables.data_ptr(),
              block_tables.shape[1], positions.data_ptr(), token_row.data_ptr(), out.data_ptr(), out.stride(0),
              _ptr(gate), 0 if gate is None else gate.stride(0), 1 if gate_per_head else 0, _ptr(slopes), _ptr(sinks),
              _ptr(bias_table), 0 if bias_table is None else bias_table.shape[0], segment or 0,
              scratch.data_ptr(), tokens, num_q, num_kv, key_dim,
              value_dim, key_cache.shape[2], window or 0, keep_first if window else 0, scale, max_context,
              _stream()), "attention_tiles_singles", 2)
    return out


# ----------------------------------------------------------------------- GEMM
def gemm_nt_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor:
    """a [m, k] . w [n, k]^T on the float32 cores, ascending k."""
    _need_cuda(a, w)
    if a.dim() != 2 or w.dim() != 2 or a.shape[1] != w.shape[1] or a.dtype != w.dtype:
        raise KernelError("gemm_nt_simt wants a [m, k] and w [n, k] of one dtype")
    if a.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_nt_simt wants rows that are contiguous")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype or a.dtype, device=a.device)
    fn = _fn("gemm_simt", "tvb_gemm_nt_simt",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_int, c_void_p])
    _check(fn(a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, dtype_tag(a.dtype), dtype_tag(out.dtype), _stream()), "gemm_nt_simt")
    return out


# ------------------------------------------------------------------- sampling
def sample_rows(logits: torch.Tensor, packed: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of logits [rows, vocab].  ``packed`` is int32 [7, capacity >= rows],
    field-major: temperature and top_p as float32 bits, top_k, low and high word of the seed,
    low and high word of the draw counter; row r reads column r."""
    _need_cuda(logits, packed)
    rows, vocab = logits.shape
    if logits.stride(1) != 1:
        raise KernelError("sample_rows wants rows that are contiguous")
    if packed.dtype != torch.int32 or packed.dim() != 2 or packed.shape[0] != 7 or \
            packed.shape[1] < rows or not packed.is_contiguous():
        raise KernelError("sample_rows: packed must be contiguous int32 [7, capacity >= rows]")
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    fn = _fn("sampling", "tvb_sample_rows",
             [c_void_p, c_longlong, c_int, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
    _check(fn(logits.data_ptr(), logits.stride(0), rows, vocab, packed.data_ptr(), packed.shape[1],
              out.data_ptr(), dtype_tag(logits.dtype), _pdl("sample"), _stream()), "sample_rows")
    return out


# ------------------------------------------------- tiled attention (bfloat16)
DECODE_MAX_PIECES = 8


def attention_decode_supports(head_dim: int, num_q: int, num_kv: int, splits: int) -> bool:
    """Head sizes 64, 128 and 256, whole groups of q heads, 1 to 8 pieces (answered here, so that
    asking compiles nothing; the libraries check the same)."""
    return (head_dim in DECODE_HEAD_DIMS and num_q > 0 and num_kv > 0 and num_q % num_kv == 0
            and 1 <= splits <= DECODE_MAX_PIECES)


def attention_decode(qkv: torch.Tensor, *, num_q: int, num_kv: int, head_dim: int,
                     positions: torch.Tensor, token_row: torch.Tensor, slots: torch.Tensor | None,
                     q_weight: torch.Tensor | None, k_weight: torch.Tensor | None, eps: float,
                     cos: torch.Tensor | None, sin: torch.Tensor | None, key_cache: torch.Tensor,
                     value_cache: torch.Tensor, block_tables: torch.Tensor, window: int | None,
                     scale: float, splits: int, max_context: int,
                     out: torch.Tensor | None = None, new_in_cache: bool = False,
                     far_groups: int = 1, far_from: int = 0,
                     library_of: torch.dtype | None = None) -> torch.Tensor:
    """One new token per request, from the raw packed projection to the attention output:
    q/k norm and rotation, cache write (unless ``slots`` is None) and attention in one launch.
    ``new_in_cache``: the new tokens' keys and values are in the cache already and q comes
    prepared (no norm weights, no tables, no slots): only the attention is left to do.
    Request i is row ``token_row[i]`` of ``block_tables`` (-1: padding) and stands at
    ``positions[i]``.  Every request's keys are cut into ``splits`` pieces, one per CTA of a cluster;
    ``max_context`` bounds ``positions + 1``."""
    _need_cuda(qkv, positions, token_row, slots, q_weight, k_weight, cos, sin, key_cache, value_cache,
               block_tables)
    requests = qkv.shape[0]
    if qkv.dtype != torch.bfloat16 or not qkv.is_contiguous() or \
            qkv.shape[1] != (num_q + 2 * num_kv) * head_dim:
        raise KernelError("attention_decode wants contiguous bfloat16 [requests, (q + 2 kv) * head_dim]")
    if not attention_decode_supports(head_dim, num_q, num_kv, splits):
        raise KernelError(f"attention_decode does not take head_dim {head_dim}, {num_q}/{num_kv} heads, "
                          f"{splits} splits")
    if key_cache.dtype != torch.bfloat16 or key_cache.dim() != 4 or \
            (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            value_cache.shape != key_cache.shape or not key_cache.is_contiguous():
        raise KernelError("attention_decode: caches must be contiguous bfloat16 "
                          "[pages, num_kv, page_size, head_dim]")
    for t in (positions, token_row, block_tables) + ((slots,) if slots is not None else ()):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_decode: index tensors must be contiguous int32")
    if new_in_cache and not (slots is None and q_weight is None and k_weight is None and cos is None and sin is None):
        raise KernelError("attention_decode: with new_in_cache nothing is normalised, rotated or stored")
    # without norm weights either library of the head size does: ``library_of`` names the type of
    # the one the caller uses elsewhere, so that no second one is compiled
    weight_tag = BF16 if library_of is None else dtype_tag(library_of)
    if q_weight is not None:
        if k_weight is None or q_weight.dtype != k_weight.dtype or q_weight.shape != (head_dim,):
            raise KernelError("attention_decode: norm weights come together, [head_dim], one dtype")
        weight_tag = dtype_tag(q_weight.dtype)
    table_positions = cos.shape[0] if cos is not None else 0
    if cos is not None and (cos.dtype != torch.float32 or cos.shape[1] != head_dim // 2):
        raise KernelError("attention_decode: tables must be float32 [positions, head_dim / 2]")
    if out is None:
        out = torch.empty((requests, num_q * head_dim), dtype=qkv.dtype, device=qkv.device)
    pdl = _pdl("attention")
    if not pdl and _pdl("attention_few") and requests <= PDL_ATTENTION_ROWS:
        # only where the launch runs as CTAs of eight warps, all on the GPU at once
        pdl = int(attention_decode_fits_wide(
            requests * far_groups, num_q=num_q, num_kv=num_kv, head_dim=head_dim, page_size=key_cache.shape[2],
            splits=splits, max_context=max_context, weight_dtype=BF16_OR_F32[weight_tag]))
    if far_groups > 1:
        # a request of far_from keys or more is cut over far_groups clusters per kv head, which
        # leave their pieces in global memory (head size 128; all clusters on the GPU at once)
        pieces, arrived = _far_scratch_of(qkv.device, requests, num_q, num_kv, head_dim, far_groups, weight_tag)
        fn = _fn_of(_decode_library(head_dim, weight_tag), "tvb_attention_decode_far",
                 [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                  c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
                  c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p])
        _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), eps, _ptr(cos), _ptr(sin), table_positions,
                  positions.data_ptr(), token_row.data_ptr(), _ptr(slots), key_cache.data_ptr(),
                  value_cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
                  key_cache.shape[2], out.data_ptr(), requests, num_q, num_kv, head_dim, window or 0, scale,
                  splits, 2 if new_in_cache else (1 if slots is not None else 0), max_context, weight_tag,
                  pdl, far_groups, max(1, far_from), pieces.data_ptr(), arrived.data_ptr(),
                  _stream()),
               "attention_decode (far)")
        return out
    fn = _fn_of(_decode_library(head_dim, weight_tag), "tvb_attention_decode",
             [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_int, c_int,
              c_int, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p])
    _check(fn(qkv.data_ptr(), _ptr(q_weight), _ptr(k_weight), eps, _ptr(cos), _ptr(sin), table_positions,
              positions.data_ptr(), token_row.data_ptr(), _ptr(slots), key_cache.data_ptr(),
              value_cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
              key_cache.shape[2], out.data_ptr(), requests, num_q, num_kv, head_dim, window or 0, scale,
              splits, 2 if new_in_cache else (1 if slots is not None else 0), max_context, weight_tag,
              pdl,
              _stream()),
           "attention_decode")
    return out


_fits_wide: dict[tuple, bool] = {}
_far_scratch: dict[int, list] = {}


def _far_scratch_of(device: torch.device, requests: int, num_q: int, num_kv: int, head_dim: int,
                    groups: int, weight_tag: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Pieces and counters of the decode attention that cuts a request over several clusters, per
    device; they grow with the largest launch and the earlier ones are kept, since CUDA graphs keep
    their addresses.  Launches that use them must follow one another (those of one stream do)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    floats = _fn_of(_decode_library(head_dim, weight_tag), "tvb_attention_decode_far_floats",
                    [c_int, c_int, c_int, c_int, c_int], c_longlong)(requests, num_q, num_kv, head_dim, groups)
    if floats <= 0:
        raise KernelError("attention_decode (far): the kernel does not take these heads")
    held = _far_scratch.setdefault(index, [])
    if not held or held[-1][0].numel() < floats or held[-1][1].numel() < requests * num_q:
        held.append((torch.empty(floats, dtype=torch.float32, device=device),
                     torch.zeros(max(requests * num_q, 1024), dtype=torch.int32, device=device)))
    return held[-1]


def attention_decode_fits_wide(rows: int, *, num_q: int, num_kv: int, head_dim: int, page_size: int,
                               splits: int, max_context: int, weight_dtype: torch.dtype | None = None) -> bool:
    """Whether ``rows`` rows cut into ``splits`` pieces run in the fused decode kernel's form for
    small grids (CTAs of eight warps, one an SM) with all their clusters on the GPU at once.  Asks
    the runtime how many clusters of that shape fit; launches nothing.  Remembered per shape."""
    tag = BF16 if weight_dtype is None else dtype_tag(weight_dtype)
    key = (rows, num_q, num_kv, head_dim, page_size, splits, max_context, tag)
    known = _fits_wide.get(key)
    if known is None:
        if head_dim not in DECODE_HEAD_DIMS:
            _fits_wide[key] = False
            return False
        fn = _fn_of(_decode_library(head_dim, tag), "tvb_attention_decode_fits_wide",
                    [c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int])
        known = _fits_wide[key] = bool(fn(rows, num_q, num_kv, head_dim, page_size, splits, max_context, tag))
    return known


def attention_prefill_supports(head_dim: int, num_q: int, num_kv: int) -> bool:
    fn = _fn("attention_prefill", "tvb_attention_prefill_supports", [c_int, c_int, c_int])
    return bool(fn(head_dim, num_q, num_kv))


PREFILL_TILE_TOKENS = 64          # query rows of a tile of the mma.sync kernels (PF_BM, TL_BM)


def attention_prefill_tile_tokens() -> int:
    """Tokens of a tile of the mma.sync prefill kernels; answered here, so that cutting a step into
    tiles compiles nothing (the launchers check their library's own value)."""
    return PREFILL_TILE_TOKENS


def attention_prefill(q: torch.Tensor, q_token_stride: int, key_cache: torch.Tensor,
                      value_cache: torch.Tensor, block_tables: torch.Tensor, positions: torch.Tensor,
                      tile_row: torch.Tensor, tile_first: torch.Tensor, tile_count: torch.Tensor, *,
                      num_q: int, num_kv: int, head_dim: int, window: int | None, scale: float,
                      out: torch.Tensor | None = None) -> torch.Tensor:
    """Paged causal attention on the tensor cores for tiles of up to 64 consecutive query
    tokens of one request (bfloat16).  Tile i holds ``tile_count[i]`` tokens from flat index
    ``tile_first[i]`` on of request row ``tile_row[i]``."""
    _need_cuda(q, key_cache, value_cache, block_tables, positions, tile_row, tile_first, tile_count)
    if q.dtype != torch.bfloat16 or key_cache.dtype != torch.bfloat16:
        raise KernelError("attention_prefill is a bfloat16 kernel")
    if not attention_prefill_supports(head_dim, num_q, num_kv):
        raise KernelError(f"attention_prefill does not take head_dim {head_dim}, {num_q}/{num_kv} heads")
    if _fn("attention_prefill", "tvb_attention_prefill_tile_tokens", [])() != PREFILL_TILE_TOKENS:
        raise KernelError("attention_prefill: the library's tile size is not the one steps are cut for")
    if key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            value_cache.shape != key_cache.shape or not key_cache.is_contiguous() or \
            not value_cache.is_contiguous():
        raise KernelError("attention_prefill: caches must be contiguous [pages, num_kv, page_size, head_dim]")
    for t in (block_tables, positions, tile_row, tile_first, tile_count):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_prefill: index tensors must be contiguous int32")
    tokens, tiles = positions.shape[0], tile_row.shape[0]
    if out is None:
        out = torch.empty((tokens, num_q * head_dim), dtype=q.dtype, device=q.device)
    fn = _fn("attention_prefill", "tvb_attention_prefill",
             [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
              c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_void_p])
    _check(fn(q.data_ptr(), q_token_stride, key_cache.data_ptr(), value_cache.data_ptr(),
              block_tables.data_ptr(), block_tables.shape[1], positions.data_ptr(), tile_row.data_ptr(),
              tile_first.data_ptr(), tile_count.data_ptr(), out.data_ptr(), tiles, num_q, num_kv,
              head_dim, key_cache.shape[2], window or 0, scale, _stream()), "attention_prefill")
    return out


# ------------------------------------------- tcgen05 prefill attention (head size 128)
_prefill_tc_tile: int | None = None
_attention_tc_unchecked = False


def attention_prefill_tc_tile_tokens() -> int:
    global _prefill_tc_tile
    if _prefill_tc_tile is None:
        _prefill_tc_tile = _fn("attention_prefill_tc", "tvb_attention_prefill_tc_tile_tokens", [])()
    return _prefill_tc_tile


def attention_prefill_tc_supports(head_dim: int, num_q: int, num_kv: int, page_size: int) -> bool:
    """Head size 128, pages of 8 to 128 tokens (a power of two), whole groups of q heads."""
    return (head_dim == 128 and num_q > 0 and num_kv > 0 and num_q % num_kv == 0
            and 8 <= page_size <= 128 and page_size & (page_size - 1) == 0)


def attention_prefill_tc(q: torch.Tensor, q_token_stride: int, key_cache: torch.Tensor,
                         value_cache: torch.Tensor, block_tables: torch.Tensor, positions: torch.Tensor,
                         tile_row: torch.Tensor, tile_first: torch.Tensor, tile_count: torch.Tensor, *,
                         num_q: int, num_kv: int, head_dim: int, window: int | None, scale: float,
                         out: torch.Tensor | None = None) -> torch.Tensor:
    """Paged causal attention on the tcgen05 tensor cores for tiles of up to 128 consecutive
    query tokens of one request (bfloat16, head size 128).  Tile i holds ``tile_count[i]`` tokens
    from flat index ``tile_first[i]`` on of request row ``tile_row[i]``; the tiles with the longest
    context come first.  The kernel reads whole pages: cache slots past a request's last key must
    hold finite values (they are multiplied by zero)."""
    _need_cuda(q, key_cache, value_cache, block_tables, positions, tile_row, tile_first, tile_count)
    if q.dtype != torch.bfloat16 or key_cache.dtype != torch.bfloat16:
        raise KernelError("attention_prefill_tc is a bfloat16 kernel")
    if key_cache.dim() != 4 or (key_cache.shape[1], key_cache.shape[3]) != (num_kv, head_dim) or \
            value_cache.shape != key_cache.shape or not key_cache.is_contiguous() or \
            not value_cache.is_contiguous():
        raise KernelError("attention_prefill_tc: caches must be contiguous [pages, num_kv, page_size, head_dim]")
    if not attention_prefill_tc_supports(head_dim, num_q, num_kv, key_cache.shape[2]):
        raise KernelError(f"attention_prefill_tc does not take head_dim {head_dim}, {num_q}/{num_kv} heads, "
                          f"pages of {key_cache.shape[2]}")
    if q.dim() != 2 or q.stride(1) != 1 or q.stride(0) != q_token_stride or q_token_stride % 8 \
            or q.shape[1] < num_q * head_dim:
        raise KernelError("attention_prefill_tc: q must be [tokens, >= num_q * head_dim] with 16-byte aligned rows")
    for t in (block_tables, positions, tile_row, tile_first, tile_count):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelError("attention_prefill_tc: index tensors must be contiguous int32")
    tokens, tiles = positions.shape[0], tile_row.shape[0]
    if out is None:
        out = torch.empty((tokens, num_q * head_dim), dtype=q.dtype, device=q.device)
    fn = _fn("attention_prefill_tc", "tvb_attention_prefill_tc",
             [c_void_p, c_longlong, c_longlong, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p,
              c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float,
              c_int, c_void_p])
    global _attention_tc_unchecked
    _check(fn(q.data_ptr(), q_token_stride, tokens, key_cache.data_ptr(), value_cache.data_ptr(),
              key_cache.shape[0], block_tables.data_ptr(), block_tables.shape[1], positions.data_ptr(),
              tile_row.data_ptr(), tile_first.data_ptr(), tile_count.data_ptr(), tiles, out.data_ptr(),
              num_q, num_kv, head_dim, key_cache.shape[2], window or 0, scale, _pdl("prefill"), _stream()),
           "attention_prefill_tc")
    _attention_tc_unchecked = True
    _guarded_counts[1] += 1
    return out


def attention_prefill_tc_status() -> int:
    """0, or which bounded wait of an attention_prefill_tc launch gave up since the last call.
    Synchronises the device; reading clears the record."""
    global _attention_tc_unchecked
    _attention_tc_unchecked = False
    return _fn("attention_prefill_tc", "tvb_attention_prefill_tc_status", [])()


# ------------------------------------------------ weight-streaming small-M GEMM
SMALL_M_MAX_ROWS = 32
PREFETCH_MAX_BYTES = 32 << 20
GEMM_BF16, GEMM_F32, GEMM_SILU = 0, 1, 2


def gemm_small_m(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16, *,
                 out: torch.Tensor | None = None, norm_weight: torch.Tensor | None = None,
                 residual: torch.Tensor | None = None, eps: float = 0.0, want_residual: bool = True,
                 row_squares: torch.Tensor | None = None, add_stream: torch.Tensor | None = None,
                 prefetch: torch.Tensor | None = None):
    """x [m <= 32, k] . w [n, k]^T, bfloat16 operands.  mode GEMM_BF16 / GEMM_F32: result
    [m, n] in that dtype; GEMM_SILU: w is [gate | up] with 2 n rows and the result is
    silu(x . gate^T) * (x . up^T), bfloat16 [m, n].

    With ``norm_weight`` the product is taken of RMSNorm(x + residual) * norm_weight instead
    of x (``residual`` may be None), and (result, rounded sum x + residual) is returned; the
    sum is None without a residual or with ``want_residual=False``.

    ``add_stream`` (GEMM_BF16; contiguous [m, n]): the result is round(round(product) + add_stream),
    the new residual stream, and (result, squares) is returned: squares [ceil(n / 16), m rounded up
    to 8] float32 holds the sum of squares of the result's rows over each tile of 16 columns.
    ``row_squares`` (with ``norm_weight``, without ``residual``): such sums for the rows of x, which
    is the stream itself; the result is (round(x * norm_weight) . w^T) * inverse RMS of the row, and
    only the result is returned.

    ``prefetch``: a tensor (the weight of the product after this one) whose first
    ``PREFETCH_MAX_BYTES`` the grid asks into L2 while it works."""
    _need_cuda(x, w, norm_weight, residual)
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2:
        raise KernelError("gemm_small_m wants bfloat16 matrices")
    m, k = x.shape
    rows = w.shape[0]
    if w.shape[1] != k or x.stride(1) != 1 or w.stride(1) != 1:
        raise KernelError("gemm_small_m: x [m, k] and w [n, k] with contiguous rows")
    if m < 1 or m > SMALL_M_MAX_ROWS or k % 8 or x.stride(0) % 8 or w.stride(0) % 8:
        raise KernelError(f"gemm_small_m takes up to {SMALL_M_MAX_ROWS} rows (and one at least), k and row strides "
                          f"multiples of 8 (m {m}, k {k})")
    if mode == GEMM_SILU and rows % 2:
        raise KernelError("gemm_small_m: a [gate | up] weight has an even number of rows")
    n = rows // 2 if mode == GEMM_SILU else rows
    residual_out = None
    weight_tag = BF16
    padded_rows = -(-m // 8) * 8
    squares_out = None
    if add_stream is not None:
        if (mode != GEMM_BF16 or add_stream.shape != (m, n) or add_stream.dtype != torch.bfloat16
                or not add_stream.is_contiguous() or out is not None):
            raise KernelError("gemm_small_m: add_stream is a contiguous bfloat16 [m, n] and the result is new")
        squares_out = torch.empty((-(-n // 16), padded_rows), dtype=torch.float32, device=x.device)
    if row_squares is not None:
        if (norm_weight is None or residual is not None or norm_weight.shape != (k,) or not x.is_contiguous()
                or row_squares.dtype != torch.float32 or row_squares.dim() != 2
                or row_squares.shape[1] != padded_rows or not row_squares.is_contiguous()
                or norm_weight.data_ptr() % 16):
            raise KernelError("gemm_small_m: row_squares [tiles, m rounded up to 8] float32 goes with a norm "
                              "weight [k], contiguous x and no residual")
        weight_tag = dtype_tag(norm_weight.dtype)
    elif norm_weight is not None:
        if norm_weight.shape != (k,) or not x.is_contiguous() or not gemm_small_m_takes_norm(m, k):
            raise KernelError("gemm_small_m: the fused norm wants contiguous x, a weight [k] and "
                              "rows that fit into shared memory")
        if residual is not None:
            if residual.shape != x.shape or residual.dtype != x.dtype or not residual.is_contiguous():
                raise KernelError("gemm_small_m: residual must match x")
            if want_residual:
                residual_out = torch.empty_like(x)
        weight_tag = dtype_tag(norm_weight.dtype)
    elif residual is not None:
        raise KernelError("gemm_small_m: a residual needs a norm weight")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32 if mode == GEMM_F32 else torch.bfloat16,
                          device=x.device)
    fn = _fn_of(f"gemm_small_m_nt{(m + 7) // 8}", "tvb_gemm_small_m",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_void_p, c_void_p, c_void_p, c_float, c_int, c_void_p, c_int, c_void_p, c_void_p,
              c_void_p, c_longlong, c_int, c_void_p])
    next_bytes = 0 if prefetch is None else min(prefetch.numel() * prefetch.element_size(),
                                                PREFETCH_MAX_BYTES)
    _check(fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, mode, _ptr(residual), _ptr(norm_weight), _ptr(residual_out), eps, weight_tag,
              _ptr(row_squares), 0 if row_squares is None else row_squares.shape[0], _ptr(add_stream),
              _ptr(squares_out), _ptr(prefetch), next_bytes, _pdl("gemm"), _stream()), "gemm_small_m")
    if add_stream is not None:
        return out, squares_out
    if norm_weight is not None and row_squares is None:
        return out, residual_out
    return out


def gemm_small_m_takes_norm(m: int, k: int) -> bool:
    """Whether the normalised rows [m rounded up to 8, k] fit into the kernel's shared memory."""
    return m <= SMALL_M_MAX_ROWS and k % 8 == 0 and (-(-m // 8) * 8) * (k + 32) * 2 <= 160 * 1024


# ------------------------------------------- tcgen05 matrix product (many rows)
def gemm_tc_takes(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16) -> bool:
    """Whether :func:`gemm_tc` takes this product: bfloat16, rows contiguous and 16-byte aligned,
    k and n multiples of 8."""
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2
            or x.shape[1] != w.shape[1] or x.stride(1) != 1 or w.stride(1) != 1):
        return False
    rows = w.shape[0]
    if mode == GEMM_SILU and rows % 2:
        return False
    n = rows // 2 if mode == GEMM_SILU else rows
    return (mode in (GEMM_BF16, GEMM_SILU) and x.shape[1] % 8 == 0 and n % 8 == 0
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tc(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16, *, out: torch.Tensor | None = None,
            tile_n: int = 0) -> torch.Tensor:
    """x [m, k] . w [n, k]^T in bfloat16 on the tcgen05 tensor cores (float32 accumulation in
    tensor memory).  GEMM_BF16: [m, n]; GEMM_SILU: w is [gate | up] with 2 n rows, the result is
    silu(x . gate^T) * (x . up^T) [m, n].  ``tile_n`` 128 or 256 forces the width of a tile."""
    _need_cuda(x, w)
    if not gemm_tc_takes(x, w, mode):
        raise KernelError("gemm_tc wants bfloat16 x [m, k] and w [n, k] with contiguous, 16-byte "
                          "aligned rows, k and n multiples of 8")
    m, k = x.shape
    n = w.shape[0] // 2 if mode == GEMM_SILU else w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.bfloat16, device=x.device)
    elif (out.dtype != torch.bfloat16 or out.shape != (m, n) or out.stride(1) != 1 or out.stride(0) % 8
          or out.data_ptr() % 16):
        raise KernelError("gemm_tc: out must be bfloat16 [m, n] with 16-byte aligned rows")
    fn = _fn("gemm_tc", "tvb_gemm_tc",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_int, c_int, c_void_p])
    global _gemm_tc_unchecked
    _check(fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, mode, tile_n, _pdl("gemm"), _stream()), "gemm_tc")
    _gemm_tc_unchecked = True
    _guarded_counts[0] += 1
    return out


# ----------------------------- tcgen05 matrix product (few rows, a large weight)
STREAM_MAX_ROWS = 128
_stream_scratch: dict[int, tuple[torch.Tensor, torch.Tensor]] = {}
_gemm_stream_used = False


def _stream_scratch_of(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Workspace (partial sums of tiles that two CTAs share) and counters of the stream-k kernel,
    one pair per device, sized for the largest launch and never freed: CUDA graphs keep their
    addresses.  Launches that use them must follow one another (those of one stream do)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    found = _stream_scratch.get(index)
    if found is None:
        sms = torch.cuda.get_device_properties(index).multi_processor_count
        workspace = torch.empty(sms * 2 * 2 * STREAM_MAX_ROWS * 128, dtype=torch.float32, device=device)
        counters = torch.zeros(1 << 16, dtype=torch.int32, device=device)
        found = _stream_scratch[index] = (workspace, counters)
    return found


def gemm_stream_takes(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16) -> bool:
    """Whether :func:`gemm_stream` takes this product: bfloat16, up to 128 rows of x, rows contiguous
    and 16-byte aligned, k a multiple of 8."""
    if (x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.dim() != 2 or w.dim() != 2
            or x.shape[1] != w.shape[1] or x.stride(1) != 1 or w.stride(1) != 1):
        return False
    rows = w.shape[0]
    if mode == GEMM_SILU and rows % 2:
        return False
    n = rows // 2 if mode == GEMM_SILU else rows
    return (mode in (GEMM_BF16, GEMM_F32, GEMM_SILU) and 0 < x.shape[0] <= STREAM_MAX_ROWS
            and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and n * 4 <= (1 << 16) * 128)


def gemm_stream(x: torch.Tensor, w: torch.Tensor, mode: int = GEMM_BF16, *, out: torch.Tensor | None = None,
                add_stream: torch.Tensor | None = None) -> torch.Tensor:
    """x [m <= 128, k] . w [n, k]^T for a large bfloat16 weight, streamed once through the tcgen05
    tensor cores with the work cut evenly over the SMs.  GEMM_BF16: bfloat16 [m, n], with
    ``add_stream`` (contiguous bfloat16 [m, n]) round(round(product) + add_stream); GEMM_F32:
    float32 [m, n]; GEMM_SILU: w is [gate | up] with 2 n rows, the result is
    silu(x . gate^T) * (x . up^T)."""
    _need_cuda(x, w, add_stream)
    if not gemm_stream_takes(x, w, mode):
        raise KernelError("gemm_stream wants bfloat16 x [m <= 128, k] and w [n, k] with contiguous, 16-byte "
                          "aligned rows and k a multiple of 8")
    m, k = x.shape
    n = w.shape[0] // 2 if mode == GEMM_SILU else w.shape[0]
    out_dtype = torch.float32 if mode == GEMM_F32 else torch.bfloat16
    if out is None:
        out = torch.empty((m, n), dtype=out_dtype, device=x.device)
    elif out.dtype != out_dtype or out.shape != (m, n) or out.stride(1) != 1:
        raise KernelError(f"gemm_stream: out must be {out_dtype} [m, n] with contiguous rows")
    if add_stream is not None and (mode != GEMM_BF16 or add_stream.shape != (m, n)
                                   or add_stream.dtype != torch.bfloat16 or not add_stream.is_contiguous()):
        raise KernelError("gemm_stream: add_stream is a contiguous bfloat16 [m, n] of a bfloat16 result")
    workspace, counters = _stream_scratch_of(x.device)
    fn = _fn("gemm_stream", "tvb_gemm_stream",
             [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_int, c_int, c_int,
              c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    global _gemm_tc_unchecked, _gemm_stream_used
    _check(fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
              m, n, k, mode, _ptr(add_stream), workspace.data_ptr(), counters.data_ptr(), _pdl("gemm"),
              _stream()), "gemm_stream")
    _gemm_tc_unchecked = _gemm_stream_used = True
    _guarded_counts[0] += 1
    return out


def gemm_stream_status() -> int:
    """0, or which bounded wait of a gemm_stream launch gave up since the last call.  Synchronises
    the device; reading clears the record."""
    return _fn("gemm_stream", "tvb_gemm_stream_status", [])()


_gemm_tc_unchecked = False


def gemm_tc_status() -> int:
    """0, or which bounded wait of a gemm_tc launch gave up since the last call (the results of
    that launch are not valid).  Synchronises the device; reading clears the record."""
    global _gemm_tc_unchecked
    _gemm_tc_unchecked = False
    return _fn("gemm_tc", "tvb_gemm_tc_status", [])()


def wait_probe(code: int = 77) -> tuple[int, int]:
    """Run the one-CTA kernel that waits on a barrier nothing arrives on: (status code the bounded
    wait recorded, millions of SM cycles it waited).  Takes about a second; the context stays
    usable.  Shows that a wait of the tcgen05 kernels that is never satisfied ends by itself."""
    waited = ctypes.c_int(0)
    fn = _fn("wait_probe", "tvb_wait_probe", [c_int, ctypes.POINTER(ctypes.c_int), c_void_p])
    status = fn(code, ctypes.byref(waited), _stream())
    if status < 0:
        raise KernelError(f"wait_probe failed ({status})")
    return status, waited.value


_guarded_counts = [0, 0]


def guarded_launch_counts() -> tuple[int, int]:
    """How often (gemm_tc or gemm_stream, attention_prefill_tc), the kernels with bounded waits, were launched
    through this module so far.  A caller that records a step into a CUDA graph compares the
    counts around one pass of the step and hands what it finds to :func:`note_guarded_launches`
    at every replay: a replay launches the kernels without passing through this module."""
    return _guarded_counts[0], _guarded_counts[1]


def note_guarded_launches(gemm: bool, attention: bool) -> None:
    """Kernels with bounded waits ran without this module seeing it (a graph replay): their status
    words are read at the next :func:`check_finished_launches`."""
    global _gemm_tc_unchecked, _attention_tc_unchecked
    _gemm_tc_unchecked = _gemm_tc_unchecked or bool(gemm)
    _attention_tc_unchecked = _attention_tc_unchecked or bool(attention)


def check_finished_launches() -> None:
    """Call after a step's results have reached the host: raises if a kernel with bounded waits
    gave up in a launch since the last call.  Costs nothing when no such kernel was launched."""
    if _gemm_tc_unchecked:
        status = gemm_tc_status()
        if status:
            raise KernelError(f"gemm_tc: a wait inside the kernel ran out (code {status}); "
                              "the results of this step are not valid")
        if _gemm_stream_used:
            status = gemm_stream_status()
            if status:
                raise KernelError(f"gemm_stream: a wait inside the kernel ran out (code {status}); "
                                  "the results of this step are not valid")
    if _attention_tc_unchecked:
        status = attention_prefill_tc_status()
        if status:
            raise KernelError(f"attention_prefill_tc: a wait inside the kernel ran out (code {status}); "
                              "the results of this step are not valid")
