"""Python entry points of the sm_100a kernels (``pylon_b200/csrc``).

Each function checks its tensors (device, dtype, contiguity, sizes), launches on torch's
current CUDA stream and returns without synchronising.  There is no CPU path: a tensor that
is not on a CUDA device, or a kernel library that cannot be built, raises.
"""
from __future__ import annotations

import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Optional, Sequence

import torch

from pylon_b200.kernels import build

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


def _dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels run in float32 or bfloat16, not {dtype}")


# The raw handle of torch's current stream, without building a Stream object (that costs some
# 15 us of host time, and an eager step asks some 300 times).
_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _ptr(tensor: Optional[torch.Tensor]) -> Optional[int]:
    """The address for a ``c_void_p`` parameter (ctypes takes an int, or None for null)."""
    return None if tensor is None else tensor.data_ptr()


def _need_cuda(*tensors: Optional[torch.Tensor]) -> None:
    for tensor in tensors:
        if tensor is not None and not tensor.is_cuda:
            raise KernelError("pylon_b200 kernels need CUDA tensors; there is no CPU path")


def _need(condition: bool, text: str) -> None:
    if not condition:
        raise KernelError(text)


# Kernels of this package launched so far in this process (library matrix products are
# not counted).  Benchmarks read it before and after a timed region.
launches = [0]


def _check(library: ctypes.CDLL, code: int) -> None:
    launches[0] += 1
    if code != 0:
        raise KernelError(library.pylon_last_error().decode(errors="replace") or f"kernel call failed ({code})")


# Kernels that wait on mbarriers (TMA copies, tensor-core completion) bound every wait; one that
# runs out sets its word here instead of hanging, and the result of that launch is void.  One
# tensor per device: [tcgen05 product, attention, TMA-fed decode product, unused].
_error_word_storage: dict[int, torch.Tensor] = {}
_ERROR_WORD_NAMES = ("tcgen05 product", "attention", "TMA-fed decode product", "cache write")
BAD_PAGE_CODE = 5   # PYLON_ERROR_BAD_PAGE of csrc/common.cuh: a block table named a page that the pool does not have


def _device_index(device: torch.device | str) -> int:
    """``cuda`` and ``cuda:N`` name the same device when N is the current one: buffers kept per device go by the number."""
    device = torch.device(device)
    return torch.cuda.current_device() if device.index is None else device.index


def _multiprocessors(device: torch.device | str) -> int:
    """How many multiprocessors ``device`` has (asked once): grids, splits and tile choices are sized by it."""
    index = _device_index(device)
    if index not in _multiprocessor_counts:
        _multiprocessor_counts[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _multiprocessor_counts[index]


_multiprocessor_counts: dict[int, int] = {}


def _error_words(device: torch.device) -> torch.Tensor:
    key = _device_index(device)
    if key not in _error_word_storage:
        _error_word_storage[key] = torch.zeros(4, dtype=torch.int32, device=torch.device("cuda", key))
    return _error_word_storage[key]


def cache_write_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the kernel that writes new keys and values into their pages sets when the block
    table names a page the pool does not have (nothing is written there).  Zero in every healthy run."""
    return _error_words(device)[3:4]


_error_word_copies: dict[int, torch.Tensor] = {}   # pinned host copies, filled by queue_error_word_read


def queue_error_word_read(device: torch.device) -> None:
    """Enqueues a copy of the error words into pinned host memory behind the work queued so far, without waiting.  A
    caller that is about to wait for the stream anyway (to read a step's tokens back) queues this first and looks at
    the words with ``raise_on_kernel_errors(device, queued=True)`` afterwards: one trip to the device instead of two."""
    key = _device_index(device)
    if key not in _error_word_storage:
        return
    if key not in _error_word_copies:
        _error_word_copies[key] = torch.zeros(4, dtype=torch.int32, pin_memory=True)
    _error_word_copies[key].copy_(_error_word_storage[key], non_blocking=True)


def queue_error_word_copy(device: torch.device) -> Optional[torch.Tensor]:
    """Like :func:`queue_error_word_read`, into a pinned buffer of the caller's own (returned; ``None`` if no kernel that
    can set the words has run): for callers that have more than one step in flight and look at each step's words when
    they come to it, with ``raise_on_kernel_errors(device, words=...)``."""
    key = _device_index(device)
    if key not in _error_word_storage:
        return None
    words = torch.zeros(4, dtype=torch.int32, pin_memory=True)
    words.copy_(_error_word_storage[key], non_blocking=True)
    return words


def raise_on_kernel_errors(device: torch.device, queued: bool = False, words: Optional[torch.Tensor] = None) -> None:
    """Reads the error words of ``device`` (a 16-byte copy that waits for the work queued so
    far; with ``queued`` the copy :func:`queue_error_word_read` enqueued, with ``words`` the one
    :func:`queue_error_word_copy` returned, which the caller has
    waited for since) and raises if, since the last call, a kernel gave up one of its bounded
    waits or met a block table that names a page outside the pool.  The words are cleared, so
    the next call reports only what happens from now on; and the counters by which the blocks
    of a decode attention find the last of them are put back to zero, since a block that gave
    up never took part in the count of the rows it shared, and the next launch must find zeros."""
    key = _device_index(device)
    if key not in _error_word_storage:
        return   # no kernel that can set them has run
    if words is not None:
        words = words.tolist()
    elif queued and key in _error_word_copies:
        words = _error_word_copies[key].tolist()
    else:
        words = _error_word_storage[key].cpu().tolist()
    if any(words):
        _error_word_storage[key].zero_()
        for (index, _purpose), buffer in _counter_buffers.items():
            if index == key:
                buffer.zero_()
        what = ", ".join(
            f"{name} ({'a block table names a page outside the pool' if code == BAD_PAGE_CODE else 'a bounded wait ran out'}, code {code})"
            for name, code in zip(_ERROR_WORD_NAMES, words) if code)
        raise KernelError(f"kernel error in: {what}; the results of that step are void")


_SIGNATURES = {
    "elementwise.cu": {
        "pylon_embed_gather": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_void_p],
        "pylon_take_tokens": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p],
        "pylon_logit_transform": [c_void_p, c_longlong, c_float, c_float, c_void_p],
        "pylon_add_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_int, c_void_p],
        "pylon_residual_add": [c_void_p, c_void_p, c_longlong, c_int, c_void_p],
        "pylon_add_parts_rmsnorm": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p],
        "pylon_qk_norm_rope_kv_write": [c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                                        c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int,
                                        c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_qk_norm_rope_kv_write_parts": [c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_void_p, c_void_p, c_int, c_int,
                                              c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                              c_int, c_void_p, c_void_p],
        "pylon_qk_norm": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_void_p],
        "pylon_swiglu": [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    },
    "gemm_f32.cu": {
        "pylon_gemm_f32_nt": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p],
    },
    "gemm_skinny.cu": {
        "pylon_gemm_skinny_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int, c_void_p],
    },
    "gemm_stream.cu": {
        "pylon_gemm_stream_partial": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_int, c_void_p, c_void_p],
        "pylon_gemm_stream_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p],
        "pylon_gemm_stream_swiglu": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p],
    },
    "gemm_tcgen05.cu": {
        "pylon_gemm_tcgen05_bf16": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong, c_int,
                                    c_void_p, c_int, c_void_p],
        "pylon_gemm_tcgen05_force_tile": [c_int],
        "pylon_gemm_tcgen05_qkv_rotate": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_longlong, c_longlong, c_longlong, c_void_p, c_void_p, c_float,
                                          c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
                                          c_int, c_void_p, c_void_p, c_int, c_void_p],
    },
    "attention_simple.cu": {
        "pylon_paged_attention_simple": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                         c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_float,
                                         c_int, c_int, c_void_p],
    },
    "attention_mma.cu": {
        "pylon_paged_attention_mma": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                      c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
                                      c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
        "pylon_attention_scratch_floats": [c_int, c_int, c_int, c_int, c_int, c_int],
        "pylon_attention_decode_blocks": [],
    },
    "attention_tcgen05.cu": {
        "pylon_paged_attention_tcgen05": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                          c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    },
    "sampling.cu": {
        "pylon_sample": [c_void_p, c_longlong, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    },
}


_typed_libraries: dict[tuple, ctypes.CDLL] = {}


def _library(source: str, defines: Optional[dict[str, int]] = None) -> ctypes.CDLL:
    key = (source, tuple(sorted(defines.items())) if defines else ())
    library = _typed_libraries.get(key)
    if library is not None:
        return library
    library = build.load(source, defines)
    if not getattr(library, "_pylon_typed", False):
        for name, argtypes in _SIGNATURES.get(source, {}).items():
            function = getattr(library, name)
            function.argtypes = argtypes
            function.restype = c_longlong if name.endswith("_floats") else c_int
        library._pylon_typed = True
    _typed_libraries[key] = library
    return library


def build_all() -> list[str]:
    """Every library with its default sizes (the tensor-core attention for head size 128)."""
    names = []
    for source in _SIGNATURES:
        defines = {"PYLON_HEAD_DIM": 128} if source in ("attention_mma.cu", "attention_tcgen05.cu") else None
        _library(source, defines)
        names.append(build.library_name(source, defines))
    return names


# ---------------------------------------------------------------------------------------
# embedding, norms, residual
# ---------------------------------------------------------------------------------------
def embed_gather(ids: torch.Tensor, table: torch.Tensor, out: Optional[torch.Tensor] = None, scale: float = 1.0) -> torch.Tensor:
    """float32 ``[T, width]`` rows of ``table`` (``[vocab, width]``) picked by int32 ``ids``, times ``scale``."""
    _need_cuda(ids, table, out)
    _need(ids.dtype == torch.int32 and ids.dim() == 1 and ids.is_contiguous(), "embed_gather: ids must be contiguous int32 [T]")
    _need(table.dim() == 2 and table.is_contiguous(), "embed_gather: table must be contiguous [vocab, width]")
    tokens, (vocab, width) = ids.shape[0], table.shape
    if out is None:
        out = torch.empty((tokens, width), dtype=torch.float32, device=table.device)
    _need(out.dtype == torch.float32 and out.shape == (tokens, width) and out.is_contiguous(), "embed_gather: out must be contiguous float32 [T, width]")
    library = _library("elementwise.cu")
    _check(library, library.pylon_embed_gather(_ptr(ids), _ptr(table), _ptr(out), tokens, width, vocab, _dtype_code(table.dtype), float(scale), _stream()))
    return out


def take_tokens(ids: torch.Tensor, source: torch.Tensor, sampled: torch.Tensor) -> torch.Tensor:
    """In place on int32 ``ids [T]``: ``ids[t] = sampled[source[t]]`` wherever ``source[t] >= 0``.  How a step gets tokens
    that the sampling kernel chose in the step before and the host has not read yet."""
    _need_cuda(ids, source, sampled)
    for name, tensor in (("ids", ids), ("source", source), ("sampled", sampled)):
        _need(tensor.dtype == torch.int32 and tensor.dim() == 1 and tensor.is_contiguous(), f"take_tokens: {name} must be contiguous int32")
    _need(source.shape[0] >= ids.shape[0], "take_tokens: a source for every token")
    library = _library("elementwise.cu")
    _check(library, library.pylon_take_tokens(_ptr(ids), _ptr(source), _ptr(sampled), sampled.shape[0], ids.shape[0], _stream()))
    return ids


def logit_transform(logits: torch.Tensor, scale: float = 1.0, softcap: Optional[float] = None) -> torch.Tensor:
    """In place on float32 ``logits``: ``y = x * scale``, then with a ``softcap`` c: ``y = c * tanh(y / c)``."""
    _need_cuda(logits)
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "logit_transform: logits must be contiguous float32")
    _need(softcap is None or softcap > 0, "logit_transform: a soft cap must be positive")
    library = _library("elementwise.cu")
    _check(library, library.pylon_logit_transform(_ptr(logits), logits.numel(), float(scale), float(softcap or 0.0), _stream()))
    return logits


def add_rmsnorm(
    residual: torch.Tensor,
    delta: Optional[torch.Tensor],
    weight: torch.Tensor,
    eps: float,
    out_dtype: torch.dtype,
    rows: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """``residual += delta`` (float32, in place, skipped when ``rows`` selects rows), then
    RMSNorm of the selected rows with the float32 ``weight``; returns ``out_dtype [n, width]``.
    ``delta`` may also be float32 partial sums ``[parts, T, width]`` (see
    :func:`linear_for_residual`): their sum is the delta."""
    _need_cuda(residual, delta, weight, rows, out)
    if delta is not None and delta.dim() == 3:
        if out is None and out_dtype == torch.bfloat16 and delta.dtype == torch.float32 and delta.is_contiguous() \
                and delta.shape[1:] == residual.shape and residual.is_contiguous() and residual.shape[1] % 4 == 0 and residual.shape[1] <= 8192 \
                and (rows is None or (rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous())):
            n_rows = residual.shape[0] if rows is None else rows.shape[0]
            normed = torch.empty((n_rows, residual.shape[1]), dtype=torch.bfloat16, device=residual.device)
            library = _library("elementwise.cu")
            _check(library, library.pylon_add_parts_rmsnorm(_ptr(residual), _ptr(delta), delta.shape[0], _ptr(weight), _ptr(rows), _ptr(normed),
                                                            n_rows, residual.shape[0], residual.shape[1], float(eps), _stream()))
            return normed
        delta = delta.sum(dim=0).to(out_dtype)
    _need(residual.dtype == torch.float32 and residual.dim() == 2 and residual.is_contiguous(), "add_rmsnorm: residual must be contiguous float32 [T, width]")
    tokens, width = residual.shape
    _need(weight.dtype == torch.float32 and weight.shape == (width,) and weight.is_contiguous(), "add_rmsnorm: weight must be float32 [width]")
    if delta is not None:
        _need(delta.shape == residual.shape and delta.is_contiguous() and delta.dtype == out_dtype, "add_rmsnorm: delta must be contiguous [T, width] in the activation dtype")
    n_rows = tokens
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.dim() == 1 and rows.is_contiguous(), "add_rmsnorm: rows must be contiguous int32")
        n_rows = rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, width), dtype=out_dtype, device=residual.device)
    _need(out.shape == (n_rows, width) and out.dtype == out_dtype and out.is_contiguous(), "add_rmsnorm: out has the wrong shape or dtype")
    library = _library("elementwise.cu")
    _check(library, library.pylon_add_rmsnorm(_ptr(residual), _ptr(delta), _ptr(weight), _ptr(rows), _ptr(out), n_rows, width,
                                              float(eps), 0 if rows is not None else 1, _dtype_code(out_dtype), _stream()))
    return out


def residual_add(residual: torch.Tensor, delta: torch.Tensor) -> None:
    _need_cuda(residual, delta)
    if delta.dim() == 3:   # partial sums
        for part in delta:
            residual_add(residual, part)
        return
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and delta.is_contiguous() and delta.shape == residual.shape, "residual_add: shapes differ or tensors are not contiguous")
    library = _library("elementwise.cu")
    _check(library, library.pylon_residual_add(_ptr(residual), _ptr(delta), residual.numel(), _dtype_code(delta.dtype), _stream()))


def qk_norm_rope_kv_write(
    qkv: torch.Tensor,
    q_weight: Optional[torch.Tensor],
    k_weight: Optional[torch.Tensor],
    eps: float,
    cos: Optional[torch.Tensor],
    sin: Optional[torch.Tensor],
    rotary_dim: int,
    positions: torch.Tensor,
    token_row: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    nq: int,
    nkv: int,
    head_dim: int,
) -> torch.Tensor:
    """On ``qkv [T, (nq + 2 nkv) * d]``: RMSNorm each q and k head (when weights are given),
    rotate them by the float32 ``cos``/``sin [positions, rotary_dim / 2]`` tables, write q
    back in place and k, v into ``[pages, nkv, page_size, d]`` pages at each token's slot.
    Returns the tensor whose first ``nq * d`` columns now hold q: ``qkv`` itself.

    ``qkv`` may also be float32 partial sums ``[parts, T, (nq + 2 nkv) * d]`` (see
    :func:`linear_for_rotation`): they are added up on the way, and q is returned in a tensor
    of its own, ``[T, nq * d]`` in the pages' dtype."""
    _need_cuda(qkv, q_weight, k_weight, cos, sin, positions, token_row, block_table, k_pages, v_pages)
    partial = qkv.dim() == 3
    tokens = qkv.shape[-2]
    _need(qkv.dim() in (2, 3) and qkv.is_contiguous() and qkv.shape[-1] == (nq + 2 * nkv) * head_dim, "qk_norm_rope_kv_write: qkv must be contiguous [T, (nq + 2 nkv) * d]")
    for weight in (q_weight, k_weight):
        if weight is not None:
            _need(weight.dtype == torch.float32 and weight.shape == (head_dim,) and weight.is_contiguous(), "qk_norm_rope_kv_write: norm weights must be float32 [d]")
    table_positions = 0
    if cos is not None:
        _need(sin is not None and cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape
              and cos.dim() == 2 and cos.shape[1] * 2 == rotary_dim and cos.is_contiguous() and sin.is_contiguous(),
              "qk_norm_rope_kv_write: cos/sin must be float32 [positions, rotary_dim / 2]")
        table_positions = cos.shape[0]
    else:
        rotary_dim = 0
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "qk_norm_rope_kv_write: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "qk_norm_rope_kv_write: block_table must be contiguous int32 [rows, width]")
    activation = k_pages.dtype if partial else qkv.dtype
    for pages in (k_pages, v_pages):
        _need(pages.dtype == activation and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1:] == (nkv, page_size, head_dim),
              "qk_norm_rope_kv_write: pages must be contiguous [pages, nkv, page_size, d] in the activation dtype")
    library = _library("elementwise.cu")
    if partial:
        _need(qkv.dtype == torch.float32 and activation == torch.bfloat16 and head_dim in (64, 128, 256) and rotary_dim in (0, head_dim),
              "qk_norm_rope_kv_write: partial sums are float32, for bfloat16 pages, head size 64, 128 or 256 and rotation over the whole head")
        q = torch.empty((tokens, nq * head_dim), dtype=torch.bfloat16, device=qkv.device)
        _check(library, library.pylon_qk_norm_rope_kv_write_parts(
            _ptr(qkv), qkv.shape[0], _ptr(q), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rotary_dim, table_positions,
            _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
            k_pages.shape[0], nq, nkv, head_dim, tokens, _ptr(cache_write_error_word(k_pages.device)), _stream()))
        return q
    _check(library, library.pylon_qk_norm_rope_kv_write(
        _ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin), rotary_dim, table_positions,
        _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
        k_pages.shape[0], nq, nkv, head_dim, tokens, _dtype_code(qkv.dtype), _ptr(cache_write_error_word(k_pages.device)), _stream()))
    return qkv


def qk_norm(qkv: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float, nq: int, nkv: int, head_dim: int) -> torch.Tensor:
    """RMSNorm of every q and k head of ``qkv [T, (nq + 2 nkv) * d]`` in place, without rotation or
    cache write: for position encodings that run as a step of their own between the norms and
    :func:`qk_norm_rope_kv_write` (called without weights and tables, it then only writes the cache)."""
    _need_cuda(qkv, q_weight, k_weight)
    _need(qkv.dim() == 2 and qkv.is_contiguous() and qkv.shape[1] == (nq + 2 * nkv) * head_dim, "qk_norm: qkv must be contiguous [T, (nq + 2 nkv) * d]")
    for weight in (q_weight, k_weight):
        if weight is not None:
            _need(weight.dtype == torch.float32 and weight.shape == (head_dim,) and weight.is_contiguous(), "qk_norm: norm weights must be float32 [d]")
    library = _library("elementwise.cu")
    _check(library, library.pylon_qk_norm(_ptr(qkv), _ptr(q_weight), _ptr(k_weight), float(eps), nq, nkv, head_dim, qkv.shape[0],
                                          _dtype_code(qkv.dtype), _stream()))
    return qkv


def swiglu(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None, interleaved: bool = False) -> torch.Tensor:
    """``silu(gate) * up`` for ``gate_up`` of shape ``[T, 2 * inter]``: ``[gate | up]`` in two
    halves, or with ``interleaved`` in alternating groups of 8 columns
    (``[g0..g7 u0..u7 g8..g15 u8..u15 ...]``, the layout :func:`interleave_gate_up` gives the
    weights)."""
    _need_cuda(gate_up, out)
    _need(gate_up.dim() == 2 and gate_up.is_contiguous() and gate_up.shape[1] % 2 == 0, "swiglu: gate_up must be contiguous [T, 2 * inter]")
    tokens, inter = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((tokens, inter), dtype=gate_up.dtype, device=gate_up.device)
    _need(out.shape == (tokens, inter) and out.dtype == gate_up.dtype and out.is_contiguous(), "swiglu: out has the wrong shape or dtype")
    library = _library("elementwise.cu")
    _check(library, library.pylon_swiglu(_ptr(gate_up), _ptr(out), tokens, inter, int(interleaved), _dtype_code(gate_up.dtype), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# matrix products: y = x @ w.T
# ---------------------------------------------------------------------------------------
SKINNY_MAX_ROWS = 8   # up to this many rows the weight-streaming kernel runs (it takes up to 64); above, the library


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``x [M, K] @ w [N, K].T`` with float32 accumulation.

    float32 operands use the plain-FMA kernel (true 32-bit, no tensor cores).  bfloat16
    operands with up to ``SKINNY_MAX_ROWS`` rows use the weight-streaming kernel; many rows
    whose 128 x 256 tiles fill whole rounds over the SMs use our tcgen05 kernel; the rest go to
    the library matrix product, as raun6k/Pylon's ``nn.Linear`` layers do
    (src/pylon/model/layers.py:17-23,95-106).  ``out_dtype=torch.float32`` keeps the 32-bit
    accumulator (used for logits).
    """
    _need_cuda(x, w)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], f"linear: shapes {tuple(x.shape)} and {tuple(w.shape)} do not match")
    _need(x.dtype == w.dtype, f"linear: activations are {x.dtype} but weights are {w.dtype}")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear: the reduced dimension must be contiguous")
    out_dtype = out_dtype or x.dtype
    m, k = x.shape
    n = w.shape[0]
    if x.dtype == torch.float32:
        _need(out_dtype == torch.float32, "linear: float32 operands give float32 results")
        y = torch.empty((m, n), dtype=torch.float32, device=x.device)
        library = _library("gemm_f32.cu")
        _check(library, library.pylon_gemm_f32_nt(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), n, _stream()))
        return y
    _need(x.dtype == torch.bfloat16, f"linear: unsupported dtype {x.dtype}")
    _need(out_dtype in (torch.bfloat16, torch.float32), f"linear: unsupported result dtype {out_dtype}")
    if m <= SKINNY_MAX_ROWS and k % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 \
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
        return linear_skinny(x, w, out_dtype)   # few rows (decode): our weight-streaming kernel
    if out_dtype == torch.bfloat16:
        if _tcgen05_fills_the_sms(m, n, _multiprocessors(x.device)) and k % 8 == 0 and n % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 \
                and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
            return linear_tcgen05(x, w)
        return torch.mm(x, w.t())
    return torch.mm(x, w.t(), out_dtype=torch.float32)


def _tcgen05_fills_the_sms(m: int, n: int, sms: int) -> bool:
    """Whether a persistent block per SM over 128 x 256 tiles wastes under a fifth of its
    rounds: there our kernel is level with the library's, elsewhere the library is ahead.  (The
    output and down projections of 2,048 rows are 160 such tiles on 148 SMs.  With tiles of 288
    columns, one round, our kernel takes 31.7 and 78.7 us for them, the library 29.6 and 71.7 us.)"""
    if m < TCGEN05_MIN_ROWS:
        return False
    tiles = -(-m // 128) * -(-n // 256)
    rounds = -(-tiles // sms)
    return tiles >= 0.8 * rounds * sms


STREAM_MAX_ROWS = 32   # up to this many rows the TMA-fed kernel beats the library (it takes up to 64)
STREAM_MAX_PARTS = 4


def linear_for_residual(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``x @ w.T`` for a result that goes straight into the residual stream: either the
    product ``[M, N]`` in the activation dtype, or - for the few rows of a decode step -
    float32 partial sums ``[parts, M, N]`` over slices of k, which the stream's next norm adds
    up (no extra kernel, no atomics).  The slices make enough blocks to fill the GPU however
    few rows the matrix has."""
    m, k = x.shape
    n = w.shape[0]
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and m <= STREAM_MAX_ROWS and k >= 1024 and k % 8 == 0
            and n % 4 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return linear_stream_partial(x, w)
    return linear(x, w)


def linear_for_rotation(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int) -> torch.Tensor:
    """The fused QKV product for :func:`qk_norm_rope_kv_write`: the product ``[M, N]`` in the
    activation dtype, or - for the few rows of a decode step, where the TMA-fed kernel with
    its slices of k is the fastest way to read the weights - float32 partial sums
    ``[parts, M, N]``, which the rotation kernel adds up as it reads them."""
    m, k = x.shape
    n = w.shape[0]
    if (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_cuda and m <= STREAM_MAX_ROWS and k >= 1024 and k % 8 == 0
            and head_dim in (64, 128, 256) and rotary_dim in (0, head_dim) and n % 4 == 0 and x.stride(1) == 1 and w.stride(1) == 1
            and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0):
        return linear_stream_partial(x, w)
    return linear(x, w)


def stream_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the TMA-fed decode product sets when one of its bounded waits ran out
    (its result is then void).  Zero in every healthy run."""
    return _error_words(device)[2:3]


def linear_stream_partial(x: torch.Tensor, w: torch.Tensor, parts: Optional[int] = None) -> torch.Tensor:
    """bfloat16 ``x [M <= 64, K] @ w [N, K].T`` as float32 partial sums ``[parts, M, N]`` over
    slices of k, the weights streamed by TMA through a shared-memory ring.  ``parts`` defaults
    to what gives every SM up to three blocks (64 weight rows x one slice each), at most
    ``STREAM_MAX_PARTS``: more parts cost the reader more than they save here (the norm that adds
    them up took 3.0 us with 4 parts and 5.1 us with 11)."""
    _need_cuda(x, w)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16,
          "linear_stream_partial: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_stream_partial: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    slabs, k_boxes = -(-n // 64), -(-k // 64)
    if parts is None:
        parts = max(1, min(STREAM_MAX_PARTS, k_boxes, (3 * _multiprocessors(x.device)) // slabs))
    y = torch.empty((parts, m, n), dtype=torch.float32, device=x.device)
    library = _library("gemm_stream.cu")
    _check(library, library.pylon_gemm_stream_partial(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), parts,
                                                      _ptr(stream_error_word(x.device)), _stream()))
    return y


def linear_stream(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """bfloat16 ``x [M <= 64, K] @ w [N, K].T`` on the TMA-fed kernel, one block per 64 weight rows
    over the whole of k; with ``swiglu`` the rows of ``w`` are interleaved gate/up groups (see
    :func:`interleave_gate_up`) and the result is ``silu(gate) * up``, ``[M, N / 2]``."""
    _need_cuda(x, w)
    _need(x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16,
          "linear_stream: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_stream: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n // 2 if swiglu else n), dtype=torch.bfloat16, device=x.device)
    library = _library("gemm_stream.cu")
    entry = library.pylon_gemm_stream_swiglu if swiglu else library.pylon_gemm_stream_bf16
    _check(library, entry(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0), _ptr(stream_error_word(x.device)), _stream()))
    return y


def linear_skinny(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """The weight-streaming kernel itself: bfloat16 ``x [M <= 64, K] @ w [N, K].T`` with ``K``
    and the row strides multiples of 8 and 16-byte aligned operands; anything else is refused."""
    _need_cuda(x, w)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1],
          "linear_skinny: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_skinny: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n), dtype=out_dtype, device=x.device)
    library = _library("gemm_skinny.cu")
    _check(library, library.pylon_gemm_skinny_bf16(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), n, _dtype_code(out_dtype), _stream()))
    return y


TCGEN05_MIN_ROWS = 128   # from this many rows the gate/up product runs on our tcgen05 kernel, SwiGLU in its epilogue

def tcgen05_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the tcgen05 kernels set when one of their bounded waits ran out
    (the result of that launch is then void).  Zero in every healthy run."""
    return _error_words(device)[0:1]


def tcgen05_force_tile(columns: int = 0) -> None:
    """For measurements: later ``linear_tcgen05`` calls use ``128 x columns`` output tiles
    (288, 256, 192, 160 or 128); 0 restores the choice by size."""
    _library("gemm_tcgen05.cu").pylon_gemm_tcgen05_force_tile(columns)


def linear_tcgen05(x: torch.Tensor, w: torch.Tensor, swiglu: bool = False) -> torch.Tensor:
    """bfloat16 ``x [M, K] @ w [N, K].T`` on the tcgen05 tensor cores (TMA-fed, accumulators in
    tensor memory).  With ``swiglu`` the rows of ``w`` are interleaved by
    :func:`interleave_gate_up` and the result is ``silu(gate) * up``, ``[M, N / 2]``."""
    _need_cuda(x, w)
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1],
          "linear_tcgen05: bfloat16 x [M, K] and w [N, K]")
    _need(x.stride(1) == 1 and w.stride(1) == 1, "linear_tcgen05: the reduced dimension must be contiguous")
    m, k = x.shape
    n = w.shape[0]
    y = torch.empty((m, n // 2 if swiglu else n), dtype=torch.bfloat16, device=x.device)
    library = _library("gemm_tcgen05.cu")
    _check(library, library.pylon_gemm_tcgen05_bf16(_ptr(x), _ptr(w), _ptr(y), m, n, k, x.stride(0), w.stride(0), y.stride(0), int(swiglu),
                                                    _ptr(tcgen05_error_word(x.device)), _multiprocessors(x.device), _stream()))
    return y

QKV_ROTATION_MIN_ROWS = 3_072


def qkv_rotation_fuses(x: torch.Tensor, w: torch.Tensor, head_dim: int, rotary_dim: int, k_pages: torch.Tensor) -> bool:
    """Whether :func:`linear_qkv_rotated` takes this step's QKV product: a long prompt portion, in bfloat16, heads of 64
    or 128 rotated as a whole.  The last tile's longer epilogue has nothing to hide behind, so the fusion pays from some
    3,000 rows on (Qwen3-4B widths: 108 us against 115 us for product and rotation kernel at 4,096 rows, 204 against 239
    at 8,192; 61 against 59 at 2,048)."""
    m, k = x.shape
    return (m >= QKV_ROTATION_MIN_ROWS and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k_pages.dtype == torch.bfloat16 and x.is_cuda and head_dim in (64, 128)
            and rotary_dim == head_dim and k % 8 == 0 and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and _tcgen05_fills_the_sms(m, w.shape[0], _multiprocessors(x.device)))


def linear_qkv_rotated(
    x: torch.Tensor, w: torch.Tensor, q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float, cos: torch.Tensor,
    sin: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor, block_table: torch.Tensor, page_size: int, k_pages: torch.Tensor,
    v_pages: torch.Tensor, nq: int, nkv: int, head_dim: int,
) -> torch.Tensor:
    """The fused QKV product ``x [T, K] @ w [(nq + 2 nkv) * d, K].T`` on the tcgen05 kernel with
    :func:`qk_norm_rope_kv_write` in its epilogue: the heads are normalised and rotated from the float32 accumulators, k
    and v go straight into their pages and q, ``[T, nq * d]`` in bfloat16, is returned; the product never goes to memory."""
    _need_cuda(x, w, q_weight, k_weight, cos, sin, positions, token_row, block_table, k_pages, v_pages)
    tokens, k = x.shape
    _need(x.dim() == 2 and w.dim() == 2 and w.shape == ((nq + 2 * nkv) * head_dim, k) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
          and x.stride(1) == 1 and w.stride(1) == 1, "linear_qkv_rotated: bfloat16 x [T, K] and w [(nq + 2 nkv) * d, K]")
    for weight in (q_weight, k_weight):
        if weight is not None:
            _need(weight.dtype == torch.float32 and weight.shape == (head_dim,) and weight.is_contiguous(), "linear_qkv_rotated: norm weights must be float32 [d]")
    _need(cos.dtype == torch.float32 and sin.dtype == torch.float32 and cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] * 2 == head_dim
          and cos.is_contiguous() and sin.is_contiguous(), "linear_qkv_rotated: cos/sin must be float32 [positions, d / 2]")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "linear_qkv_rotated: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "linear_qkv_rotated: block_table must be contiguous int32 [rows, width]")
    for pages in (k_pages, v_pages):
        _need(pages.dtype == torch.bfloat16 and pages.is_contiguous() and pages.dim() == 4 and pages.shape[1:] == (nkv, page_size, head_dim),
              "linear_qkv_rotated: pages must be contiguous bfloat16 [pages, nkv, page_size, d]")
    q = torch.empty((tokens, nq * head_dim), dtype=torch.bfloat16, device=x.device)
    library = _library("gemm_tcgen05.cu")
    _check(library, library.pylon_gemm_tcgen05_qkv_rotate(
        _ptr(x), _ptr(w), _ptr(q), tokens, k, x.stride(0), w.stride(0), q.stride(0), _ptr(q_weight), _ptr(k_weight), float(eps), _ptr(cos), _ptr(sin),
        cos.shape[0], _ptr(positions), _ptr(token_row), _ptr(block_table), block_table.shape[1], page_size, _ptr(k_pages), _ptr(v_pages),
        k_pages.shape[0], nq, nkv, head_dim, _ptr(cache_write_error_word(k_pages.device)), _ptr(tcgen05_error_word(x.device)),
        _multiprocessors(x.device), _stream()))
    return q


# Small integer buffers kernels use to find out which of their blocks finishes last.  They
# are zero between launches (a kernel leaves its counters as it found them) and launches on
# one stream follow each other, so one buffer per device and purpose is enough.
_counter_buffers: dict[tuple, torch.Tensor] = {}


def _zeroed_counters(device: torch.device, purpose: str, count: int) -> torch.Tensor:
    key = (_device_index(device), purpose)
    buffer = _counter_buffers.get(key)
    if buffer is None or buffer.numel() < count:
        if buffer is not None:
            _retired_counter_buffers.append(buffer)   # a captured graph may still hold its address
        buffer = torch.zeros(max(count, 1 << 16), dtype=torch.int32, device=device)
        _counter_buffers[key] = buffer
    return buffer


_retired_counter_buffers: list[torch.Tensor] = []


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Stacks the ``[inter, K]`` gate and up matrices in alternating groups of 8 rows (8 gate
    rows, their 8 up rows, ...), so that one block of 16 weight rows holds both halves of 8
    outputs.  ``inter`` must be a multiple of 8."""
    inter, k = gate.shape
    _need(up.shape == gate.shape and inter % 8 == 0, "interleave_gate_up: equal shapes with a row count that is a multiple of 8")
    return torch.stack((gate.reshape(inter // 8, 8, k), up.reshape(inter // 8, 8, k)), dim=1).reshape(2 * inter, k).contiguous()


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """``silu(x @ gate.T) * (x @ up.T)`` for weights stacked by :func:`interleave_gate_up`:
    one kernel for few rows (the TMA-fed decode kernel) and for many (the tcgen05 kernel), the
    library product and the SwiGLU kernel in between."""
    _need_cuda(x, w_interleaved)
    n, k = w_interleaved.shape
    m = x.shape[0]
    if (x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and x.dim() == 2 and m <= STREAM_MAX_ROWS and x.shape[1] == k
            and k % 8 == 0 and n % 16 == 0 and x.stride(1) == 1 and w_interleaved.stride(1) == 1 and x.stride(0) % 8 == 0
            and w_interleaved.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w_interleaved.data_ptr() % 16 == 0):
        return linear_stream(x, w_interleaved, swiglu=True)
    if (x.dtype == torch.bfloat16 and w_interleaved.dtype == torch.bfloat16 and m >= TCGEN05_MIN_ROWS and k % 8 == 0
            and n % 16 == 0 and x.stride(1) == 1 and w_interleaved.stride(1) == 1 and x.stride(0) % 8 == 0 and w_interleaved.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w_interleaved.data_ptr() % 16 == 0):
        return linear_tcgen05(x, w_interleaved, swiglu=True)   # many rows: our tcgen05 kernel with SwiGLU in its epilogue
    return swiglu(linear(x, w_interleaved), interleaved=True)


# ---------------------------------------------------------------------------------------
# attention over the paged cache
# ---------------------------------------------------------------------------------------
def attention_error_word(device: torch.device) -> torch.Tensor:
    """The int32 word the attention kernels set when a bounded wait for one of their TMA copies
    ran out (the output of that launch is then void).  Zero in every healthy run."""
    return _error_words(device)[1:2]


def attention_splits(num_rows: int, nkv: int, group: int, max_q: int, max_kv: int, sms: int) -> int:
    """How many key/value splits the tiled attention kernel uses for rows with more than 16
    packed query rows (tokens x group), on a device with ``sms`` multiprocessors.

    Steps with long rows (prefill) have enough query tiles to fill the GPU and use one; a few
    short portions over a long context are split so that two blocks per SM have work.  Rows
    of decoded tokens do not use this: their kernel cuts all rows' tiles into equal runs.
    """
    if max_q * group <= 16:
        return 1
    kv_tiles = max(1, -(-max_kv // 64))
    blocks = num_rows * nkv * -(-max_q * group // 64)
    if blocks >= sms or kv_tiles == 1:
        return 1
    return int(max(1, min(kv_tiles, 64, 2 * sms // blocks)))


def paged_attention(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    positions: torch.Tensor,
    token_row: torch.Tensor,
    q_start: torch.Tensor,
    kv_len: torch.Tensor,
    block_table: torch.Tensor,
    nq: int,
    max_q: int,
    max_kv: int,
    window: Optional[int] = None,
    scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    num_splits: Optional[int] = None,
    force_simple: bool = False,
    decode_blocks: Optional[int] = None,
    prefill_kernel: Optional[str] = None,
    row_tokens: Optional[Sequence[int]] = None,
    rows_alike: bool = False,
) -> torch.Tensor:
    """Causal attention of every token of a step over its request's pages.

    ``q``: ``[T, >= nq * d]`` (only the first ``nq * d`` columns of each row are read, so
    the fused qkv buffer can be passed as it is); pages ``[P, nkv, page_size, d]``;
    ``positions``/``token_row`` int32 ``[T]``; ``q_start`` int32 ``[rows + 1]``; ``kv_len``
    int32 ``[rows]`` (tokens each row holds after this step, so a row's first new token is
    at position ``kv_len - (q_start[r + 1] - q_start[r])``); ``block_table`` int32
    ``[rows, width]``; ``max_q``/``max_kv``: longest row and longest context (upper bounds
    are fine).  ``num_splits`` and ``decode_blocks`` override the split of long rows' keys and
    the number of blocks that share the decoded rows' tiles, ``prefill_kernel`` (``"tcgen05"`` or
    ``"mma"``) the kernel for rows of more than 16 packed query rows (for tests).
    ``row_tokens``: the rows' token counts on the host, if the caller has them: the kernel
    for prompt portions then launches blocks only for the rows that are its own (a step that
    mixes one portion with 63 decoded rows would otherwise start 63 rows of blocks that find
    nothing to do).  ``rows_alike``: the caller knows that the rows hold about equally many tokens;
    a step of a few decoded rows then gives every (row, KV head) pair a thread-block cluster of
    its own, whose blocks combine their results through distributed shared memory (right for any
    lengths, but slow if they differ much).  Returns ``[T, nq * d]``.

    bfloat16 with a head size that is a multiple of 16 up to 256 runs on the tensor cores
    (built per head size on first use): prompt portions on ``tcgen05.mma`` with the accumulators
    in tensor memory where the head size is 64 or 128 and a page holds a multiple of 64 keys,
    else on ``mma.sync``; decoded tokens on their own kernel.  float32, and other head sizes up
    to 512, take the plain kernel.
    """
    _need_cuda(q, k_pages, v_pages, positions, token_row, q_start, kv_len, block_table, out)
    _need(k_pages.dim() == 4 and k_pages.shape == v_pages.shape and k_pages.is_contiguous() and v_pages.is_contiguous(), "paged_attention: pages must be contiguous [P, nkv, page_size, d]")
    num_pages, nkv, page_size, d = k_pages.shape
    tokens = q.shape[0]
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= nq * d and q.dtype == k_pages.dtype, "paged_attention: q must be [T, >= nq * d] in the cache dtype")
    _need(nq % nkv == 0, f"paged_attention: {nq} query heads over {nkv} KV heads")
    for meta in (positions, token_row):
        _need(meta.dtype == torch.int32 and meta.is_contiguous() and meta.shape[0] >= tokens, "paged_attention: positions/token_row must be int32 [T]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(), "paged_attention: block_table must be contiguous int32 [rows, width]")
    rows = block_table.shape[0]
    _need(q_start.dtype == torch.int32 and q_start.is_contiguous() and q_start.shape[0] >= rows + 1, "paged_attention: q_start must be int32 [rows + 1]")
    _need(kv_len.dtype == torch.int32 and kv_len.is_contiguous() and kv_len.shape[0] >= rows, "paged_attention: kv_len must be int32 [rows]")
    if out is None:
        out = torch.empty((tokens, nq * d), dtype=q.dtype, device=q.device)
    _need(out.shape == (tokens, nq * d) and out.dtype == q.dtype and out.is_contiguous(), "paged_attention: out has the wrong shape or dtype")
    scale = 1.0 / math.sqrt(d) if scale is None else float(scale)
    _need(scale > 0, "paged_attention: the softmax scale must be positive")
    if q.dtype == torch.bfloat16 and d % 16 == 0 and d <= 256 and not force_simple:
        library = _library("attention_mma.cu", {"PYLON_HEAD_DIM": d})
        group = nq // nkv
        any_large = max_q * group > 16
        # Rows of decoded tokens can occur unless the step is one long row.
        maybe_small = not any_large or rows > 1
        if row_tokens is not None and len(row_tokens) == rows and all(count * group > 16 for count in row_tokens):
            maybe_small = False   # the host knows that every row is a prompt portion: no launch of the decode kernel
        # Prompt portions go to the tcgen05 kernel where it exists: head size 64 or 128, pages of a multiple of 64 keys.
        if prefill_kernel is None:
            prefill_kernel = "tcgen05" if d in (64, 128) and page_size % 64 == 0 and num_splits in (None, 1) else "mma"
        _need(prefill_kernel in ("tcgen05", "mma"), f"paged_attention: unknown prefill kernel {prefill_kernel!r}")
        use_tcgen05 = any_large and prefill_kernel == "tcgen05"
        if use_tcgen05:
            _need(d in (64, 128) and page_size % 64 == 0, "paged_attention: the tcgen05 kernel needs head size 64 or 128 and pages of a multiple of 64 keys")
            fast = _library("attention_tcgen05.cu", {"PYLON_HEAD_DIM": d})
            first_row, row_count = 0, rows
            if row_tokens is not None and len(row_tokens) == rows:
                large = [index for index, count in enumerate(row_tokens) if count * group > 16]
                if large and large[-1] - large[0] + 1 == len(large):   # one run of rows: the scheduler puts decoded rows first
                    first_row, row_count = large[0], len(large)
            _check(fast, fast.pylon_paged_attention_tcgen05(
                _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(q_start), _ptr(kv_len), _ptr(block_table),
                block_table.shape[1], page_size, num_pages, nq, nkv, int(window or 0), scale, first_row, row_count, int(max_q), int(maybe_small),
                _ptr(attention_error_word(q.device)), _stream()))
            if not maybe_small:
                return out
        splits = 1 if use_tcgen05 else (attention_splits(rows, nkv, group, max_q, max_kv, _multiprocessors(q.device)) if num_splits is None else int(num_splits))
        blocks = 0
        if maybe_small:
            blocks = library.pylon_attention_decode_blocks() if decode_blocks is None else int(decode_blocks)
            _need(blocks >= 1, "paged_attention: the decode kernel does not fit on this device")
        scratch = counters = None
        floats = library.pylon_attention_scratch_floats(splits, tokens, nq, rows, nkv, blocks)
        if floats:
            scratch = torch.empty((floats,), dtype=torch.float32, device=q.device)
        if blocks:
            counters = _zeroed_counters(q.device, "attention", rows * nkv)
        _check(library, library.pylon_paged_attention_mma(
            _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(scratch), _ptr(counters), _ptr(q_start), _ptr(kv_len),
            _ptr(block_table), block_table.shape[1], page_size, num_pages, nq, nkv, int(window or 0), scale, rows, tokens,
            int(max_q), splits, blocks, int(use_tcgen05), int(bool(rows_alike)), _ptr(attention_error_word(q.device)), _stream()))
        return out
    _need(d <= 512, f"paged_attention: head size {d} is larger than 512")
    library = _library("attention_simple.cu")
    _check(library, library.pylon_paged_attention_simple(
        _ptr(q), q.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(out), _ptr(positions), _ptr(token_row), _ptr(block_table),
        block_table.shape[1], page_size, num_pages, nq, nkv, d, int(window or 0), scale, tokens, _dtype_code(q.dtype), _stream()))
    return out


# ---------------------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------------------
def sample(
    logits: torch.Tensor,
    temperature: Optional[torch.Tensor] = None,
    top_p: Optional[torch.Tensor] = None,
    uniform: Optional[torch.Tensor] = None,
    out: Optional[torch.Tensor] = None,
    host_copy: Optional[torch.Tensor] = None,
) -> torch.Tensor:
    """One token per row of float32 ``logits [R, vocab]``: arg-max where a row's temperature
    is 0 (or none is given), else a draw from ``softmax(logits / T)`` cut to the ``top_p``
    nucleus, using the row's number from ``uniform`` (float32 in [0, 1)).  The per-row parameters may lie in pinned
    host memory, which the kernel then reads where it is.  ``host_copy``: int32 ``[R + 4]`` in pinned host memory, into
    which the kernel also writes the tokens and, behind them, the kernels' four error words as they stand: whoever
    waits for the launch can read both there, and no copy has to follow it."""
    _need_cuda(logits, out)
    _need(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: logits must be float32 [R, vocab]")
    rows, vocab = logits.shape
    for per_row in (temperature, top_p, uniform):
        if per_row is not None:
            _need(per_row.dtype == torch.float32 and per_row.is_contiguous() and per_row.shape[0] >= rows
                  and (per_row.is_cuda or per_row.is_pinned()), "sample: per-row parameters must be float32 [R] on the device or in pinned memory")
    words = None
    if host_copy is not None:
        _need(host_copy.dtype == torch.int32 and host_copy.is_contiguous() and host_copy.shape == (rows + 4,) and host_copy.is_pinned(),
              "sample: host_copy must be int32 [R + 4] in pinned memory")
        words = _error_words(logits.device)
    if out is None:
        out = torch.empty((rows,), dtype=torch.int32, device=logits.device)
    _need(out.dtype == torch.int32 and out.is_contiguous() and out.shape[0] >= rows, "sample: out must be int32 [R]")
    library = _library("sampling.cu")
    _check(library, library.pylon_sample(
        _ptr(logits), logits.stride(0), rows, vocab, _ptr(temperature), _ptr(top_p), _ptr(uniform), _ptr(out),
        None if host_copy is None else host_copy.data_ptr(), _ptr(words), None if host_copy is None else host_copy.data_ptr() + 4 * rows, _stream()))
    return out
