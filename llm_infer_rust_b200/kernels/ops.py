"""The engine's operations: thin checked wrappers over the package's CUDA kernels.

Every function takes CUDA tensors and launches on the current stream.  There
is no CPU path and no silent fallback: a CPU tensor, an unsupported dtype or a
refused size raises.  Matrix products of the bfloat16 engine go to cuBLAS
through ``torch.mm`` (the reference uses the same library for them:
src/layers/linear.rs:5-7); everything else is this package's own code.
"""
from __future__ import annotations

import contextlib
import ctypes
import gc
import os
import sys
from typing import Optional

import torch

from .build import load_cuda_library

F32, BF16 = 0, 1
_CODES = {torch.float32: F32, torch.bfloat16: BF16}
ERROR_BITS = {1: "a token id outside the embedding table", 2: "a cache slot outside the pool",
              4: "a position beyond the rotary table", 8: "sampling found no valid token",
              16: "a bounded wait inside a kernel ran out"}
_RC = {-1: "unsupported dtype", -2: "a size the kernel refuses", -3: "misaligned pointer"}


class KernelError(RuntimeError):
    pass


def _code(t: torch.Tensor) -> int:
    try:
        return _CODES[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not supported (float32 and bfloat16 are)") from None


def _cuda(*tensors: Optional[torch.Tensor]) -> None:
    """Checks that the operands are on the device.  Every wrapper that launches calls this first, so it is also
    where products that wait in the chain (see ``chain_linear``) are launched: whatever runs next may read them."""
    flush_chain()
    _cuda_only(*tensors)


def _cuda_only(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("the kernels run on CUDA tensors only; there is no CPU path")


def _contig(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_contiguous():
            raise KernelError("a kernel was given a non-contiguous tensor")


def _p(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


# Launches of this package's kernels so far (library matrix products are not counted).
_launches = [0]


def launch_count() -> int:
    return _launches[0]


def add_launches(n: int) -> None:
    """Account for kernels that ran without passing through a wrapper (a replayed graph)."""
    _launches[0] += n


def _ok(rc: int, name: str, kernels: int = 1) -> None:
    if rc == 0:
        _launches[0] += kernels
        return
    if rc in _RC:
        raise KernelError(f"{name}: {_RC[rc]}")
    raise KernelError(f"{name}: CUDA error {rc} at launch")


# --------------------------------------------------------------------------- error word
_error_words = {}


def error_word(device: torch.device) -> torch.Tensor:
    """The device word into which kernels OR their error bits."""
    key = torch.device(device).index or 0
    if key not in _error_words:
        _error_words[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _error_words[key]


def check_errors(device: torch.device) -> None:
    """Read the error word (synchronises) and raise if a kernel flagged a fault."""
    flush_chain()
    word = error_word(device)
    value = int(word.item())
    if value:
        word.zero_()
        _reset_chain_state(device)
        what = [text for bit, text in ERROR_BITS.items() if value & bit]
        raise KernelError("a kernel refused an access: " + "; ".join(what))


_staging = {}


class PendingRead:
    """Token ids and the error word on their way to the host: ``begin_read`` enqueues the copies and an event,
    ``finish`` waits for that event only, so kernels enqueued after ``begin_read`` keep the GPU busy meanwhile."""

    def __init__(self, buf, n, event, device):
        self.buf, self.n, self.event, self.device = buf, n, event, device

    def finish(self) -> list:
        self.event.synchronize()
        value = int(self.buf[self.n])
        if value:
            error_word(self.device).zero_()
            _reset_chain_state(self.device)
            what = [text for bit, text in ERROR_BITS.items() if value & bit]
            raise KernelError("a kernel refused an access: " + "; ".join(what))
        return self.buf[:self.n].tolist()


def begin_read(ids: torch.Tensor) -> PendingRead:
    """Start copying ``ids`` (int32, on the device) and the error word into pinned memory (two small copies on
    the current stream, then an event).  Four staging buffers per device take turns: at most three reads may be
    pending when a fourth begins."""
    flush_chain()
    device = ids.device
    key = device.index or 0
    n = ids.numel()
    ring = _staging.get(key)
    if ring is None or ring[0][0].numel() < n + 1:
        size = max(1024, 2 * (n + 1))
        ring = _staging[key] = ([torch.empty(size, dtype=torch.int32).pin_memory() for _ in range(4)], [0])
    bufs, turn = ring
    buf = bufs[turn[0] % len(bufs)]
    turn[0] += 1
    buf[:n].copy_(ids.reshape(-1), non_blocking=True)
    buf[n:n + 1].copy_(error_word(device), non_blocking=True)
    event = torch.cuda.Event()
    event.record(torch.cuda.current_stream(device))
    return PendingRead(buf, n, event, device)


# --------------------------------------------------------------------------- libraries
def _elementwise():
    return load_cuda_library("elementwise.cu")


def padded_head_dim(head_dim: int) -> int:
    """The compile-time head size of the all-sizes attention kernels for a real head size: the next multiple of 16."""
    return -(-head_dim // 16) * 16


def _attention(head_dim: int):
    """The all-sizes attention library for a real head size (any even number up to 512)."""
    if head_dim % 2 != 0 or not 2 <= head_dim <= 512:
        raise KernelError(f"head size {head_dim} is refused: the attention kernels take even head sizes up to 512")
    return load_cuda_library("attention.cu", {"HEAD_DIM": padded_head_dim(head_dim)})


# --------------------------------------------------------------------------- element-wise
def embedding(ids: torch.Tensor, table: torch.Tensor, out_dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    """out[t] = table[ids[t]] * scale (the product in float, rounded once to ``out_dtype``)."""
    _cuda(ids, table)
    _contig(ids, table)
    if ids.dtype != torch.int32:
        raise KernelError("token ids must be int32")
    out = torch.empty((ids.numel(), table.shape[1]), dtype=out_dtype, device=table.device)
    rc = _elementwise().b200_embedding(_p(out), _p(table), _p(ids), ids.numel(), table.shape[1],
                                       table.shape[0], ctypes.c_float(scale), _code(out), _code(table),
                                       _p(error_word(table.device)), _stream())
    _ok(rc, "embedding")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: Optional[torch.Tensor] = None,
             rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = rms_norm(x[rows[r]]) * weight (rows None: every row, in place allowed)."""
    return _norm(x, None, weight, eps, out, rows, False)


def add_rms_norm(x: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, eps: float,
                 out: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
                 write_residual: bool = True) -> torch.Tensor:
    """s = x + residual in float; residual <- round(s); out = rms_norm(s) * weight."""
    return _norm(x, residual, weight, eps, out, rows, write_residual)


def _norm(x, residual, weight, eps, out, rows, write_residual):
    _cuda(x, residual, weight, out, rows)
    _contig(x, residual, weight, out, rows)
    width = x.shape[-1]
    if weight.numel() != width:
        raise KernelError(f"norm weight has {weight.numel()} elements, the rows have {width}")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
        raise KernelError("the residual must have the shape and dtype of x")
    n = x.numel() // width if rows is None else rows.numel()
    if rows is not None and rows.dtype != torch.int32:
        raise KernelError("row indices must be int32")
    if out is None:
        out = torch.empty((n, width), dtype=x.dtype, device=x.device)
    elif out.dtype != x.dtype or out.numel() != n * width:
        raise KernelError("norm output has the wrong dtype or size")
    rc = _elementwise().b200_rms_norm(_p(out), _p(x), _p(residual), _p(weight), _p(rows), n, width,
                                      ctypes.c_float(eps), int(bool(write_residual)), _code(x),
                                      _code(weight), _stream())
    _ok(rc, "rms_norm")
    return out


def silu_mul(gate_up: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""
    _cuda(gate_up, out)
    _contig(gate_up, out)
    tokens, width2 = gate_up.shape
    if width2 % 2:
        raise KernelError("silu_mul needs an even width")
    if out is None:
        out = torch.empty((tokens, width2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    rc = _elementwise().b200_silu_mul(_p(out), _p(gate_up), tokens, width2 // 2, _code(gate_up), _stream())
    _ok(rc, "silu_mul")
    return out


def cast(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    _cuda(x)
    _contig(x)
    if x.dtype == dtype:
        return x
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    rc = _elementwise().b200_cast(_p(out), _p(x), ctypes.c_longlong(x.numel()), _code(out), _code(x), _stream())
    _ok(rc, "cast")
    return out


def scale_floats(z: torch.Tensor, scale: float) -> torch.Tensor:
    """z <- z * scale in place on a contiguous float32 tensor."""
    _cuda(z)
    _contig(z)
    _f32(z)
    rc = _elementwise().b200_scale_floats(_p(z), ctypes.c_longlong(z.numel()), ctypes.c_float(scale), _stream())
    _ok(rc, "scale_floats")
    return z


# --------------------------------------------------------------------------- between QKV and attention
def qkv_post(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
             v_cache: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
             k_weight: Optional[torch.Tensor], eps: float, cos: Optional[torch.Tensor],
             sin: Optional[torch.Tensor], rot_dim: int, positions: torch.Tensor,
             slots: Optional[torch.Tensor], num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Per-head norm, rotary encoding, cache store.  ``slots`` None: nothing is stored."""
    _cuda(qkv, q_out, k_cache, v_cache, q_weight, k_weight, cos, sin, positions, slots)
    _contig(qkv, q_out, k_cache, v_cache, q_weight, k_weight, cos, sin, positions, slots)
    tokens = qkv.shape[0]
    if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelError("qkv width does not match the head counts")
    if slots is not None and (k_cache is None or k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype):
        raise KernelError("the cache must have the activations' dtype")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("q and k norm weights come together")
    if cos is not None and (cos.dtype != torch.float32 or sin.dtype != torch.float32):
        raise KernelError("rotary tables must be float32")
    wcode = _code(q_weight) if q_weight is not None else _code(qkv)
    if q_weight is not None and k_weight.dtype != q_weight.dtype:
        raise KernelError("q and k norm weights must share a dtype")
    # cache tensors are [pages + 1, kv_heads, page_size, head_dim]
    page_size = 1 if k_cache is None else k_cache.shape[2]
    cache_slots = 0 if k_cache is None else k_cache.shape[0] * k_cache.shape[2]
    if k_cache is not None and (k_cache.shape[1] != num_kv_heads or k_cache.shape[3] != head_dim):
        raise KernelError("the cache must be [pages + 1, kv_heads, page_size, head_dim]")
    max_pos = 0 if cos is None else cos.shape[0]
    lib = load_cuda_library("qkv_post.cu")
    rc = lib.b200_qkv_post(_p(qkv), _p(q_out), _p(k_cache), _p(v_cache), _p(q_weight), _p(k_weight),
                           ctypes.c_float(eps), _p(cos), _p(sin), rot_dim, max_pos, _p(positions), _p(slots),
                           tokens, num_heads, num_kv_heads, head_dim, page_size, ctypes.c_longlong(cache_slots),
                           _code(qkv), wcode, _p(error_word(qkv.device)), _stream())
    _ok(rc, "qkv_post")


# --------------------------------------------------------------------------- attention
def tcgen05_attention_launches() -> tuple:
    """(launches of the one-tile kernel, launches of the two-tile kernel) of the tcgen05 prefill attention so far."""
    lib = load_cuda_library("attention_tcgen05.cu")
    lib.b200_attention_tcgen05_launches.restype = ctypes.c_longlong
    return int(lib.b200_attention_tcgen05_launches(0)), int(lib.b200_attention_tcgen05_launches(1))


def prefill_attention(q, k_cache, v_cache, out, block_table, cu_q, kv_len, prefix_len, rows, n_rows,
                      max_q_len, num_heads, num_kv_heads, head_dim, page_size, window, scale,
                      tiles_per_cta: int = 0, v_head_dim: Optional[int] = None, softcap: float = 0.0,
                      precise_weights: bool = False, chunk: Optional[int] = None,
                      sinks: Optional[torch.Tensor] = None, shared_values: bool = False) -> None:
    """Causal attention of prompt portions over the paged cache (rows: which batch rows).

    ``v_head_dim``: the width of a value (and of an output) vector where it differs from a key's;
    ``softcap`` > 0: a score becomes cap * tanh(score / cap) before the mask; ``precise_weights``: the softmax
    weights enter the product with the values as two bfloat16 terms (about 16 bits) instead of one.  Values of
    another width than keys take the all-sizes kernel, whose weights are floats; a soft-cap or precise weights take
    the mma.sync kernel, not the tcgen05 one (whose weights are single bfloat16 numbers in tensor memory).

    ``chunk`` C: a query at position p sees only keys from p - p % C on (its own block of C positions, counted from
    the sequence's start); ``sinks`` (float32, one per query head): exp(sink) joins the softmax's denominator.  Both
    are served by the mma.sync and the all-sizes kernels, not by the tcgen05 one.  ``shared_values``: one KV head
    whose values are the first ``v_head_dim`` columns of the key rows (``v_cache`` is not read and may be None): the
    mma.sync kernels fetch a block's rows once for both products and take the values in column tiles.

    ``tiles_per_cta`` (head size 128 on the tcgen05 kernel only): 1 or 2 tiles of 128 query vectors per
    CTA, 0 lets the kernel's launcher choose by the size of the grid."""
    _cuda(q, k_cache, v_cache, out, block_table, cu_q, kv_len, prefix_len, rows, sinks)
    _contig(q, k_cache, v_cache, out, block_table, sinks)
    if n_rows == 0:
        return
    if k_cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("q, cache and output must share a dtype")
    dv = int(v_head_dim or head_dim)
    cap = float(softcap or 0.0)
    _check_sinks(sinks, num_heads)
    plain_mask = not chunk and sinks is None
    if shared_values:
        if num_kv_heads != 1 or k_cache.shape[1] != 1:
            raise KernelError("values that are columns of the key rows need one KV head")
        if latent_uses_tensor_cores(q.dtype, num_heads, head_dim, dv, page_size):
            tile, group = shared_value_tile(dv), latent_head_group(num_heads)
            lib = _attention_mma(head_dim, tile)
            kmap = kv_tensor_map(k_cache, min(page_size, 32), lib)
            for col0 in range(0, dv, tile):
                rc = lib.b200_prefill_attention_mma(
                    _p(q), kmap, kmap, _p(out), _p(block_table), block_table.shape[-1], _p(cu_q), _p(kv_len),
                    _p(prefix_len), _p(rows), n_rows, max_q_len, num_heads, num_heads // group, page_size,
                    int(window or 0), ctypes.c_float(scale), ctypes.c_float(cap), int(bool(precise_weights)),
                    int(chunk or 0), _p(sinks), col0, dv, col0, _p(error_word(q.device)), _stream())
                _ok(rc, "prefill_attention_mma_shared")
            return
        v_cache = k_cache
    if not shared_values and dv == head_dim and decode_uses_tensor_cores(q.dtype, num_heads, num_kv_heads, head_dim, page_size):
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[2] != page_size:
            raise KernelError("the cache must be [pages + 1, kv_heads, page_size, head_dim]")
        box_rows = min(page_size, 32)
        group = num_heads // num_kv_heads
        if head_dim == 128 and 128 % group == 0 and max_q_len * group >= 128 and not cap > 0.0 and not precise_weights \
                and plain_mask:
            # head size 128 and at least one full tile of 128 query vectors: the tcgen05 kernel
            rc = load_cuda_library("attention_tcgen05.cu").b200_prefill_attention_tcgen05(
                _p(q), kv_tensor_map(k_cache, box_rows), kv_tensor_map(v_cache, box_rows), _p(out), _p(block_table),
                block_table.shape[-1], _p(cu_q), _p(kv_len), _p(prefix_len), _p(rows), n_rows, max_q_len, num_heads,
                num_kv_heads, page_size, int(window or 0), ctypes.c_float(scale), int(tiles_per_cta),
                _p(error_word(q.device)), _stream())
            _ok(rc, "prefill_attention_tcgen05")
            return
        rc = _attention_mma(head_dim).b200_prefill_attention_mma(
            _p(q), kv_tensor_map(k_cache, box_rows), kv_tensor_map(v_cache, box_rows), _p(out), _p(block_table),
            block_table.shape[-1], _p(cu_q), _p(kv_len), _p(prefix_len), _p(rows), n_rows, max_q_len, num_heads,
            num_kv_heads, page_size, int(window or 0), ctypes.c_float(scale), ctypes.c_float(cap),
            int(bool(precise_weights)), int(chunk or 0), _p(sinks), 0, 0, 0, _p(error_word(q.device)), _stream())
        _ok(rc, "prefill_attention_mma")
        return
    rc = _attention(max(head_dim, dv)).b200_prefill_attention(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(block_table), block_table.shape[-1], _p(cu_q),
        _p(kv_len), _p(prefix_len), _p(rows), n_rows, max_q_len, num_heads, num_kv_heads, page_size,
        int(window or 0), ctypes.c_float(scale), _code(q), head_dim, dv, ctypes.c_float(cap), int(chunk or 0),
        _p(sinks), head_dim if shared_values else 0, _stream())
    _ok(rc, "prefill_attention")


def _check_sinks(sinks: Optional[torch.Tensor], num_heads: int) -> None:
    if sinks is not None and (sinks.dtype != torch.float32 or sinks.numel() != num_heads):
        raise KernelError("sinks must be float32, one per query head")


MMA_MAX_GROUP = 16
MMA_MAX_HEAD_DIM = 256


def _attention_mma(head_dim: int, shared_value_tile: Optional[int] = None):
    """The tensor-core attention library for a head size; ``shared_value_tile``: the form whose values are a range of
    that many columns of the key rows."""
    if shared_value_tile:
        return load_cuda_library("attention_mma.cu", {"HEAD_DIM": head_dim, "V_DIM": shared_value_tile, "V_SHARED": 1})
    return load_cuda_library("attention_mma.cu", {"HEAD_DIM": head_dim})


def shared_value_tile(value_dim: int) -> int:
    """Columns of the values that one launch of the shared-row tensor-core kernels takes: the largest multiple of 16 up
    to 256 that divides ``value_dim`` (0: none)."""
    return next((t for t in range(256, 15, -16) if value_dim % t == 0), 0)


def latent_head_group(num_heads: int) -> int:
    """Query heads that one CTA of the shared-row kernels serves: the largest divisor of ``num_heads`` up to 16."""
    return next(g for g in range(min(MMA_MAX_GROUP, num_heads), 0, -1) if num_heads % g == 0)


def latent_uses_tensor_cores(dtype: torch.dtype, num_heads: int, key_dim: int, value_dim: int, page_size: int) -> bool:
    """bfloat16 key rows of a multiple of 16 up to 512 columns whose leading ``value_dim`` columns are the values, cut
    into tiles of a multiple of 16, pages of a power of two."""
    return (dtype == torch.bfloat16 and key_dim % 16 == 0 and key_dim <= 512 and value_dim <= key_dim
            and shared_value_tile(value_dim) > 0 and page_size > 0 and page_size & (page_size - 1) == 0)


def decode_uses_tensor_cores(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int,
                             page_size: int) -> bool:
    """bfloat16 caches with at most 16 query heads per KV head, heads up to 256 wide and a page size
    that is a power of two take the TMA / tensor-core kernel; everything else the all-sizes kernel."""
    return (dtype == torch.bfloat16 and num_heads // num_kv_heads <= MMA_MAX_GROUP
            and head_dim <= MMA_MAX_HEAD_DIM and head_dim % 16 == 0
            and page_size > 0 and page_size & (page_size - 1) == 0)


_kv_maps = {}


def kv_tensor_map(cache: torch.Tensor, box_rows: int, lib=None):
    """The 128-byte TMA descriptor of a cache tensor [pages + 1, kv_heads, page_size, head_dim] (made once)."""
    key = (cache.data_ptr(), tuple(cache.shape), box_rows)
    buf = _kv_maps.get(key)
    if buf is None:
        if cache.dtype != torch.bfloat16 or not cache.is_contiguous() or cache.dim() != 4:
            raise KernelError("a TMA descriptor needs a contiguous bfloat16 cache [pages + 1, kv_heads, page_size, head_dim]")
        buf = ctypes.create_string_buffer(128)
        rows = cache.shape[0] * cache.shape[1] * cache.shape[2]
        rc = (lib or _attention_mma(cache.shape[3])).b200_kv_tensor_map(buf, _p(cache), ctypes.c_longlong(rows), box_rows)
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a cache tensor could not be made (code {rc})")
        if len(_kv_maps) > 4096:
            _kv_maps.clear()
        _kv_maps[key] = buf
    return buf


def decode_ctas_per_split(dtype: torch.dtype, n_rows: int, num_heads: int, num_kv_heads: int, head_dim: int,
                          page_size: int, plain: bool = True) -> int:
    """CTAs that the decode kernel launches for each split of the keys (``plain``: values as wide as keys, the
    case the tensor-core kernel takes)."""
    if plain and decode_uses_tensor_cores(dtype, num_heads, num_kv_heads, head_dim, page_size):
        return n_rows * num_kv_heads
    return n_rows * num_kv_heads * ((num_heads // num_kv_heads + 3) // 4)


def decode_scratch_floats(n_rows: int, num_heads: int, head_dim: int, splits: int) -> int:
    """Floats of scratch that decode attention needs (partial outputs are rows of the padded head size)."""
    return 0 if splits <= 1 else n_rows * num_heads * splits * (padded_head_dim(head_dim) + 2)


def decode_attention(q, k_cache, v_cache, out, scratch, block_table, cu_q, kv_len, rows, n_rows,
                     num_heads, num_kv_heads, head_dim, page_size, window, scale, splits,
                     v_head_dim: Optional[int] = None, softcap: float = 0.0, precise_weights: bool = False,
                     chunk: Optional[int] = None, sinks: Optional[torch.Tensor] = None,
                     shared_values: bool = False) -> None:
    """Attention of single decoded tokens, the keys split over ``splits`` blocks per row (``v_head_dim``,
    ``softcap``, ``precise_weights``, ``chunk``, ``sinks``, ``shared_values``: see ``prefill_attention``)."""
    _cuda(q, k_cache, v_cache, out, scratch, block_table, cu_q, kv_len, rows, sinks)
    _contig(q, k_cache, v_cache, out, block_table, scratch, sinks)
    _check_sinks(sinks, num_heads)
    if n_rows == 0:
        return
    if k_cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("q, cache and output must share a dtype")
    dv = int(v_head_dim or head_dim)
    plain = dv == head_dim and not shared_values
    need = decode_scratch_floats(n_rows, num_heads, max(head_dim, dv), splits)
    if need and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need):
        raise KernelError(f"decode attention needs {need} floats of scratch")
    if shared_values:
        if num_kv_heads != 1 or k_cache.shape[1] != 1:
            raise KernelError("values that are columns of the key rows need one KV head")
        if latent_uses_tensor_cores(q.dtype, num_heads, head_dim, dv, page_size):
            tile, group = shared_value_tile(dv), latent_head_group(num_heads)
            lib = _attention_mma(head_dim, tile)
            kmap = kv_tensor_map(k_cache, min(page_size, 32), lib)
            groups = num_heads // group
            in_kernel = splits == 1 or (splits in (2, 4, 8) and splits * groups * n_rows <= _sm_count(q.device))
            for col0 in range(0, dv, tile):
                rc = lib.b200_decode_attention_mma(
                    _p(q), kmap, kmap, _p(out), _p(scratch), _p(block_table), block_table.shape[-1], _p(cu_q),
                    _p(kv_len), _p(rows), n_rows, num_heads, groups, page_size, int(window or 0),
                    ctypes.c_float(scale), splits, ctypes.c_float(softcap or 0.0), int(bool(precise_weights)),
                    int(chunk or 0), _p(sinks), col0, dv, col0, _p(error_word(q.device)), _stream())
                _ok(rc, "decode_attention_mma_shared", 1 if in_kernel else 2)
            return
        v_cache = k_cache
    if plain and decode_uses_tensor_cores(q.dtype, num_heads, num_kv_heads, head_dim, page_size):
        if k_cache.shape[1] != num_kv_heads or k_cache.shape[2] != page_size:
            raise KernelError("the cache must be [pages + 1, kv_heads, page_size, head_dim]")
        box_rows = min(page_size, 32)
        rc = _attention_mma(head_dim).b200_decode_attention_mma(
            _p(q), kv_tensor_map(k_cache, box_rows), kv_tensor_map(v_cache, box_rows), _p(out), _p(scratch), _p(block_table), block_table.shape[-1],
            _p(cu_q), _p(kv_len), _p(rows), n_rows, num_heads, num_kv_heads, page_size, int(window or 0),
            ctypes.c_float(scale), splits, ctypes.c_float(softcap or 0.0), int(bool(precise_weights)),
            int(chunk or 0), _p(sinks), 0, 0, 0, _p(error_word(q.device)), _stream())
        in_kernel = splits == 1 or (splits in (2, 4, 8) and splits * num_kv_heads * n_rows <= _sm_count(q.device))
        _ok(rc, "decode_attention_mma", 1 if in_kernel else 2)      # (a cluster of 2, 4 or 8 splits combines them itself)
        return
    rc = _attention(max(head_dim, dv)).b200_decode_attention(
        _p(q), _p(k_cache), _p(v_cache), _p(out), _p(scratch), _p(block_table), block_table.shape[-1],
        _p(cu_q), _p(kv_len), _p(rows), n_rows, num_heads, num_kv_heads, page_size, int(window or 0),
        ctypes.c_float(scale), splits, _code(q), head_dim, dv, ctypes.c_float(softcap or 0.0), int(chunk or 0),
        _p(sinks), head_dim if shared_values else 0, _stream())
    _ok(rc, "decode_attention", 2 if splits > 1 else 1)


# --------------------------------------------------------------------------- few-row products with fused ends
SKINNY_MAX_ROWS = 16
EPI_PLAIN_BF16, EPI_PLAIN_F32, EPI_SWIGLU, EPI_QKV = 0, 1, 2, 3


class _SkinnyParams(ctypes.Structure):
    """Mirror of ``SkinnyParams`` in csrc/skinny_linear.cu (same order, native alignment)."""
    _fields_ = [("x", ctypes.c_void_p), ("x_rows", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("residual_out", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("norm_w_f32", ctypes.c_int),
                ("eps", ctypes.c_float), ("M", ctypes.c_int), ("N", ctypes.c_int), ("K", ctypes.c_int),
                ("ksplit", ctypes.c_int), ("mode", ctypes.c_int), ("out", ctypes.c_void_p),
                ("nh", ctypes.c_int), ("nkv", ctypes.c_int), ("rot_dim", ctypes.c_int), ("max_pos", ctypes.c_int),
                ("page_size", ctypes.c_int), ("cache_slots", ctypes.c_longlong), ("qk_eps", ctypes.c_float),
                ("q_w", ctypes.c_void_p), ("k_w", ctypes.c_void_p), ("qk_w_f32", ctypes.c_int),
                ("cos_table", ctypes.c_void_p), ("sin_table", ctypes.c_void_p), ("positions", ctypes.c_void_p),
                ("slots", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("err", ctypes.c_void_p), ("post_residual", ctypes.c_void_p), ("post_sum_out", ctypes.c_void_p),
                ("post_stats", ctypes.c_void_p), ("stats_in", ctypes.c_void_p), ("stats_tiles", ctypes.c_int),
                ("trace", ctypes.c_void_p), ("inv_freq", ctypes.c_void_p), ("qkv_flags", ctypes.c_int)]


# For tuning: an int64 tensor [4096, 32] on the device; the first thread of every CTA of the next single-product
# launches then leaves the nanosecond clock there at the kernel's phases (0 start, 1 dependency wait over, 2 x staged,
# 3 products done, 4 own sums stored, 5 the cluster's sums have met, 6 a rank other than 0 leaves, 7 epilogue done),
# and in slots 16 to 31 the SM's cycle counter at the same places.
skinny_trace: Optional[torch.Tensor] = None


class PendingNorm:
    """An RMSNorm (with or without a residual add before it) that has not run: the product that consumes it runs
    it as its prologue.

    ``residual`` None: the plain norm of ``x``.  ``residual_out`` is the tensor that will hold the rounded sum
    (None: the sum is not kept).  ``materialize()`` runs the norm as a kernel of its own, for a consumer that
    cannot fuse it.
    """

    def __init__(self, x, residual, weight, eps, rows=None, write_residual=True):
        self.x, self.residual, self.weight, self.eps, self.rows = x, residual, weight, float(eps), rows
        self.residual_out = torch.empty_like(residual) if write_residual and residual is not None else None
        self.dtype, self.device = x.dtype, x.device
        n = x.shape[0] if rows is None else rows.numel()
        self.shape = (n, x.shape[-1])

    def materialize(self) -> torch.Tensor:
        if self.residual is None:
            return rms_norm(self.x, self.weight, self.eps, rows=self.rows)
        if self.residual_out is not None:
            flush_chain()
            self.residual_out.copy_(self.residual)
            return add_rms_norm(self.x, self.residual_out, self.weight, self.eps, rows=self.rows)
        return add_rms_norm(self.x, self.residual, self.weight, self.eps, rows=self.rows, write_residual=False)


_weight_maps = {}
_sm_counts = {}


def _sm_count(device) -> int:
    key = torch.device(device).index or 0
    if key not in _sm_counts:
        _sm_counts[key] = torch.cuda.get_device_properties(device).multi_processor_count
    return _sm_counts[key]


def _skinny(qkv_forms: bool = False):
    # (with a trace buffer set, the build that stamps its clocks: a tuning aid, compiled when first asked for;
    # ``qkv_forms``: the build whose QKV epilogue knows the further forms, which the dense models' build leaves out)
    defines = {}
    if skinny_trace is not None:
        defines["SKINNY_TRACE"] = 1
    if qkv_forms:
        defines["SKINNY_QKV_FORMS"] = 1
    lib = load_cuda_library("skinny_linear.cu", defines or None)
    if not getattr(lib, "_checked", False):
        if lib.b200_skinny_params_size() != ctypes.sizeof(_SkinnyParams):
            raise KernelError("the parameter block of skinny_linear.cu and its Python mirror differ")
        lib._checked = True
    return lib


def _weight_map(weight: torch.Tensor, box_rows: int):
    key = (weight.data_ptr(), tuple(weight.shape), box_rows)
    buf = _weight_maps.get(key)
    if buf is None:
        buf = ctypes.create_string_buffer(128)
        rc = _skinny().b200_weight_tensor_map(buf, _p(weight), ctypes.c_longlong(weight.shape[0]),
                                              ctypes.c_longlong(weight.shape[1]), box_rows)
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a weight matrix could not be made (code {rc})")
        if len(_weight_maps) > 8192:
            _weight_maps.clear()
        _weight_maps[key] = buf
    return buf


def skinny_ok(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
              head_dim: int = 0) -> bool:
    """Whether the few-row kernel takes this product: bfloat16 activations and weight, at most 16 rows,
    K a multiple of 8 and at most 8 x 4032 (8 rows) or 8 x 1984 (16 rows); QKV: head size 64, 128 or 256."""
    if act_dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.dim() != 2:
        return False
    k = weight.shape[1]
    if not 0 < rows <= SKINNY_MAX_ROWS or k % 8 or not weight.is_contiguous() or weight.data_ptr() % 16:
        return False
    if k > 8 * (4032 if rows <= 8 else 1984):
        return False
    if mode == EPI_QKV and head_dim not in (64, 128, 256):
        return False
    if mode == EPI_SWIGLU and weight.shape[0] % 2:
        return False
    return True


@contextlib.contextmanager
def graph_capture(graph: "torch.cuda.CUDAGraph"):
    """Capture the stream's work into ``graph``.

    Python's cycle collector runs first and is held off until the capture has ended.  A dead reference cycle that
    owns CUDA graphs or device memory (an engine that the caller dropped, say) is else freed at whatever allocation
    inside the capture happens to start a collection; destroying a graph or returning its memory is not permitted
    while a stream captures, and the capture ends with "operation failed due to a previous error during capture"."""
    flush_chain()
    gc.collect()
    held = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            yield
            flush_chain()
    finally:
        if held:
            gc.enable()


def skinny_linear(x, weight: torch.Tensor, mode: int = EPI_PLAIN_BF16, x_rows: Optional[torch.Tensor] = None,
                  qkv: Optional[dict] = None, out: Optional[torch.Tensor] = None, norm_after=None,
                  stats=None) -> torch.Tensor:
    """epilogue(prologue(x) . weight^T) for at most 16 rows, in one kernel.

    ``out``: the tensor to fill (PLAIN and SWIGLU; made here when None).  ``norm_after`` = (residual, sum_out,
    stats): a PLAIN bfloat16 product also begins the add + RMSNorm that follows it: round(y + residual) goes to
    ``sum_out`` and the sums of squares per tile of columns to ``stats`` (float32 [tiles, 16]).  ``stats`` =
    (that tensor, tiles): a product whose ``x`` is a ``PendingNorm`` of such a y and residual takes the rows'
    statistics from there and reads only its own columns (``residual_out`` is then not written: it is ``sum_out``).

    ``x``: a bfloat16 tensor [rows, K], or a ``PendingNorm`` (then the residual add and the norm run as the
    prologue and ``x.residual_out`` is filled).  ``mode``: EPI_PLAIN_BF16 / EPI_PLAIN_F32: the product;
    EPI_SWIGLU: silu(gate) * up for a weight of gate rows then up rows; EPI_QKV: per-head norm, rotary
    encoding and the cache store, with ``qkv`` = the keyword arguments of ``qkv_post`` (without ``qkv``);
    the result is then ``q_out``.  Further keys of ``qkv``: ``inv_freq`` (float32 [rot_dim / 2]: angles are
    position * inv_freq, their cosines and sines taken in the kernel, instead of the tables ``cos`` / ``sin``),
    ``plain_norm`` (q and k heads normed without weights), ``norm_after_rotation``, ``values_are_keys`` (the weight
    holds q and k heads only and a key head's product, as it comes out, is also stored as the token's value).
    """
    _flush_held()
    if isinstance(x, PendingNorm) and x.residual is None:
        x = x.materialize()                                    # (this kernel's prologue always adds a residual)
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    _cuda(src, weight, rows_t)
    _contig(src, weight, rows_t)
    m = src.shape[0] if rows_t is None else rows_t.numel()
    n, k = weight.shape
    if src.shape[-1] != k:
        raise KernelError(f"the rows have {src.shape[-1]} columns, the weight has {k}")
    head_dim = qkv["head_dim"] if qkv else 0
    if not skinny_ok(m, weight, src.dtype, mode, head_dim):
        raise KernelError("the few-row product refuses this size or dtype")
    lib = _skinny(qkv_forms=bool(qkv) and (qkv.get("inv_freq") is not None or bool(qkv.get("plain_norm"))
                                           or bool(qkv.get("norm_after_rotation")) or bool(qkv.get("values_are_keys"))))
    P = _SkinnyParams()
    P.x, P.x_rows = src.data_ptr(), (0 if rows_t is None else rows_t.data_ptr())
    if pending is not None:
        if pending.residual.dtype != torch.bfloat16 or pending.residual.shape != src.shape:
            raise KernelError("the residual must be bfloat16 and have the shape of x")
        P.residual = pending.residual.data_ptr()
        P.residual_out = 0 if pending.residual_out is None or stats is not None else pending.residual_out.data_ptr()
        if stats is not None:
            P.stats_in, P.stats_tiles = stats[0].data_ptr(), int(stats[1])
        P.norm_w, P.norm_w_f32, P.eps = pending.weight.data_ptr(), int(pending.weight.dtype == torch.float32), pending.eps
        if pending.weight.numel() != k or pending.weight.dtype not in (torch.float32, torch.bfloat16):
            raise KernelError("the norm weight must have K elements, bfloat16 or float32")
    P.M, P.N, P.K, P.mode = m, n, k, mode
    dev = src.device
    P.err = error_word(dev).data_ptr()
    P.trace = 0 if skinny_trace is None else skinny_trace.data_ptr()
    if mode == EPI_QKV:
        nh, nkv = qkv["num_heads"], qkv["num_kv_heads"]
        out = qkv["q_out"]
        kc, vc = qkv.get("k_cache"), qkv.get("v_cache")
        qw, kw = qkv.get("q_weight"), qkv.get("k_weight")
        cos, sin = qkv.get("cos"), qkv.get("sin")
        slots = qkv.get("slots")
        inv_freq = qkv.get("inv_freq")
        flags = (1 if qkv.get("plain_norm") else 0) | (2 if qkv.get("norm_after_rotation") else 0) | \
            (4 if qkv.get("values_are_keys") else 0)
        _cuda(out, kc, vc, qw, kw, cos, sin, qkv["positions"], slots, inv_freq)
        _f32(inv_freq)
        kv_tiles = nkv if flags & 4 else 2 * nkv
        if n != (nh + kv_tiles) * head_dim or out.shape != (m, nh * head_dim) or out.dtype != torch.bfloat16:
            raise KernelError("qkv sizes do not fit the weight")
        if inv_freq is not None and (cos is not None or inv_freq.numel() * 2 != int(qkv.get("rot_dim", 0))
                                     or not inv_freq.is_contiguous()):
            raise KernelError("frequencies come instead of tables, one for every rotated pair")
        if flags & 4 and slots is not None and (vc is None or vc.shape != kc.shape or vc.dtype != kc.dtype):
            raise KernelError("values that are the keys need a value cache of the key cache's shape")
        P.inv_freq, P.qkv_flags = (0 if inv_freq is None else inv_freq.data_ptr()), flags
        if slots is not None and (kc is None or kc.dtype != torch.bfloat16 or kc.shape[1] != nkv or kc.shape[3] != head_dim):
            raise KernelError("the cache must be bfloat16 [pages + 1, kv_heads, page_size, head_dim]")
        if (qw is None) != (kw is None) or (qw is not None and qw.dtype != kw.dtype):
            raise KernelError("q and k norm weights come together and share a dtype")
        P.nh, P.nkv, P.rot_dim = nh, nkv, int(qkv.get("rot_dim", 0))
        P.max_pos = 0 if cos is None else cos.shape[0]
        P.page_size = 1 if kc is None else kc.shape[2]
        P.cache_slots = 0 if kc is None else kc.shape[0] * kc.shape[2]
        P.qk_eps = float(qkv.get("eps", 0.0))
        P.q_w, P.k_w = (0 if qw is None else qw.data_ptr()), (0 if kw is None else kw.data_ptr())
        P.qk_w_f32 = int(qw is not None and qw.dtype == torch.float32)
        P.cos_table, P.sin_table = (0 if cos is None else cos.data_ptr()), (0 if sin is None else sin.data_ptr())
        P.positions = qkv["positions"].data_ptr()
        P.slots = 0 if slots is None else slots.data_ptr()
        P.k_cache, P.v_cache = (0 if kc is None else kc.data_ptr()), (0 if vc is None else vc.data_ptr())
    elif out is None:
        out = _few_row_out(m, n, mode, dev)
    if norm_after is not None:
        P.post_residual, P.post_sum_out, P.post_stats = (t.data_ptr() for t in norm_after)
    P.out = out.data_ptr()
    sms = _sm_count(dev)
    box = lib.b200_skinny_box_rows(mode, head_dim, n, sms)
    rc = lib.b200_skinny_linear(_weight_map(weight, box), ctypes.byref(P), head_dim, sms, _stream())
    _ok(rc, "skinny_linear")
    return out


def _few_row_out(m: int, n: int, mode: int, device) -> torch.Tensor:
    if mode == EPI_SWIGLU:
        return torch.empty((m, n // 2), dtype=torch.bfloat16, device=device)
    return torch.empty((m, n), dtype=torch.float32 if mode == EPI_PLAIN_F32 else torch.bfloat16, device=device)


class _StreamParams(ctypes.Structure):
    """Mirror of ``StreamParams`` in csrc/stream_linear.cu (same order, native alignment)."""
    _fields_ = [("x", ctypes.c_void_p), ("x_rows", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("residual_out", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("norm_w_f32", ctypes.c_int),
                ("eps", ctypes.c_float), ("w", ctypes.c_void_p), ("M", ctypes.c_int), ("N", ctypes.c_int),
                ("K", ctypes.c_int), ("mode", ctypes.c_int), ("out", ctypes.c_void_p),
                ("post_residual", ctypes.c_void_p), ("post_sum_out", ctypes.c_void_p), ("post_stats", ctypes.c_void_p),
                ("rw", ctypes.c_int), ("ks", ctypes.c_int), ("groups", ctypes.c_int), ("tiles", ctypes.c_int),
                ("xd", ctypes.c_int), ("pair", ctypes.c_int)]


def _stream_lib():
    lib = load_cuda_library("stream_linear.cu")
    if not getattr(lib, "_checked", False):
        if lib.b200_stream_params_size() != ctypes.sizeof(_StreamParams):
            raise KernelError("the parameter block of stream_linear.cu and its Python mirror differ")
        lib._checked = True
    return lib


# Few-row products on weights of at least this many bytes take the streaming kernel (every thread copies its own share
# of the weights, one CTA an SM walks over many tiles: csrc/stream_linear.cu) instead of the ring kernel
# (csrc/skinny_linear.cu), where the rows of x fit its shared memory: a rule of sizes, fixed by the environment or by
# assignment, never by a measurement.  Measured in a decode step at batch 8: 4.28 -> 3.91 ms at the Qwen3-8B sizes
# (gate/up and the head), 1.320 -> 1.308 ms at the Qwen3-0.6B sizes (the head); smaller matrices are faster on the
# ring kernel (1.41 ms with the 0.6B gate/up here).
stream_min_bytes = int(os.environ.get("LLM_INFER_B200_STREAM_MIN_BYTES", 64 << 20))
stream_pair = int(os.environ.get("LLM_INFER_B200_STREAM_PAIR", -1))


def stream_ok(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
              norm: bool = True) -> bool:
    """Whether the streaming kernel can run this product: bfloat16 activations and weight, at most 16 rows, K a
    multiple of 32; plain or SwiGLU.  Behind a norm (``norm``) the rows must fit its shared memory beside the weights
    on their way (8 rows of about 6,000 columns, 16 of about 3,000); without one, longer rows come with the weights'
    copies."""
    if act_dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.dim() != 2:
        return False
    if not 0 < rows <= SKINNY_MAX_ROWS or weight.shape[1] % 32 or not weight.is_contiguous() or weight.data_ptr() % 16:
        return False
    if mode not in (EPI_PLAIN_BF16, EPI_PLAIN_F32, EPI_SWIGLU) or (mode == EPI_SWIGLU and weight.shape[0] % 2):
        return False
    return bool(_stream_lib().b200_stream_fits(mode, rows, weight.shape[0], weight.shape[1], int(norm)))


def stream_takes(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
                 norm: bool = True) -> bool:
    """Whether a few-row product (behind a norm or not) is routed to the streaming kernel: a weight of
    ``stream_min_bytes`` or more, and rows of x that fit the kernel's shared memory; rows that do not fit (and have no
    norm before them) only for more than 8 rows of a weight that the ring kernel would else take, since it falls off
    there (Qwen3-8B down projection, 16 rows: 22.8 against 37.4 us, a decode step at batch 16 6.36 -> 5.96 ms; with 8
    rows 20.2 against 21.3 us alone and a decode step no faster for it; the Qwen3-32B down projection is faster on
    the library: 49 against 64 us)."""
    nbytes = 2 * weight.shape[0] * weight.shape[1]
    if few_row_route != "single" or nbytes < stream_min_bytes:
        return False
    if stream_ok(rows, weight, act_dtype, mode, True):
        return True
    return not norm and rows > 8 and nbytes < single_max_bytes and stream_ok(rows, weight, act_dtype, mode, False)


def stream_tile_cols(mode: int, m: int, n: int, k: int, norm: bool) -> int:
    """Columns of the output that one tile of the streaming kernel covers for a product of ``m`` rows with a weight
    [n, k] (its tiles of statistics)."""
    return _stream_lib().b200_stream_tile_cols(mode, m, n, k, int(norm))


def stream_linear(x, weight: torch.Tensor, mode: int = EPI_PLAIN_BF16, x_rows: Optional[torch.Tensor] = None,
                  out: Optional[torch.Tensor] = None, norm_after=None, rw: int = 0, ks: int = 0,
                  xd: int = -1, pair: Optional[int] = None) -> torch.Tensor:
    """epilogue(prologue(x) . weight^T) for at most 16 rows and a large weight (csrc/stream_linear.cu).

    ``x``: a bfloat16 tensor [rows, K] or a ``PendingNorm`` (with or without a residual); ``mode``: EPI_PLAIN_BF16,
    EPI_PLAIN_F32 or EPI_SWIGLU; ``norm_after`` = (residual, sum_out, stats [tiles, 16]) as for ``skinny_linear``,
    with tiles = ceil(N / ``stream_tile_cols(...)``); ``rw``, ``ks``: the launch's shape (groups of 16 weight rows a
    tile: 1 or 2; warps that split K: up to 24), 0 for the launcher's choice; ``xd``: whether the rows of x come with
    the weights' copies instead of waiting in shared memory (1, 0, or -1: where they do not fit; never behind a norm);
    ``pair``: clusters of two CTAs that stage half of the rows of x each (1, 0, or -1: where the grid fills the GPU).
    """
    _flush_held()
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    _cuda(src, weight, rows_t)
    _contig(src, weight, rows_t)
    m = src.shape[0] if rows_t is None else rows_t.numel()
    n, k = weight.shape
    if src.shape[-1] != k:
        raise KernelError(f"the rows have {src.shape[-1]} columns, the weight has {k}")
    if not stream_ok(m, weight, src.dtype, mode, pending is not None):
        raise KernelError("the streaming product refuses this size or dtype")
    P = _StreamParams()
    P.x, P.x_rows = src.data_ptr(), (0 if rows_t is None else rows_t.data_ptr())
    if pending is not None:
        w = pending.weight
        if w.numel() != k or w.dtype not in (torch.float32, torch.bfloat16) or not w.is_cuda:
            raise KernelError("the norm weight must have K elements, bfloat16 or float32, on the device")
        P.norm_w, P.norm_w_f32, P.eps = w.data_ptr(), int(w.dtype == torch.float32), pending.eps
        if pending.residual is not None:
            res = pending.residual
            if res.dtype != torch.bfloat16 or res.shape != src.shape or not res.is_contiguous():
                raise KernelError("the residual must be bfloat16, contiguous and have the shape of x")
            P.residual = res.data_ptr()
            P.residual_out = 0 if pending.residual_out is None else pending.residual_out.data_ptr()
    P.w, P.M, P.N, P.K, P.mode = weight.data_ptr(), m, n, k, mode
    if out is None:
        out = _few_row_out(m, n, mode, src.device)
    if norm_after is not None:
        P.post_residual, P.post_sum_out, P.post_stats = (t.data_ptr() for t in norm_after)
    P.out, P.rw, P.ks, P.xd = out.data_ptr(), rw, ks, xd
    P.pair = stream_pair if pair is None else pair
    rc = _stream_lib().b200_stream_linear(ctypes.byref(P), _sm_count(src.device), _stream())
    _ok(rc, "stream_linear")
    return out


# A lazy PLAIN bfloat16 product of the "single" route is held back until the next launch is known: if that is a
# product behind an add + RMSNorm of this product's result, the held product's epilogue begins the norm (the rounded
# sum and the rows' sums of squares), and the next product reads only its own columns instead of whole rows, which
# every one of its CTAs would otherwise fetch (at 4,096 columns that read took 5 of a product's 20 us).
class _Held:
    def __init__(self, x, weight, x_rows, out, stream=False):
        self.x, self.weight, self.x_rows, self.out, self.stream = x, weight, x_rows, out, stream


_held: Optional[_Held] = None


def _flush_held(norm_after=None) -> None:
    """Launch the product that is held back (with the norm that follows it begun in its epilogue, if given)."""
    global _held
    h = _held
    if h is None:
        return
    _held = None
    if h.stream:
        stream_linear(h.x, h.weight, EPI_PLAIN_BF16, x_rows=h.x_rows, out=h.out, norm_after=norm_after)
    else:
        skinny_linear(h.x, h.weight, EPI_PLAIN_BF16, x_rows=h.x_rows, out=h.out, norm_after=norm_after)


def _single_lazy(x, weight, mode, x_rows, qkv, lazy) -> torch.Tensor:
    """The "single" route of ``few_row_linear``."""
    global _held
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    m = src.shape[0] if rows_t is None else rows_t.numel()
    to_stream = mode != EPI_QKV and src.is_cuda and stream_takes(m, weight, src.dtype, mode, pending is not None)
    h = _held
    stats = None
    # (the streaming kernel gets the rows' statistics from its own loop: nothing is handed to it)
    if (h is not None and not to_stream and pending is not None and pending.x is h.out and pending.residual is not None
            and x_rows is None and pending.residual.dtype == torch.bfloat16
            and pending.residual.shape == h.out.shape and pending.residual.is_contiguous()):
        n = h.weight.shape[0]
        if h.stream:
            cols = stream_tile_cols(EPI_PLAIN_BF16, h.out.shape[0], n, h.weight.shape[1], isinstance(h.x, PendingNorm))
        else:
            cols = _skinny().b200_skinny_tile_rows(EPI_PLAIN_BF16, 0, n, _sm_count(h.out.device))
        if 0 < cols <= 128:
            tiles = -(-n // cols)
            stat_t = torch.empty((tiles, SKINNY_MAX_ROWS), dtype=torch.float32, device=h.out.device)
            sum_out = pending.residual_out if pending.residual_out is not None else torch.empty_like(pending.residual)
            _flush_held((pending.residual, sum_out, stat_t))
            stats = (stat_t, tiles)
    _flush_held()
    if (lazy and mode == EPI_PLAIN_BF16 and stats is None and (pending is None or pending.residual is not None)
            and src.is_cuda and (to_stream or skinny_ok(m, weight, src.dtype, mode))):
        _held = _Held(x, weight, x_rows, _few_row_out(m, weight.shape[0], mode, src.device), stream=to_stream)
        return _held.out
    if to_stream:
        return stream_linear(x, weight, mode, x_rows=x_rows)
    return skinny_linear(x, weight, mode, x_rows=x_rows, qkv=qkv, stats=stats)


# --------------------------------------------------------------------------- chains of few-row products
CHAIN_MAX_ROWS = 64
PRO_NONE, PRO_ADD_NORM, PRO_NORM = 0, 1, 2
# How products of few rows are routed: "single" (one kernel per product, up to 16 rows: csrc/skinny_linear.cu),
# "chain" (one persistent kernel for consecutive products, up to 64 rows: csrc/linear_chain.cu) or "library" (cuBLAS
# with the norm, rotation and activation as kernels of their own).  Fixed by the environment or by assignment,
# never by a measurement, so that two processes given the same input run the same kernels.  Measured on B200
# (decode, batch 8, context 4,096): "single" 1.42 ms a step at the Qwen3-0.6B sizes and 4.4 ms at the 8B sizes,
# "chain" 1.86 ms and 6.2 ms (its barriers and tile hand-overs cost what the launches did), so "single" is the default.
few_row_route = os.environ.get("LLM_INFER_B200_FEW_ROW", "single")
single_max_bytes = int(os.environ.get("LLM_INFER_B200_SINGLE_MAX_BYTES", 224 << 20))
# Weights up to this size are multiplied in tiles of 16 rows that one CTA owns (see csrc/linear_chain.cu).
chain_narrow_bytes = int(os.environ.get("LLM_INFER_B200_CHAIN_NARROW_BYTES", 48 << 20))


class _ChainOp(ctypes.Structure):
    """Mirror of ``ChainOp`` in csrc/linear_chain.cu (same order, native alignment)."""
    _fields_ = [("x", ctypes.c_void_p), ("x_rows", ctypes.c_void_p), ("residual", ctypes.c_void_p),
                ("residual_out", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("stats_in", ctypes.c_void_p),
                ("stats_out", ctypes.c_void_p), ("stats_res_in", ctypes.c_void_p), ("stats_res_out", ctypes.c_void_p),
                ("out", ctypes.c_void_p), ("q_w", ctypes.c_void_p), ("k_w", ctypes.c_void_p),
                ("cos_table", ctypes.c_void_p), ("sin_table", ctypes.c_void_p), ("positions", ctypes.c_void_p),
                ("slots", ctypes.c_void_p), ("k_cache", ctypes.c_void_p), ("v_cache", ctypes.c_void_p),
                ("cache_slots", ctypes.c_longlong), ("prologue", ctypes.c_int), ("norm_w_f32", ctypes.c_int),
                ("eps", ctypes.c_float), ("stats_tiles", ctypes.c_int), ("M", ctypes.c_int), ("N", ctypes.c_int),
                ("K", ctypes.c_int), ("mode", ctypes.c_int), ("nh", ctypes.c_int), ("nkv", ctypes.c_int),
                ("head_dim", ctypes.c_int), ("rot_dim", ctypes.c_int), ("max_pos", ctypes.c_int),
                ("page_size", ctypes.c_int), ("qk_w_f32", ctypes.c_int), ("qk_eps", ctypes.c_float),
                ("narrow", ctypes.c_int), ("box_rows", ctypes.c_int), ("tiles", ctypes.c_int), ("kblocks", ctypes.c_int), ("per", ctypes.c_int), ("ctas", ctypes.c_int),
                ("first_cta", ctypes.c_int), ("ticket_off", ctypes.c_int)]


def _chain_lib():
    lib = load_cuda_library("linear_chain.cu")
    if not getattr(lib, "_checked", False):
        if lib.b200_chain_op_size() != ctypes.sizeof(_ChainOp):
            raise KernelError("the product block of linear_chain.cu and its Python mirror differ")
        lib.b200_chain_scratch_floats.restype = ctypes.c_longlong
        lib._checked = True
    return lib


_chain_maps = {}
_chain_state = {}
_CHAIN_TICKETS = 1 << 16


def _chain_map(weight: torch.Tensor, box_rows: int):
    key = (weight.data_ptr(), tuple(weight.shape), box_rows)
    buf = _chain_maps.get(key)
    if buf is None:
        buf = ctypes.create_string_buffer(128)
        rc = _chain_lib().b200_chain_weight_map(buf, _p(weight), ctypes.c_longlong(weight.shape[0]),
                                                ctypes.c_longlong(weight.shape[1]), box_rows)
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a weight matrix could not be made (code {rc})")
        if len(_chain_maps) > 8192:
            _chain_maps.clear()
        _chain_maps[key] = buf
    return buf


def _chain_buffers(device):
    """Scratch for partial sums (sized for 64 rows on every SM: 9.7 MB), tickets and the grid barrier's words of
    one device; made once, so that a graph may capture launches that use them."""
    key = torch.device(device).index or 0
    st = _chain_state.get(key)
    if st is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the chain kernel's buffers must exist before a graph is captured")
        floats = int(_chain_lib().b200_chain_scratch_floats(CHAIN_MAX_ROWS, _sm_count(device)))
        st = _chain_state[key] = dict(scratch=torch.empty(floats, dtype=torch.float32, device=device),
                                      tickets=torch.zeros(_CHAIN_TICKETS, dtype=torch.int32, device=device),
                                      sync=torch.zeros(_chain_lib().b200_chain_sync_words(), dtype=torch.int32,
                                                       device=device))
    return st


def _reset_chain_state(device) -> None:
    """After a wait inside the chain kernel ran out its barrier words and tickets may hold anything."""
    st = _chain_state.get(torch.device(device).index or 0)
    if st is not None:
        st["tickets"].zero_()
        st["sync"].zero_()


def chain_takes(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
                head_dim: int = 0) -> bool:
    """Whether the chain kernel takes this product: bfloat16 activations and weight, at most 64 rows, K a multiple
    of 8; QKV: a head size that divides 128."""
    if act_dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not weight.is_cuda or weight.dim() != 2:
        return False
    if not 0 < rows <= CHAIN_MAX_ROWS or weight.shape[1] % 8 or not weight.is_contiguous() or weight.data_ptr() % 16:
        return False
    if mode == EPI_QKV and (head_dim <= 0 or 128 % head_dim):
        return False
    if mode == EPI_SWIGLU and weight.shape[0] % 2:
        return False
    return True


def few_row_takes(rows: int, weight: torch.Tensor, act_dtype: torch.dtype, mode: int = EPI_PLAIN_BF16,
                  head_dim: int = 0, norm: bool = True) -> bool:
    """Whether a product of ``rows`` rows runs on this package's few-row kernels (with the norm before it and the
    epilogue after it fused in) rather than as a library product with those as kernels of their own.  ``norm``: the
    product may come behind a norm (False: its input is a plain tensor)."""
    if few_row_route == "chain" and chain_takes(rows, weight, act_dtype, mode, head_dim):
        return True
    if few_row_route == "library":
        return False
    if mode != EPI_QKV and stream_takes(rows, weight, act_dtype, mode, norm):
        return True
    if not skinny_ok(rows, weight, act_dtype, mode, head_dim):
        return False
    # The single-product kernel gives every CTA the rows of x to normalise and one tile of 128 weight rows; on the
    # largest layer matrices (gate/up and down at the Qwen3-32B sizes, 262 and 524 MB) the library product with the norm
    # and activation as kernels of their own was measured faster (14.8 against 18.9 ms a decode step at batch 8).
    return mode == EPI_PLAIN_F32 or 2 * weight.shape[0] * weight.shape[1] < single_max_bytes


class _Chain:
    def __init__(self, device):
        self.device = device
        self.ops, self.weights, self.keep = [], [], []
        self.by_out = {}                 # data pointer of a product's output -> (index, output tensor)
        self.stats_from = {}             # index of a product -> index of the product that leaves its rows' statistics


_chain: Optional[_Chain] = None
# For tuning: an int64 tensor [SMs, 64] on the device; every CTA's first thread then leaves the nanosecond clock there at
# eight places of every product of the next launches (start, barrier passed, row scales, x staged, products done,
# sums added, epilogue done).
chain_trace: Optional[torch.Tensor] = None
chain_stages = int(os.environ.get("LLM_INFER_B200_CHAIN_STAGES", 8))


def few_row_linear(x, weight: torch.Tensor, mode: int = EPI_PLAIN_BF16, x_rows: Optional[torch.Tensor] = None,
                   qkv: Optional[dict] = None, lazy: bool = False) -> torch.Tensor:
    """epilogue(prologue(x) . weight^T) for few rows; arguments as ``skinny_linear``.

    ``lazy`` (on the "chain" route): the product is not launched here.  It joins the products that wait, and all
    of them run in one persistent kernel when something else is about to be launched (``flush_chain``; every
    wrapper of this module does that first).  The returned tensor is filled by then: code that touches it with
    anything but this module's wrappers must call ``flush_chain()`` before.  Without ``lazy`` the product (and
    whatever waited before it) is launched before this returns."""
    pending = x if isinstance(x, PendingNorm) else None
    src = pending.x if pending is not None else x
    rows_t = pending.rows if pending is not None and pending.rows is not None else x_rows
    m = src.shape[0] if rows_t is None else rows_t.numel()
    head_dim = qkv["head_dim"] if qkv else 0
    further = bool(qkv) and any(qkv.get(key) is not None and qkv.get(key) is not False
                                for key in ("inv_freq", "plain_norm", "norm_after_rotation", "values_are_keys"))
    if few_row_route == "chain" and not further and chain_takes(m, weight, src.dtype, mode, head_dim):
        out = _chain_append(pending, src, rows_t, m, weight, mode, qkv)
        if not lazy:
            flush_chain()
        return out
    return _single_lazy(x, weight, mode, x_rows, qkv, lazy)


def _chain_append(pending, src, rows_t, m, weight, mode, qkv) -> torch.Tensor:
    global _chain
    _cuda_only(src, weight, rows_t)
    _contig(src, weight, rows_t)
    n, k = weight.shape
    if src.shape[-1] != k or src.dim() != 2:
        raise KernelError(f"the rows have {src.shape[-1]} columns, the weight has {k}")
    dev = src.device
    if _chain is not None and _chain.device != dev:
        flush_chain()
    if _chain is None:
        _chain = _Chain(dev)
    ch = _chain
    op = _ChainOp()
    op.x, op.x_rows = src.data_ptr(), (0 if rows_t is None else rows_t.data_ptr())
    op.M, op.N, op.K, op.mode = m, n, k, mode
    if pending is not None:
        w = pending.weight
        if w.numel() != k or w.dtype not in (torch.float32, torch.bfloat16) or not w.is_cuda:
            raise KernelError("the norm weight must have K elements, bfloat16 or float32, on the device")
        op.norm_w, op.norm_w_f32, op.eps = w.data_ptr(), int(w.dtype == torch.float32), pending.eps
        op.prologue = PRO_NORM
        if pending.residual is not None:
            res = pending.residual
            if res.dtype != torch.bfloat16 or res.shape != src.shape or not res.is_contiguous():
                raise KernelError("the residual must be bfloat16, contiguous and have the shape of x")
            op.prologue = PRO_ADD_NORM
            op.residual = res.data_ptr()
            made = ch.by_out.get(src.data_ptr())
            if made is not None and made[1] is src and ch.ops[made[0]].mode == EPI_PLAIN_BF16 \
                    and ch.ops[made[0]].stats_out is None:
                # x is the output of a product of this chain: that product's epilogue adds the residual, stores the
                # rounded sum and leaves the rows' sums of squares, so nobody has to read whole rows again
                prev = ch.ops[made[0]]
                tiles = _chain_lib().b200_chain_tiles(EPI_PLAIN_BF16, prev.N, 1)      # (narrow tiles are the most)
                stats = torch.empty(tiles * CHAIN_MAX_ROWS, dtype=torch.float32, device=dev)
                sum_out = pending.residual_out if pending.residual_out is not None else torch.empty_like(res)
                prev.stats_out, prev.stats_res_in, prev.stats_res_out = stats.data_ptr(), res.data_ptr(), sum_out.data_ptr()
                op.stats_in = stats.data_ptr()
                ch.stats_from[len(ch.ops)] = made[0]          # (how many tiles wrote them is known at the launch)
                ch.keep += [stats, sum_out]
            else:
                op.residual_out = 0 if pending.residual_out is None else pending.residual_out.data_ptr()
        ch.keep.append(pending)
    if mode == EPI_QKV:
        nh, nkv, head_dim = qkv["num_heads"], qkv["num_kv_heads"], qkv["head_dim"]
        out = qkv["q_out"]
        kc, vc = qkv.get("k_cache"), qkv.get("v_cache")
        qw, kw = qkv.get("q_weight"), qkv.get("k_weight")
        cos, sin = qkv.get("cos"), qkv.get("sin")
        slots = qkv.get("slots")
        _cuda_only(out, kc, vc, qw, kw, cos, sin, qkv["positions"], slots)
        _contig(out, kc, vc, qw, kw, cos, sin, qkv["positions"], slots)
        if n != (nh + 2 * nkv) * head_dim or out.shape != (m, nh * head_dim) or out.dtype != torch.bfloat16:
            raise KernelError("qkv sizes do not fit the weight")
        if slots is not None and (kc is None or kc.dtype != torch.bfloat16 or kc.shape[1] != nkv or kc.shape[3] != head_dim
                                  or vc is None or vc.dtype != torch.bfloat16):
            raise KernelError("the cache must be bfloat16 [pages + 1, kv_heads, page_size, head_dim]")
        if (qw is None) != (kw is None) or (qw is not None and qw.dtype != kw.dtype):
            raise KernelError("q and k norm weights come together and share a dtype")
        if cos is not None and (cos.dtype != torch.float32 or sin.dtype != torch.float32):
            raise KernelError("rotary tables must be float32")
        op.nh, op.nkv, op.head_dim, op.rot_dim = nh, nkv, head_dim, int(qkv.get("rot_dim", 0)) if cos is not None else 0
        op.max_pos = 0 if cos is None else cos.shape[0]
        op.page_size = 1 if kc is None else kc.shape[2]
        op.cache_slots = 0 if kc is None else kc.shape[0] * kc.shape[2]
        op.qk_eps = float(qkv.get("eps", 0.0))
        op.q_w, op.k_w = (0 if qw is None else qw.data_ptr()), (0 if kw is None else kw.data_ptr())
        op.qk_w_f32 = int(qw is not None and qw.dtype == torch.float32)
        op.cos_table, op.sin_table = (0 if cos is None else cos.data_ptr()), (0 if sin is None else sin.data_ptr())
        op.positions = qkv["positions"].data_ptr()
        op.slots = 0 if slots is None else slots.data_ptr()
        op.k_cache, op.v_cache = (0 if kc is None else kc.data_ptr()), (0 if vc is None else vc.data_ptr())
        ch.keep.append(qkv)
    elif mode == EPI_SWIGLU:
        out = torch.empty((m, n // 2), dtype=torch.bfloat16, device=dev)
    else:
        out = torch.empty((m, n), dtype=torch.float32 if mode == EPI_PLAIN_F32 else torch.bfloat16, device=dev)
    op.out = out.data_ptr()
    ch.ops.append(op)
    ch.weights.append(weight)
    ch.keep += [src, rows_t, out]
    ch.by_out[out.data_ptr()] = (len(ch.ops) - 1, out)
    return out


def chain_pending() -> int:
    """Products that wait in the chain."""
    return 0 if _chain is None else len(_chain.ops)


def flush_chain() -> None:
    """Launch the products that wait in the chain (at most six per launch of the persistent kernel)."""
    global _chain
    _flush_held()
    ch = _chain
    if ch is None:
        return
    _chain = None
    lib = _chain_lib()
    st = _chain_buffers(ch.device)
    most = lib.b200_chain_max_ops()
    sms = _sm_count(ch.device)
    groups = [range(at, min(at + most, len(ch.ops))) for at in range(0, len(ch.ops), most)]
    for group in groups:                                   # the kind of tile depends on the launch's largest row count
        rows = max(ch.ops[i].M for i in group)
        for i in group:
            op, w = ch.ops[i], ch.weights[i]
            op.narrow = lib.b200_chain_narrow(op.mode, op.N, op.K, rows, ctypes.c_longlong(chain_narrow_bytes))
            op.box_rows = lib.b200_chain_box_rows(op.mode, op.narrow)
    for i, source in ch.stats_from.items():
        ch.ops[i].stats_tiles = lib.b200_chain_tiles(ch.ops[source].mode, ch.ops[source].N, ch.ops[source].narrow)
    with torch.cuda.device(ch.device):
        for group in groups:
            ops_now = [ch.ops[i] for i in group]
            if sum(lib.b200_chain_tiles(o.mode, o.N, o.narrow) for o in ops_now) > _CHAIN_TICKETS:
                raise KernelError("a chain of products has more tiles than the ticket array holds")
            block = (_ChainOp * len(ops_now))(*ops_now)
            maps = ctypes.create_string_buffer(b"".join(_chain_map(ch.weights[i], ch.ops[i].box_rows).raw for i in group),
                                               128 * len(ops_now))
            rc = lib.b200_linear_chain(block, maps, len(ops_now), _p(st["scratch"]), _p(st["tickets"]), _p(st["sync"]),
                                       _p(error_word(ch.device)), _p(chain_trace), chain_stages, sms, _stream())
            _ok(rc, "linear_chain")


# --------------------------------------------------------------------------- many-row products on tcgen05
GEMM_PLAIN, GEMM_SWIGLU = 0, 1
_gemm_maps = {}


def _gemm_map(t: torch.Tensor):
    key = (t.data_ptr(), tuple(t.shape))
    buf = _gemm_maps.get(key)
    if buf is None:
        buf = ctypes.create_string_buffer(128)
        rc = load_cuda_library("gemm_tcgen05.cu").b200_gemm_tensor_map(buf, _p(t), ctypes.c_longlong(t.shape[0]),
                                                                       ctypes.c_longlong(t.shape[1]))
        if rc != 0:
            raise KernelError(f"the TMA descriptor of a matrix could not be made (code {rc})")
        if len(_gemm_maps) > 8192:
            _gemm_maps.clear()
        _gemm_maps[key] = buf
    return buf


def gemm_tc_ok(x: torch.Tensor, weight: torch.Tensor, mode: int = GEMM_PLAIN) -> bool:
    """bfloat16 row-major operands on the device, K a multiple of 8 (16-byte rows for TMA); SwiGLU: even N."""
    return (x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.is_cuda and weight.is_cuda
            and x.dim() == 2 and weight.dim() == 2 and x.is_contiguous() and weight.is_contiguous()
            and x.shape[1] == weight.shape[1] and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0
            and weight.data_ptr() % 16 == 0 and (mode == GEMM_PLAIN or weight.shape[0] % 2 == 0))


def gemm_tc_pays(x: torch.Tensor, weight: torch.Tensor, mode: int = GEMM_PLAIN) -> bool:
    """Whether the tcgen05 product is the faster way: measured on B200, the fused SwiGLU form ties or beats the
    library product followed by the activation kernel once every SM has several tiles of 128 x 256 and K is
    long (1,369 against 1,354 TFLOP/s at 2,048 x 24,576 x 4,096); on smaller shapes the library is ahead."""
    if mode != GEMM_SWIGLU or not gemm_tc_ok(x, weight, mode):
        return False
    tiles = -(-x.shape[0] // 128) * -(-(weight.shape[0] // 2) // 128)
    return x.shape[1] >= 2048 and tiles >= 4 * _sm_count(x.device)


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, mode: int = GEMM_PLAIN) -> torch.Tensor:
    """x . weight^T on the tcgen05 tensor cores (TMA-fed, float sums in tensor memory), bfloat16 out.
    ``GEMM_SWIGLU``: weight = [gate rows; up rows]; the result is silu(x . gate^T) * (x . up^T)."""
    flush_chain()
    if not gemm_tc_ok(x, weight, mode):
        raise KernelError("the tcgen05 product takes contiguous bfloat16 [M, K] and [N, K] with K a multiple of 8")
    m, k = x.shape
    n = weight.shape[0]
    out = torch.empty((m, n // 2 if mode == GEMM_SWIGLU else n), dtype=torch.bfloat16, device=x.device)
    a_map = ctypes.create_string_buffer(128)          # activations move: their descriptor is made per call
    lib = load_cuda_library("gemm_tcgen05.cu")
    rc = lib.b200_gemm_tensor_map(a_map, _p(x), ctypes.c_longlong(m), ctypes.c_longlong(k))
    if rc != 0:
        raise KernelError(f"the TMA descriptor of the activations could not be made (code {rc})")
    rc = lib.b200_gemm_tcgen05(a_map, _gemm_map(weight), _p(out), m, n, k, mode, _p(error_word(x.device)), _stream())
    _ok(rc, "gemm_tcgen05")
    return out


# --------------------------------------------------------------------------- matrix products
def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """a[M, K] . w[N, K]^T in true 32-bit on CUDA cores."""
    _cuda(a, w, out)
    _contig(a, w, out)
    if a.dtype != torch.float32 or w.dtype != torch.float32 or a.shape[1] != w.shape[1]:
        raise KernelError("gemm_f32 takes float32 [M, K] and [N, K]")
    m, k = a.shape
    n = w.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    rc = load_cuda_library("gemm_f32.cu").b200_gemm_f32(_p(a), _p(w), _p(out), m, n, k, _stream())
    _ok(rc, "gemm_f32")
    return out


def head_products(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One small product per head: out[h] = x[h] . weight[h]^T with x [heads, rows, k] (any strides with a unit inner
    one, so a head may be a column range of a wider matrix), weight [heads, n, k] contiguous, out [heads, rows, n]
    (given: any strides with a unit inner one).  float32: this package's 32-bit kernel; bfloat16: the library's
    batched product with float accumulation."""
    _cuda(x, weight, out)
    heads, rows, k = x.shape
    n = weight.shape[1]
    if weight.shape[0] != heads or weight.shape[2] != k or not weight.is_contiguous() or x.stride(2) != 1 \
            or x.dtype != weight.dtype:
        raise KernelError("head_products takes x [heads, rows, k] and contiguous weights [heads, n, k] of one dtype")
    if out is None:
        out = torch.empty((heads, rows, n), dtype=x.dtype, device=x.device)
    elif tuple(out.shape) != (heads, rows, n) or out.stride(2) != 1 or out.dtype != x.dtype:
        raise KernelError("head_products: the output must be [heads, rows, n] with a unit inner stride")
    if x.dtype == torch.float32:
        rc = load_cuda_library("gemm_f32.cu").b200_gemm_f32_batched(
            _p(x), _p(weight), _p(out), rows, n, k, heads, x.stride(1), k, out.stride(1),
            ctypes.c_longlong(x.stride(0)), ctypes.c_longlong(n * k), ctypes.c_longlong(out.stride(0)), _stream())
        _ok(rc, "gemm_f32_batched")
        return out
    if x.dtype != torch.bfloat16:
        raise KernelError("head_products takes float32 or bfloat16")
    torch.bmm(x, weight.transpose(1, 2), out=out)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           lazy: bool = False) -> torch.Tensor:
    """x[M, K] . weight[N, K]^T, no bias.  ``lazy``: see ``few_row_linear``.

    float32 x float32: this package's 32-bit kernel.  bfloat16 x bfloat16: few rows (see ``few_row_takes``) on
    this package's few-row kernels, more on cuBLAS with float accumulation.  Mixed dtypes are multiplied in
    32-bit (the narrower operand is widened first).
    """
    out_dtype = out_dtype or x.dtype
    if x.dtype == torch.float32 and weight.dtype == torch.float32:
        return cast(gemm_f32(x, weight), out_dtype)
    if x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16:
        if out_dtype in (torch.bfloat16, torch.float32) and x.dim() == 2 and x.is_contiguous() and x.is_cuda:
            mode = EPI_PLAIN_F32 if out_dtype == torch.float32 else EPI_PLAIN_BF16
            if few_row_takes(x.shape[0], weight, x.dtype, mode, norm=False):
                return few_row_linear(x, weight, mode, lazy=lazy)
        _cuda(x, weight)
        if out_dtype == torch.bfloat16:
            return torch.mm(x, weight.t())
        return torch.mm(x, weight.t(), out_dtype=out_dtype)
    if weight.dtype == torch.float32:
        return cast(gemm_f32(cast(x, torch.float32), weight), out_dtype)
    return cast(gemm_f32(x, cast(weight, torch.float32)), out_dtype)


# --------------------------------------------------------------------------- sampling
def argmax(logits: torch.Tensor) -> torch.Tensor:
    _cuda(logits)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("argmax takes float32 logits [rows, vocab] with unit inner stride")
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    rc = load_cuda_library("sampling.cu").b200_argmax(_p(logits), ctypes.c_longlong(logits.stride(0)),
                                                      logits.shape[0], logits.shape[1], _p(out),
                                                      _p(error_word(logits.device)), _stream())
    _ok(rc, "argmax")
    return out


def sample(logits: torch.Tensor, params: torch.Tensor, uniforms: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``params``: uint8 [rows, 32] device tensor of packed rows (see sampling.pack_rows)."""
    _cuda(logits, params, uniforms)
    if logits.dtype != torch.float32 or logits.dim() != 2 or logits.stride(1) != 1:
        raise KernelError("sample takes float32 logits [rows, vocab] with unit inner stride")
    if params.numel() * params.element_size() != logits.shape[0] * 32:
        raise KernelError("sampling parameters must hold 32 bytes per row")
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    rc = load_cuda_library("sampling.cu").b200_sample(_p(logits), ctypes.c_longlong(logits.stride(0)),
                                                      logits.shape[0], logits.shape[1], _p(params), _p(out),
                                                      _p(uniforms), _p(error_word(logits.device)), _stream())
    _ok(rc, "sample")
    return out


# --------------------------------------------------------------------------- float32 residual stream, one-gain norms
def _token_conv():
    return load_cuda_library("token_conv.cu")


def _f32(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and t.dtype != torch.float32:
            raise KernelError("this operand must be float32")


def _i32(*tensors: Optional[torch.Tensor]) -> None:
    for t in tensors:
        if t is not None and t.dtype != torch.int32:
            raise KernelError("index arrays must be int32")


def residual_scale(x: torch.Tensor, y: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                   want_scale: bool = True) -> Optional[torch.Tensor]:
    """x += y in place (x float32 [tokens, width], the sum in float; ``y`` None: nothing is added), and the scale
    of a one-gain RMS norm of the new x for every token: gain / sqrt(mean(x^2) + eps), float32 [tokens]."""
    _cuda(x, y, gain)
    _contig(x, y, gain)
    _f32(x, gain)
    if x.dim() != 2 or (y is not None and y.shape != x.shape) or gain.numel() != 1:
        raise KernelError("residual_scale takes x and y [tokens, width] and one gain")
    scale = torch.empty(x.shape[0], dtype=torch.float32, device=x.device) if want_scale else None
    rc = _token_conv().b200_residual_scale(_p(x), _p(y), _code(y) if y is not None else F32, _p(gain),
                                           ctypes.c_float(eps), _p(scale), x.shape[0], x.shape[1], _stream())
    _ok(rc, "residual_scale")
    return scale


def scaled_rows(x: torch.Tensor, scale: torch.Tensor, rows: Optional[torch.Tensor], out_dtype: torch.dtype) -> torch.Tensor:
    """out[r] = x[rows[r]] * scale[rows[r]] (rows None: every row), rounded once to ``out_dtype``."""
    _cuda(x, scale, rows)
    _contig(x, scale, rows)
    _f32(x, scale)
    _i32(rows)
    n = x.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, x.shape[1]), dtype=out_dtype, device=x.device)
    rc = _token_conv().b200_scaled_rows(_p(out), _code(out), _p(x), _p(scale), _p(rows), n, x.shape[1], _stream())
    _ok(rc, "scaled_rows")
    return out


def _all_single(ctx) -> int:
    """1 when the step is known to bring every row one token (the rows' convolution states are then brought up to
    date inside the convolution kernels and the kernel that does it for longer rows is not launched)."""
    return int(getattr(ctx, "num_prefill", None) == 0)


def causal_taps(x: torch.Tensor, weight: Optional[torch.Tensor], state: Optional[torch.Tensor], ctx,
                out_dtype: torch.dtype, scale: Optional[torch.Tensor] = None, identity: bool = False,
                channels: Optional[int] = None, update_state: bool = True) -> torch.Tensor:
    """A short causal convolution over time on every channel, for a step's rows:

        y[t] = (u[t] if identity) + sum_j weight[:, j] * u[t - taps + 1 + j],   u[t] = x[t] * scale[t]

    with the inputs before a row's first token taken from ``state[slot]`` ([taps - 1, channels] float32, oldest
    first; zeros for a row that starts its sequence), and the rows' states brought up to date afterwards.
    ``channels``: only the first so many columns of ``x`` pass through.  ``ctx`` gives the step's index arrays."""
    _cuda(x, weight, state, scale)
    _contig(x, weight, state, scale)
    _f32(weight, state, scale)
    c = int(channels or x.shape[1])
    taps = 1 if weight is None else weight.shape[1]
    if weight is not None and weight.shape[0] != c:
        raise KernelError("the taps must be [channels, taps]")
    if taps > 1 and (state is None or tuple(state.shape[1:]) != (taps - 1, c)):
        raise KernelError("the state of a convolution must be [slots + 1, taps - 1, channels]")
    out = torch.empty((x.shape[0], c), dtype=out_dtype, device=x.device)
    rc = _token_conv().b200_causal_taps(
        _p(x), _code(x), x.shape[1], _p(scale), _p(weight), taps, c, _p(state), _p(ctx.row_of_token), _p(ctx.cu_q),
        _p(ctx.prefix_len), _p(ctx.state_slots), _p(out), _code(out), c, int(bool(identity)), x.shape[0],
        ctx.num_rows, int(bool(update_state)), _all_single(ctx), _stream())
    _ok(rc, "causal_taps", 2 if update_state and taps > 1 and not _all_single(ctx) else 1)
    return out


def add_norm_taps_single(x: torch.Tensor, y: Optional[torch.Tensor], gain: torch.Tensor, eps: float,
                         weight: torch.Tensor, state: Optional[torch.Tensor], ctx, out_dtype: torch.dtype,
                         identity: bool) -> Optional[torch.Tensor]:
    """``residual_scale`` and ``causal_taps`` in one kernel, for a step whose rows all bring ONE token (a decode
    step): x += y, the one-gain norm's scale, the convolution over the normed rows, the rows' states.  None when
    the step has longer rows or the rows are no whole 16-byte pieces: the caller then runs the two."""
    taps = weight.shape[1]
    if not _all_single(ctx) or x.shape[1] % 8 or (taps > 1 and state is None):
        return None
    _cuda(x, y, gain, weight, state)
    _contig(x, y, gain, weight, state)
    _f32(x, gain, weight, state)
    if weight.shape[0] != x.shape[1] or (taps > 1 and tuple(state.shape[1:]) != (taps - 1, x.shape[1])):
        raise KernelError("the taps must be [channels, taps] and the state [slots + 1, taps - 1, channels]")
    scale = torch.empty(x.shape[0], dtype=torch.float32, device=x.device)
    out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
    rc = _token_conv().b200_add_norm_taps_single(
        _p(x), _p(y), _code(y) if y is not None else F32, _p(gain), ctypes.c_float(eps), _p(scale), _p(weight), taps,
        x.shape[1], _p(state), _p(ctx.row_of_token), _p(ctx.cu_q), _p(ctx.prefix_len), _p(ctx.state_slots), _p(out),
        _code(out), int(bool(identity)), x.shape[0], _stream())
    if rc in (-2, -3):
        return None
    _ok(rc, "add_norm_taps_single")
    return out


def taps_state_update(x: torch.Tensor, taps: int, channels: int, state: torch.Tensor, ctx) -> None:
    """The last ``taps - 1`` rows of x (first ``channels`` columns) of every row of the step become its state."""
    if taps <= 1:
        return
    _cuda(x, state)
    _contig(x, state)
    _f32(state)
    rc = _token_conv().b200_taps_state_update(_p(x), _code(x), x.shape[1], None, taps, channels, _p(state),
                                              _p(ctx.cu_q), _p(ctx.prefix_len), _p(ctx.state_slots), ctx.num_rows,
                                              0, _stream())
    _ok(rc, "taps_state_update")


def conv_qkv_post(x: torch.Tensor, conv_weight: Optional[torch.Tensor], state: Optional[torch.Tensor], ctx,
                  q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], rot_dim: int, slots: Optional[torch.Tensor], num_heads: int,
                  num_kv_heads: int, head_dim: int, v_head_dim: int, vmix: Optional[torch.Tensor] = None,
                  v_first: Optional[torch.Tensor] = None, v_mode: int = 0) -> None:
    """Short convolution of the packed q, k, v columns of ``x`` (state as in ``causal_taps``), rotation of q and
    k by position * inv_freq, value mixing (``v_mode`` 1: this v is written to ``v_first``; 2: v becomes
    (1 - vmix) v + vmix v_first), q to ``q_out``, k and v into the paged cache at ``slots``; the rows' convolution
    states are brought up to date."""
    _cuda(x, conv_weight, state, q_out, k_cache, v_cache, inv_freq, slots, vmix, v_first)
    _contig(x, conv_weight, state, q_out, k_cache, v_cache, inv_freq, slots, vmix, v_first)
    _f32(conv_weight, state, inv_freq, vmix, v_first)
    c = (num_heads + num_kv_heads) * head_dim + num_kv_heads * v_head_dim
    if x.shape[1] < c or q_out.dtype != x.dtype or k_cache.dtype != x.dtype or v_cache.dtype != x.dtype:
        raise KernelError("conv_qkv_post: the projection is too narrow, or q, cache and projection differ in dtype")
    taps = 1 if conv_weight is None else conv_weight.shape[1]
    if conv_weight is not None and conv_weight.shape[0] != c:
        raise KernelError("the taps must be [q + k + v channels, taps]")
    if taps > 1 and (state is None or tuple(state.shape[1:]) != (taps - 1, c)):
        raise KernelError("the state of a convolution must be [slots + 1, taps - 1, channels]")
    if tuple(k_cache.shape[1:]) != (num_kv_heads, k_cache.shape[2], head_dim) or \
            tuple(v_cache.shape[1:]) != (num_kv_heads, k_cache.shape[2], v_head_dim):
        raise KernelError("the cache must be [pages + 1, kv_heads, page_size, width]")
    if inv_freq is not None and inv_freq.numel() * 2 != rot_dim:
        raise KernelError("one frequency for every rotated pair is needed")
    page_size = k_cache.shape[2]
    rc = load_cuda_library("conv_qkv_post.cu").b200_conv_qkv_post(
        _p(x), _code(x), x.shape[1], _p(conv_weight), taps, _p(state), _p(ctx.row_of_token), _p(ctx.cu_q),
        _p(ctx.prefix_len), _p(ctx.state_slots), _p(q_out), _p(k_cache), _p(v_cache), _p(inv_freq),
        int(rot_dim if inv_freq is not None else 0), _p(ctx.positions), _p(slots), num_heads, num_kv_heads, head_dim,
        v_head_dim, page_size, ctypes.c_longlong(k_cache.shape[0] * page_size), _p(vmix), _p(v_first), int(v_mode),
        x.shape[0], ctx.num_rows, _all_single(ctx), _p(error_word(x.device)), _stream())
    _ok(rc, "conv_qkv_post", 2 if taps > 1 and not _all_single(ctx) else 1)


RETENTION_CHUNKED_FROM = 32        # a step whose longest row has this many tokens takes the chunked kernels


def retention(x: torch.Tensor, state: torch.Tensor, decay: torch.Tensor, inv_freq: Optional[torch.Tensor],
              rot_dim: int, k_scale: float, ctx, heads: int, head_dim: int, v_head_dim: int,
              chunked: Optional[bool] = None) -> torch.Tensor:
    """o [tokens, heads * v_head_dim] (float32) of S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t over the step's
    rows; q, k (rotated by position * inv_freq, k then times ``k_scale``) and v are the first columns of ``x``;
    ``state`` [slots + 1, heads, head_dim, v_head_dim] float32 is read (rows with a prefix) and written.
    Two forms with the same result up to rounding: a scan that runs the recurrence token by token (steps of short
    rows), and, for steps with long rows and heads up to 128 wide (whole 16-byte pieces), chunks of 64 tokens
    (``chunked`` asks for one)."""
    _cuda(x, state, decay, inv_freq)
    _contig(x, state, decay, inv_freq)
    _f32(state, decay, inv_freq)
    if x.shape[1] < heads * (2 * head_dim + v_head_dim) or tuple(state.shape[1:]) != (heads, head_dim, v_head_dim) \
            or decay.numel() != heads:
        raise KernelError("retention: sizes of the projection, the state or the decays do not fit")
    o = torch.empty((x.shape[0], heads * v_head_dim), dtype=torch.float32, device=x.device)
    lib = load_cuda_library("retention.cu")
    tokens = x.shape[0]
    longest = int(getattr(ctx, "max_q_len", 0) or tokens)
    fits = head_dim <= 128 and v_head_dim <= 128 and head_dim % 4 == 0 and v_head_dim % 8 == 0 and x.shape[1] % 8 == 0
    if (chunked if chunked is not None else longest >= RETENTION_CHUNKED_FROM) and fits:
        # long rows: the state is carried chunk by chunk and every chunk's outputs are computed on their own
        max_chunks = tokens // 64 + ctx.num_rows
        qf = torch.empty((2, tokens, heads * head_dim), dtype=torch.float32, device=x.device)
        before = torch.empty((max_chunks, heads, head_dim, v_head_dim), dtype=torch.float32, device=x.device)
        chunk_base = torch.empty(ctx.num_rows + 1, dtype=torch.int32, device=x.device)
        rc = lib.b200_retention_chunked(
            _p(x), _code(x), x.shape[1], _p(o), _p(state), _p(decay), _p(inv_freq),
            int(rot_dim if inv_freq is not None else 0), ctypes.c_float(k_scale), _p(ctx.positions), _p(ctx.cu_q),
            _p(ctx.prefix_len), _p(ctx.state_slots), ctx.num_rows, heads, head_dim, v_head_dim, tokens, max_chunks,
            _p(qf[0]), _p(qf[1]), _p(before), _p(chunk_base), _stream())
        _ok(rc, "retention_chunked", 4)
        return o
    rc = lib.b200_retention(
        _p(x), _code(x), x.shape[1], _p(o), _p(state), _p(decay), _p(inv_freq),
        int(rot_dim if inv_freq is not None else 0), ctypes.c_float(k_scale), _p(ctx.positions), _p(ctx.cu_q),
        _p(ctx.prefix_len), _p(ctx.state_slots), ctx.num_rows, heads, head_dim, v_head_dim, _stream())
    _ok(rc, "retention")
    return o


# --------------------------------------------------------------------------- gates and PolyNorm
def _gated():
    return load_cuda_library("gated.cu")


def poly_norm(z: torch.Tensor, coef: torch.Tensor, eps: float) -> torch.Tensor:
    """coef[0] N(z) + coef[1] N(z^2) + coef[2] N(z^3) + coef[3], N = division by the root mean square of a row."""
    _cuda(z, coef)
    _contig(z, coef)
    _f32(coef)
    if coef.numel() != 4 or z.dim() != 2:
        raise KernelError("poly_norm takes rows and four coefficients")
    out = torch.empty_like(z)
    rc = _gated().b200_poly_norm(_p(out), _p(z), _p(coef), ctypes.c_float(eps), z.shape[0], z.shape[1], _code(z),
                                 _stream())
    _ok(rc, "poly_norm")
    return out


def head_unit_norm_gate(o: torch.Tensor, packed: torch.Tensor, gate_column: int, heads: int, v_head_dim: int,
                        eps: float) -> torch.Tensor:
    """Every head's vector of ``o`` (float32) divided by its root mean square, times silu of the gate that lies
    in ``packed`` from column ``gate_column`` on; the result has ``packed``'s dtype."""
    _cuda(o, packed)
    _contig(o, packed)
    _f32(o)
    if packed.shape[1] < gate_column + heads * v_head_dim or o.shape[1] != heads * v_head_dim:
        raise KernelError("head_unit_norm_gate: the gate's columns do not fit")
    out = torch.empty((o.shape[0], o.shape[1]), dtype=packed.dtype, device=o.device)
    gate = packed.view(-1)[gate_column:]
    rc = _gated().b200_head_unit_norm_gate(_p(out), _p(o), ctypes.c_void_p(gate.data_ptr()), packed.shape[1],
                                           o.shape[0], heads, v_head_dim, ctypes.c_float(eps), _code(packed), _stream())
    _ok(rc, "head_unit_norm_gate")
    return out


def sigmoid_gate_mul(a: torch.Tensor, packed: torch.Tensor, gate_column: int, per: int = 1) -> torch.Tensor:
    """a * sigmoid(gate), the gate lying in ``packed`` from column ``gate_column`` on; in place.  ``per``: how many
    neighbouring columns of ``a`` share one gate value (1: a gate a column; a head's size: one gate a head)."""
    _cuda(a, packed)
    _contig(a, packed)
    if per <= 0 or a.shape[1] % per or a.dtype != packed.dtype or packed.shape[1] < gate_column + a.shape[1] // per:
        raise KernelError("sigmoid_gate_mul: dtype or columns do not fit")
    gate = packed.view(-1)[gate_column:]
    rc = _gated().b200_sigmoid_gate_mul(_p(a), _p(a), ctypes.c_void_p(gate.data_ptr()), packed.shape[1], a.shape[0],
                                        a.shape[1], int(per), _code(a), _stream())
    _ok(rc, "sigmoid_gate_mul")
    return a


# --------------------------------------------------------------------------- activations, joint norm with a gate, caps
ACTIVATIONS = {"silu": 1, "gelu_erf": 2, "gelu_tanh": 3, "relu_squared": 4}


def activate(x: torch.Tensor, act: str, columns: Optional[int] = None, in_place: bool = False) -> torch.Tensor:
    """act(x) element by element on the first ``columns`` columns of x [tokens, width] (all by default): silu,
    gelu_erf (the exact one), gelu_tanh or relu_squared (max(x, 0)^2); computed in float, rounded once.  ``in_place``: x itself is changed."""
    _cuda(x)
    _contig(x)
    if act not in ACTIVATIONS or x.dim() != 2:
        raise KernelError(f"activation {act!r} is refused: {sorted(ACTIVATIONS)} on [tokens, width]")
    c = int(columns if columns is not None else x.shape[1])
    out = x if in_place else torch.empty((x.shape[0], c), dtype=x.dtype, device=x.device)
    rc = _gated().b200_activate_columns(_p(out), out.shape[1], _p(x), x.shape[1], x.shape[0], c, ACTIVATIONS[act],
                                        _code(x), _stream())
    _ok(rc, "activate_columns")
    return out


def row_norm_gate(o: torch.Tensor, weight: torch.Tensor, packed: torch.Tensor, gate_column: int, eps: float) -> torch.Tensor:
    """o (float32 [tokens, width]) divided by each row's root mean square, times ``weight``, times sigmoid of the
    gate that lies in ``packed`` from column ``gate_column`` on; the result has ``packed``'s dtype."""
    _cuda(o, weight, packed)
    _contig(o, weight, packed)
    _f32(o, weight)
    if packed.shape[1] < gate_column + o.shape[1] or weight.numel() != o.shape[1]:
        raise KernelError("row_norm_gate: the gate's columns or the weight do not fit")
    out = torch.empty(o.shape, dtype=packed.dtype, device=o.device)
    gate = packed.view(-1)[gate_column:]
    rc = _gated().b200_row_norm_gate(_p(out), _p(o), _p(weight), ctypes.c_void_p(gate.data_ptr()), packed.shape[1],
                                     o.shape[0], o.shape[1], ctypes.c_float(eps), _code(packed), _stream())
    _ok(rc, "row_norm_gate")
    return out


def tanh_cap(z: torch.Tensor, cap: float) -> torch.Tensor:
    """z <- cap * tanh(z / cap), in place on float32."""
    _cuda(z)
    _contig(z)
    _f32(z)
    rc = _gated().b200_tanh_cap(_p(z), ctypes.c_longlong(z.numel()), ctypes.c_float(cap), _stream())
    _ok(rc, "tanh_cap")
    return z


# --------------------------------------------------------------------------- a residual of several streams
MAX_STREAMS = 8


def stream_step(streams: torch.Tensor, norm_weight: torch.Tensor, offset: float, eps: float, out_dtype: torch.dtype,
                start: Optional[torch.Tensor] = None, y: Optional[torch.Tensor] = None,
                before: Optional[torch.Tensor] = None, read_in: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None, store: bool = True) -> torch.Tensor:
    """One write-back and read of a residual held as S float32 streams [tokens, S, width].

    With ``start`` ([tokens, width] float32) every stream becomes a copy of it; else, with ``before`` (the packed
    coefficients in[S], out[S], mix[S, S] of the sublayer whose output ``y`` is), X_t <- sum_s mix[s, t] X_s +
    out[t] y for all t at once.  Then u = sum_s read_in[s] X_s (ones without ``read_in``) and the result is
    u / sqrt(mean(u^2) + eps) * (norm_weight + offset), rounded once to ``out_dtype``; for ``rows`` only if given.
    ``store`` False leaves the streams unwritten (the model's last read)."""
    _cuda(streams, norm_weight, start, y, before, read_in, rows)
    _contig(streams, norm_weight, start, y, before, read_in, rows)
    _f32(streams, norm_weight, start, before, read_in)
    _i32(rows)
    tokens, s, width = streams.shape
    if not 1 <= s <= MAX_STREAMS or norm_weight.numel() != width:
        raise KernelError(f"stream_step takes 1 to {MAX_STREAMS} streams and a weight per column")
    if before is not None and (y is None or before.numel() != s * (s + 2) or tuple(y.shape) != (tokens, width)):
        raise KernelError("stream_step: the write-back needs y [tokens, width] and in, out, mix of its sublayer")
    if start is not None and tuple(start.shape) != (tokens, width):
        raise KernelError("stream_step: the start must be [tokens, width]")
    if read_in is not None and read_in.numel() != s:
        raise KernelError("stream_step: one read coefficient per stream")
    n = tokens if rows is None else rows.numel()
    out = torch.empty((n, width), dtype=out_dtype, device=streams.device)
    rc = load_cuda_library("residual_streams.cu").b200_stream_step(
        _p(streams), s, _p(start), _p(y), _code(y) if y is not None else F32, _p(before), _p(read_in), _p(norm_weight),
        ctypes.c_float(offset), ctypes.c_float(eps), _p(rows), _p(out), _code(out), n, width, int(bool(store)), _stream())
    _ok(rc, "stream_step")
    return out


# --------------------------------------------------------------------------- between a packed projection and attention
def heads_prepare(x: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                  positions: torch.Tensor, slots: Optional[torch.Tensor], num_heads: int, num_kv_heads: int,
                  head_dim: int, v_head_dim: int, bias: Optional[torch.Tensor] = None,
                  q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                  inv_freq: Optional[torch.Tensor] = None, rot_dims: int = 0, interleaved: bool = True,
                  plain_norm: bool = False, norm_after_rotation: bool = False, values_are_keys: bool = False) -> None:
    """q, k, v are the first columns of ``x``: optional bias (float32, one per column), optional per-head RMS norm
    of q and k (float32 weights over a head; ``plain_norm``: no weights, x / sqrt(mean(x^2) + eps)), optional rotation
    of the first ``rot_dims`` coordinates of every q and k head by position * inv_freq (pairs (2i, 2i+1) if
    ``interleaved`` else (i, i + rot_dims/2)); the norm precedes the rotation unless ``norm_after_rotation``; q to
    ``q_out``, k and v into the paged cache at ``slots`` (None: nothing is stored).  ``values_are_keys``: ``x`` holds
    no v columns and a token's value is its key as projected (biased, neither normed nor rotated)."""
    _cuda(x, q_out, k_cache, v_cache, positions, slots, bias, q_weight, k_weight, inv_freq)
    _contig(x, q_out, k_cache, v_cache, positions, slots, bias, q_weight, k_weight, inv_freq)
    _f32(bias, q_weight, k_weight, inv_freq)
    if values_are_keys and v_head_dim != head_dim:
        raise KernelError("values that are the keys are as wide as the keys")
    c = (num_heads + num_kv_heads) * head_dim + (0 if values_are_keys else num_kv_heads * v_head_dim)
    flags = (1 if plain_norm else 0) | (2 if norm_after_rotation else 0) | (4 if values_are_keys else 0)
    if x.shape[1] < c or q_out.dtype != x.dtype or k_cache.dtype != x.dtype or v_cache.dtype != x.dtype:
        raise KernelError("heads_prepare: the projection is too narrow, or q, cache and projection differ in dtype")
    if tuple(k_cache.shape[1:]) != (num_kv_heads, k_cache.shape[2], head_dim) or \
            tuple(v_cache.shape[1:]) != (num_kv_heads, k_cache.shape[2], v_head_dim):
        raise KernelError("the cache must be [pages + 1, kv_heads, page_size, width]")
    if (bias is not None and bias.numel() != c) or (q_weight is None) != (k_weight is None) or \
            (q_weight is not None and (q_weight.numel() != head_dim or k_weight.numel() != head_dim)):
        raise KernelError("heads_prepare: bias or norm weights of the wrong size")
    if inv_freq is not None and inv_freq.numel() * 2 != rot_dims:
        raise KernelError("one frequency for every rotated pair is needed")
    page_size = k_cache.shape[2]
    rc = load_cuda_library("attention_prepare.cu").b200_heads_prepare(
        _p(x), _code(x), x.shape[1], _p(bias), _p(q_weight), _p(k_weight), ctypes.c_float(eps), _p(inv_freq),
        int(rot_dims if inv_freq is not None else 0), int(bool(interleaved)), _p(positions), _p(slots), x.shape[0],
        num_heads, num_kv_heads, head_dim, v_head_dim, flags, page_size,
        ctypes.c_longlong(k_cache.shape[0] * page_size), _p(q_out), _p(k_cache), _p(v_cache),
        _p(error_word(x.device)), _stream())
    _ok(rc, "heads_prepare")


def joint_heads_prepare(x: torch.Tensor, q_out: torch.Tensor, k_cache: Optional[torch.Tensor],
                        v_cache: Optional[torch.Tensor], positions: torch.Tensor, slots: Optional[torch.Tensor],
                        num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, has_kv: bool = True,
                        bias: Optional[torch.Tensor] = None, q_weight: Optional[torch.Tensor] = None,
                        k_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                        inv_freq: Optional[torch.Tensor] = None, rot_dims: int = 0, interleaved: bool = True) -> None:
    """As ``heads_prepare``, but the RMS norm of q runs over all of a token's q columns at once (before they are split
    into heads; ``q_weight`` has num_heads * head_dim entries) and the norm of k over all of its k columns.
    ``has_kv`` False: ``x`` holds the q columns only (a layer that reads another layer's keys and values); nothing is
    stored and the caches may be None."""
    _cuda(x, q_out, k_cache, v_cache, positions, slots, bias, q_weight, k_weight, inv_freq)
    _contig(x, q_out, k_cache, v_cache, positions, slots, bias, q_weight, k_weight, inv_freq)
    _f32(bias, q_weight, k_weight, inv_freq)
    nq, nk, nv = num_heads * head_dim, num_kv_heads * head_dim, num_kv_heads * v_head_dim
    c = nq + (nk + nv if has_kv else 0)
    if x.shape[1] < c or q_out.dtype != x.dtype or tuple(q_out.shape) != (x.shape[0], nq):
        raise KernelError("joint_heads_prepare: the projection is too narrow, or q and projection differ")
    page_size, cache_slots = 1, 0
    if has_kv:
        if k_cache is None or v_cache is None or k_cache.dtype != x.dtype or v_cache.dtype != x.dtype or \
                tuple(k_cache.shape[1:]) != (num_kv_heads, k_cache.shape[2], head_dim) or \
                tuple(v_cache.shape[1:]) != (num_kv_heads, k_cache.shape[2], v_head_dim):
            raise KernelError("the cache must be [pages + 1, kv_heads, page_size, width] in the projection's dtype")
        page_size, cache_slots = k_cache.shape[2], k_cache.shape[0] * k_cache.shape[2]
    if (bias is not None and bias.numel() != c) or (q_weight is not None and q_weight.numel() != nq) or \
            (has_kv and k_weight is not None and k_weight.numel() != nk):
        raise KernelError("joint_heads_prepare: bias or norm weights of the wrong size")
    if inv_freq is not None and inv_freq.numel() * 2 != rot_dims:
        raise KernelError("one frequency for every rotated pair is needed")
    rc = load_cuda_library("attention_prepare.cu").b200_joint_heads_prepare(
        _p(x), _code(x), x.shape[1], _p(bias), _p(q_weight), _p(k_weight if has_kv else None), ctypes.c_float(eps),
        _p(inv_freq), int(rot_dims if inv_freq is not None else 0), int(bool(interleaved)), _p(positions),
        _p(slots if has_kv else None), x.shape[0], num_heads, num_kv_heads, head_dim, v_head_dim, int(bool(has_kv)),
        page_size, ctypes.c_longlong(cache_slots), _p(q_out), _p(k_cache if has_kv else None),
        _p(v_cache if has_kv else None), _p(error_word(x.device)), _stream())
    _ok(rc, "joint_heads_prepare")


def latent_prepare(x: torch.Tensor, q_lat: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor,
                   v_cache: Optional[torch.Tensor], latent_weight: torch.Tensor, eps: float, positions: torch.Tensor,
                   slots: Optional[torch.Tensor], num_heads: int, head_dim: int, rot_dim: int, latent_dim: int,
                   inv_freq: Optional[torch.Tensor] = None, rot_dims: int = 0, interleaved: bool = True,
                   down: Optional[torch.Tensor] = None) -> None:
    """``x`` holds per head [head_dim plain | rot_dim rotated] query coordinates, then [latent_dim | rot_dim] of the
    down projection; or ``down`` holds the latter (a view with a unit inner stride whose first latent_dim + rot_dim
    columns are read: a column range of another matrix).  The latent is RMS-normed (``latent_weight``) and stored with the rotated key part behind it as
    the token's one key [latent_dim + rot_dim] and, if a value cache is given, alone as its value; the query that meets such keys is
    [q_lat[h, t] | rotated part] and goes to ``q_out`` [tokens, heads * (latent_dim + rot_dim)]."""
    _cuda(x, q_lat, q_out, k_cache, v_cache, latent_weight, positions, slots, inv_freq, down)
    _contig(x, q_lat, q_out, k_cache, v_cache, latent_weight, positions, slots, inv_freq)
    _f32(latent_weight, inv_freq)
    tokens = x.shape[0]
    q_columns = num_heads * (head_dim + rot_dim)
    if down is None:
        down = x[:, q_columns:]
    if down.dim() != 2 or down.shape[0] != tokens or down.shape[1] < latent_dim + rot_dim or down.stride(1) != 1 or \
            down.dtype != x.dtype:
        raise KernelError("latent_prepare: the down projection's rows do not fit")
    if x.shape[1] < q_columns or \
            tuple(q_lat.shape) != (num_heads, tokens, latent_dim) or latent_weight.numel() != latent_dim or \
            q_lat.dtype != x.dtype or q_out.dtype != x.dtype or k_cache.dtype != x.dtype or \
            (v_cache is not None and v_cache.dtype != x.dtype):
        raise KernelError("latent_prepare: sizes or dtypes do not fit")
    if tuple(k_cache.shape[1:]) != (1, k_cache.shape[2], latent_dim + rot_dim) or \
            (v_cache is not None and tuple(v_cache.shape[1:]) != (1, k_cache.shape[2], latent_dim)):
        raise KernelError("the latent cache must be [pages + 1, 1, page_size, latent_dim + rot_dim] and [.., latent_dim]")
    if inv_freq is not None and inv_freq.numel() * 2 != rot_dims:
        raise KernelError("one frequency for every rotated pair is needed")
    page_size = k_cache.shape[2]
    rc = load_cuda_library("attention_prepare.cu").b200_latent_prepare(
        _p(x), _code(x), x.shape[1], ctypes.c_void_p(down.data_ptr()), down.stride(0), _p(q_lat), _p(latent_weight), ctypes.c_float(eps), _p(inv_freq),
        int(rot_dims if inv_freq is not None else 0), int(bool(interleaved)), _p(positions), _p(slots), tokens,
        num_heads, head_dim, rot_dim, latent_dim, page_size, ctypes.c_longlong(k_cache.shape[0] * page_size),
        _p(q_out), _p(k_cache), _p(v_cache), _p(error_word(x.device)), _stream())
    _ok(rc, "latent_prepare")


def columns_rms_norm(x: torch.Tensor, width: int, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm (with ``weight``, float32) of the first ``width`` columns of every row of ``x`` [tokens, >= width]
    (contiguous): a new contiguous [tokens, width] tensor of x's dtype."""
    _cuda(x, weight)
    _contig(x, weight)
    _f32(weight)
    if x.dim() != 2 or x.shape[1] < width or weight.numel() != width:
        raise KernelError("columns_rms_norm: the rows are too narrow or the weight does not fit")
    out = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
    rc = load_cuda_library("attention_prepare.cu").b200_columns_rms_norm(
        _p(x), _code(x), x.shape[1], _p(weight), ctypes.c_float(eps), x.shape[0], int(width), _p(out), _stream())
    _ok(rc, "columns_rms_norm")
    return out


# --------------------------------------------------------------------------- experts chosen by a table or a router
EXPERTS_TCGEN05_FROM_PAIRS = 512      # steps with this many (token, expert) pairs take the tcgen05 products
GLU_KINDS = {"silu": 0, "clamped_swish": 1}


def _experts_buffers(x: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor, top: int, what: str):
    tokens, width = x.shape
    experts, ff2, _ = gate_up.shape
    ff = ff2 // 2
    if gate_up.dtype != x.dtype or down.dtype != x.dtype or tuple(down.shape) != (experts, width, ff) \
            or gate_up.shape[2] != width:
        raise KernelError(f"{what}: sizes or dtypes do not fit")
    lib = load_cuda_library("experts.cu")
    lib.b200_expert_route_ints.restype = ctypes.c_longlong
    pairs = tokens * top
    route = torch.empty(int(lib.b200_expert_route_ints(tokens, top, experts)), dtype=torch.int32, device=x.device)
    h = torch.empty((pairs, ff), dtype=x.dtype, device=x.device)
    y = torch.empty((pairs, width), dtype=torch.float32, device=x.device)
    out = torch.empty((tokens, width), dtype=torch.float32, device=x.device)
    return lib, experts, ff, pairs, route, h, y, out


def _experts_on_tcgen05(x: torch.Tensor, ff: int, pairs: int, tensor_memory: Optional[bool]) -> bool:
    fits = x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and ff % 8 == 0 and pairs >= 128
    if tensor_memory and not fits:
        raise KernelError("the tcgen05 experts take bfloat16 with width and ff multiples of 8")
    return fits and (tensor_memory if tensor_memory is not None else pairs >= EXPERTS_TCGEN05_FROM_PAIRS)


def table_experts(x: torch.Tensor, token_ids: torch.Tensor, table: torch.Tensor, gate_up: torch.Tensor,
                  down: torch.Tensor, tensor_memory: Optional[bool] = None) -> torch.Tensor:
    """out[t] = (1 / top) sum_k down[e] (silu(gate[e] x_t) * (up[e] x_t)), e = table[token_ids[t], k]; float32
    [tokens, width].  gate_up [experts, 2 ff, width] (gate rows, then up rows), down [experts, width, ff].
    bfloat16 steps with many pairs (``EXPERTS_TCGEN05_FROM_PAIRS``) and widths that are whole 16-byte pieces run the
    two products on tcgen05 (``tensor_memory`` asks for or forbids it); the others on the tiled kernels."""
    _cuda(x, token_ids, table, gate_up, down)
    _contig(x, token_ids, table, gate_up, down)
    _i32(token_ids, table)
    tokens, width = x.shape
    vocab, top = table.shape
    if token_ids.numel() != tokens:
        raise KernelError("table_experts: sizes or dtypes do not fit")
    lib, experts, ff, pairs, route, h, y, out = _experts_buffers(x, gate_up, down, top, "table_experts")
    if _experts_on_tcgen05(x, ff, pairs, tensor_memory):
        xs = torch.empty((pairs, width), dtype=x.dtype, device=x.device)
        rc = load_cuda_library("experts_tcgen05.cu").b200_table_experts_tcgen05(
            _p(x), _p(token_ids), _p(table), vocab, top, experts, _p(gate_up), _p(down), tokens, width, ff, _p(xs),
            _p(h), _p(y), _p(route), _p(out), _p(error_word(x.device)), _stream())
        _ok(rc, "table_experts_tcgen05", 5)
        return out
    rc = lib.b200_table_experts(_p(x), _code(x), _p(token_ids), _p(table), vocab, top, experts, _p(gate_up), _p(down),
                                tokens, width, ff, _p(h), _p(y), _p(route), _p(out), _p(error_word(x.device)), _stream())
    _ok(rc, "table_experts", 4)
    return out


def expert_router(x: torch.Tensor, weight: torch.Tensor, top: int, groups: int = 1, keep: int = 1,
                  scores: str = "softmax", renormalize: bool = False, correction: Optional[torch.Tensor] = None,
                  group_members: int = 1, gain_scale: float = 1.0, gate: Optional[torch.Tensor] = None):
    """A router's choice for every token: logits = weight x in float (FFMA, whatever the dtypes), scores = softmax over
    all experts (or ``sigmoid`` of each).  The choice compares scores + ``correction`` (float32, one an expert; None:
    the scores): the experts form ``groups`` equal groups of neighbours, a group's score is the sum of its
    ``group_members`` largest (1: its largest), and only experts of the ``keep`` best groups can be chosen; the ``top``
    largest of those are.  Returns (choice int32 [tokens, top], weights float32 [tokens, top]): the chosen experts'
    scores (without the correction), divided by their sum if ``renormalize``, times ``gain_scale``.  Ties go to the
    lower index.  ``gate`` (one more row [1, width] of the weight's dtype): a third result, sigmoid(gate x) as float32
    [tokens], summed like a logit."""
    _cuda(x, weight, correction, gate)
    _contig(x, weight, correction, gate)
    _f32(correction)
    tokens, width = x.shape
    experts = weight.shape[0]
    if weight.shape[1] != width or scores not in ("softmax", "sigmoid") or \
            (correction is not None and correction.numel() != experts) or \
            (gate is not None and (gate.numel() != width or gate.dtype != weight.dtype)):
        raise KernelError("expert_router: the router's matrix, correction or gate does not fit, or unknown scores")
    choice = torch.empty((tokens, top), dtype=torch.int32, device=x.device)
    gains = torch.empty((tokens, top), dtype=torch.float32, device=x.device)
    gate_out = torch.empty((tokens,), dtype=torch.float32, device=x.device) if gate is not None else None
    rc = load_cuda_library("experts.cu").b200_expert_router(
        _p(x), _code(x), _p(weight), _code(weight), tokens, width, experts, int(groups), int(keep), int(top),
        int(scores == "sigmoid"), int(bool(renormalize)), _p(correction), int(group_members),
        ctypes.c_float(gain_scale), _p(gate), _p(gate_out), _p(choice), _p(gains), _stream())
    _ok(rc, "expert_router")
    return (choice, gains) if gate is None else (choice, gains, gate_out)


def routed_experts(x: torch.Tensor, choice: torch.Tensor, gains: torch.Tensor, gate_up: torch.Tensor,
                   down: torch.Tensor, glu: str = "silu", limit: float = 0.0, alpha: float = 1.0,
                   add: Optional[torch.Tensor] = None, tensor_memory: Optional[bool] = None,
                   add_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = sum_k gains[t, k] down[e] glu(gate[e] x_t, up[e] x_t) (+ add_scale[t] * add[t]), e = choice[t, k]; float32
    [tokens, width].  ``glu``: "silu" (silu(g) u) or "clamped_swish" (g' sigmoid(alpha g') (u' + 1), g' = min(g, limit),
    u' = clamp(u, -limit, limit)).  ``add`` [tokens, width] (float32 or x's dtype) joins the sum in float: what every
    token gets besides its experts, times ``add_scale`` (float32 [tokens]; None: 1).  Weights and the choice of product
    kernels as in ``table_experts``."""
    _cuda(x, choice, gains, gate_up, down, add, add_scale)
    _contig(x, choice, gains, gate_up, down, add, add_scale)
    _i32(choice)
    _f32(gains, add_scale)
    if add_scale is not None and (add is None or add_scale.numel() != x.shape[0]):
        raise KernelError("routed_experts: add_scale needs add and one factor a token")
    tokens, width = x.shape
    top = choice.shape[1]
    if glu not in GLU_KINDS or tuple(choice.shape) != (tokens, top) or tuple(gains.shape) != (tokens, top) or \
            (add is not None and (tuple(add.shape) != (tokens, width) or add.dtype not in (torch.float32, x.dtype))):
        raise KernelError("routed_experts: sizes or dtypes do not fit")
    lib, experts, ff, pairs, route, h, y, out = _experts_buffers(x, gate_up, down, top, "routed_experts")
    add_code = _code(add) if add is not None else F32
    if _experts_on_tcgen05(x, ff, pairs, tensor_memory):
        xs = torch.empty((pairs, width), dtype=x.dtype, device=x.device)
        rc = load_cuda_library("experts_tcgen05.cu").b200_routed_experts_tcgen05(
            _p(x), _p(choice), _p(gains), top, experts, _p(gate_up), _p(down), tokens, width, ff, GLU_KINDS[glu],
            ctypes.c_float(limit), ctypes.c_float(alpha), _p(add), add_code, _p(add_scale), _p(xs), _p(h), _p(y),
            _p(route), _p(out),
            _p(error_word(x.device)), _stream())
        _ok(rc, "routed_experts_tcgen05", 5)
        return out
    rc = lib.b200_routed_experts(_p(x), _code(x), _p(choice), _p(gains), top, experts, _p(gate_up), _p(down), tokens,
                                 width, ff, GLU_KINDS[glu], ctypes.c_float(limit), ctypes.c_float(alpha), _p(add),
                                 add_code, _p(add_scale), _p(h), _p(y), _p(route), _p(out), _p(error_word(x.device)),
                                 _stream())
    _ok(rc, "routed_experts", 4)
    return out


def glu_columns(gate_up: torch.Tensor, glu: str = "silu", limit: float = 0.0, alpha: float = 1.0) -> torch.Tensor:
    """out = glu(gate_up[:, :F], gate_up[:, F:]) with the forms of ``routed_experts``; computed in float, rounded once."""
    _cuda(gate_up)
    _contig(gate_up)
    tokens, width2 = gate_up.shape
    if width2 % 2 or glu not in GLU_KINDS:
        raise KernelError("glu_columns needs an even width and a known form")
    out = torch.empty((tokens, width2 // 2), dtype=gate_up.dtype, device=gate_up.device)
    rc = _gated().b200_glu_columns(_p(out), _p(gate_up), tokens, width2 // 2, GLU_KINDS[glu], ctypes.c_float(limit),
                                   ctypes.c_float(alpha), _code(gate_up), _stream())
    _ok(rc, "glu_columns")
    return out


def add_row_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """y[t] += bias (float32, one per column), in place; the sum is taken in float and rounded once."""
    _cuda(y, bias)
    _contig(y, bias)
    _f32(bias)
    if y.dim() != 2 or bias.numel() != y.shape[1]:
        raise KernelError("add_row_bias: one bias per column of y [tokens, width]")
    rc = _gated().b200_add_row_bias(_p(y), _p(bias), y.shape[0], y.shape[1], _code(y), _stream())
    _ok(rc, "add_row_bias")
    return y


def act_table_mul(z: torch.Tensor, act: str, table: torch.Tensor, ids: torch.Tensor, column: int) -> torch.Tensor:
    """out[t, c] = act(z[t, c]) * table[ids[t], column + c]: a gate on a token's row of a second embedding table."""
    _cuda(z, table, ids)
    _contig(z, table, ids)
    _i32(ids)
    tokens, dim = z.shape
    if act not in ACTIVATIONS or table.dtype != z.dtype or ids.numel() != tokens or column + dim > table.shape[1]:
        raise KernelError("act_table_mul: sizes or dtypes do not fit")
    out = torch.empty_like(z)
    rc = _gated().b200_act_table_mul(_p(out), _p(z), _p(table), _p(ids), tokens, table.shape[0], table.shape[1],
                                     int(column), dim, ACTIVATIONS[act], _code(z), _p(error_word(z.device)), _stream())
    _ok(rc, "act_table_mul")
    return out


TOKEN_SIDE_FEW = 16     # a step of at most this many tokens takes the one-kernel form of the token table's gated read


def token_side_few(stream: torch.Tensor, x: torch.Tensor, gate: torch.Tensor, table: torch.Tensor, ids: torch.Tensor,
                   column: int, proj: torch.Tensor, norm: torch.Tensor, eps: float, act: str,
                   cast_to: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """For a step of few tokens, in one kernel: g = act(gate x) * table[ids, column : column + dim]; y = proj g;
    stream <- stream + y / sqrt(mean(y^2) + eps) * norm, in place on the float32 ``stream``.  ``x`` is the stream
    rounded to the dtype of gate, table and proj (the stream itself in float32).  Returns as ``norm_add`` does."""
    _cuda(stream, x, gate, table, ids, proj, norm)
    _contig(stream, x, gate, table, ids, proj, norm)
    _f32(stream, norm)
    _i32(ids)
    tokens, width = stream.shape
    dim = gate.shape[0]
    if act not in ACTIVATIONS or tuple(x.shape) != (tokens, width) or tuple(gate.shape) != (dim, width) or \
            tuple(proj.shape) != (width, dim) or norm.numel() != width or ids.numel() != tokens or \
            not (x.dtype == gate.dtype == table.dtype == proj.dtype) or column + dim > table.shape[1]:
        raise KernelError("token_side_few: sizes or dtypes do not fit")
    out = None
    if cast_to is not None and cast_to != torch.float32:
        if cast_to != x.dtype:
            raise KernelError("token_side_few: the rounded copy has the dtype of x")
        out = torch.empty((tokens, width), dtype=cast_to, device=x.device)
    rc = _gated().b200_token_side_few(
        _p(stream), _p(x), _p(gate), _p(table), _p(ids), _p(proj), _p(norm), ctypes.c_float(eps), _p(out), tokens,
        table.shape[0], table.shape[1], int(column), dim, width, ACTIVATIONS[act], _code(x), _p(error_word(x.device)),
        _stream())
    _ok(rc, "token_side_few")
    if cast_to is None:
        return None
    return out if out is not None else stream


# --------------------------------------------------------------------------- a float stream with norms on the outputs
def norm_add(x: torch.Tensor, y: torch.Tensor, weight: torch.Tensor, eps: float, bias: Optional[torch.Tensor] = None,
             cast_to: Optional[torch.dtype] = None) -> Optional[torch.Tensor]:
    """x <- x + (y + bias) / sqrt(mean((y + bias)^2) + eps) * weight, in place on the float32 stream x [tokens, width];
    y float32 or bfloat16, weight and bias float32.  With ``cast_to`` the new x is also returned rounded once to that
    dtype (float32: x itself is returned)."""
    _cuda(x, y, weight, bias)
    _contig(x, y, weight, bias)
    _f32(x, weight, bias)
    tokens, width = x.shape
    if tuple(y.shape) != (tokens, width) or weight.numel() != width or (bias is not None and bias.numel() != width):
        raise KernelError("norm_add: y, the weight or the bias do not fit the stream")
    out = None
    if cast_to is not None and cast_to != torch.float32:
        out = torch.empty((tokens, width), dtype=cast_to, device=x.device)
    rc = load_cuda_library("post_norm.cu").b200_norm_add(
        _p(x), _p(y), _code(y), _p(bias), _p(weight), ctypes.c_float(eps), _p(out),
        _code(out) if out is not None else F32, tokens, width, _stream())
    _ok(rc, "norm_add")
    if cast_to is None:
        return None
    return out if out is not None else x


def norm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
              rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[r] = x[rows[r]] / sqrt(mean(x[rows[r]]^2) + eps) * weight for the float32 stream x (every row without
    ``rows``), rounded once to ``out_dtype``."""
    _cuda(x, weight, rows)
    _contig(x, weight, rows)
    _f32(x, weight)
    _i32(rows)
    width = x.shape[1]
    if weight.numel() != width:
        raise KernelError("norm_rows: one weight per column is needed")
    n = x.shape[0] if rows is None else rows.numel()
    out = torch.empty((n, width), dtype=out_dtype, device=x.device)
    rc = load_cuda_library("post_norm.cu").b200_norm_rows(_p(out), _code(out), _p(x), _p(rows), _p(weight),
                                                          ctypes.c_float(eps), n, width, _stream())
    _ok(rc, "norm_rows")
    return out
