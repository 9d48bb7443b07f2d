"""Torch-tensor front end of the direct C launchers.

Each function takes CUDA tensors, validates shapes and dtypes in Python before any
native call (the reference validates before dispatch too:
python/pypto/runtime/device_runner.py:761-786), and launches on torch's current
stream.  torch supplies device memory and streams only; all arithmetic is in the
library's kernels.  There is no CPU path: CPU tensors raise.
"""

from __future__ import annotations

import math

import torch

from . import _lib

_DT = {torch.float32: _lib.PTO_FP32, torch.bfloat16: _lib.PTO_BF16, torch.float16: _lib.PTO_FP16,
       torch.int32: _lib.PTO_INT32, torch.int64: _lib.PTO_INT64, torch.uint8: _lib.PTO_UINT8}
if hasattr(torch, "float8_e4m3fn"):
    _DT[torch.float8_e4m3fn] = _lib.PTO_FP8E4M3

_scratch: dict[tuple[int, int], torch.Tensor] = {}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DT[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def _need_cuda(*tensors: torch.Tensor) -> torch.device:
    dev = None
    for t in tensors:
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"expected a torch.Tensor, got {type(t).__name__}")
        if not t.is_cuda:
            raise _lib.BackendUnavailable("operators run on CUDA tensors only; there is no CPU fallback")
        if not t.is_contiguous():
            raise ValueError("tensors must be contiguous")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError("tensors are on different devices")
    return dev


def _stream_ptr(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def scratch(dev: torch.device, nbytes: int) -> torch.Tensor:
    """Per (device, stream) scratch buffer; zero-initialised when (re)allocated so the
    error word at its start begins clear."""
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream_ptr(dev))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=dev)
        _scratch[key] = buf
    return buf


def device_status(dev=None, clear: bool = True) -> tuple[int, int, int, int]:
    """Read the device error word of the current stream's scratch buffer
    (code, site, CTA, detail); synchronises."""
    dev = torch.device("cuda", torch.cuda.current_device()) if dev is None else torch.device(dev)
    key = (dev.index if dev.index is not None else torch.cuda.current_device(), _stream_ptr(dev))
    buf = _scratch.get(key)
    if buf is None:
        return (0, 0, 0, 0)
    words = buf[:16].view(torch.int32).cpu().tolist()
    if words[0] != 0 and clear:
        buf[:64].zero_()
    return tuple(words)


def check_device_status(dev=None) -> None:
    code, site, cta, extra = device_status(dev)
    if code == 1:
        raise _lib.PtoError(4, f"device wait timed out (site {site}, CTA {cta}, detail {extra})")
    if code == 2:
        raise _lib.PtoError(1, f"block id or row outside the pool (site {site}, CTA {cta}, value {extra})")


def paged_attention(query, key_cache, value_cache, block_table, context_lens, *, num_heads: int,
                    kv_heads: int = 1, head_dim: int | None = None, block_size: int, scale: float | None = None,
                    q_len: int = 1, out: torch.Tensor | None = None, out_dtype: torch.dtype = torch.bfloat16):
    """Paged-attention decode (examples/models/04_paged_attention.py:272-367 as one kernel).

    query [batch*q_len*num_heads, D] bf16; caches [pool_blocks*kv_heads*block_size, D] bf16;
    block_table int32 [batch, max_blocks] (or flat); context_lens int32 [batch].
    Returns ``out`` (bf16 by default, fp32 if asked or if ``out`` is fp32)."""
    dev = _need_cuda(query, key_cache, value_cache, block_table, context_lens)
    if query.dtype != torch.bfloat16 or key_cache.dtype != torch.bfloat16 or value_cache.dtype != torch.bfloat16:
        raise TypeError("query, key_cache and value_cache must be bfloat16")
    if block_table.dtype != torch.int32 or context_lens.dtype != torch.int32:
        raise TypeError("block_table and context_lens must be int32")
    head_dim = query.shape[-1] if head_dim is None else head_dim
    batch = context_lens.numel()
    if query.numel() != batch * q_len * num_heads * head_dim:
        raise ValueError(f"query has {query.numel()} elements, expected batch*q_len*num_heads*head_dim = "
                         f"{batch * q_len * num_heads * head_dim}")
    if num_heads % kv_heads:
        raise ValueError("num_heads must be a multiple of kv_heads")
    if key_cache.shape != value_cache.shape:
        raise ValueError("key_cache and value_cache shapes differ")
    rows = key_cache.numel() // head_dim
    if rows % (kv_heads * block_size):
        raise ValueError("cache rows must be a multiple of kv_heads*block_size")
    pool_blocks = rows // (kv_heads * block_size)
    if batch and block_table.numel() % batch:
        raise ValueError("block_table size must be a multiple of batch")
    max_blocks = block_table.numel() // batch if batch else 1
    if out is None:
        out = torch.empty(batch * q_len * num_heads, head_dim, dtype=out_dtype, device=dev)
    else:
        _need_cuda(out)
        if out.numel() != query.numel() or out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("out must be bf16 or fp32 with the query's element count")
    if batch == 0:
        return out
    scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)
    lib = _lib.load()
    need = lib.pto_paged_attention_scratch_bytes(batch, num_heads, kv_heads, q_len)
    buf = scratch(dev, need)
    with torch.cuda.device(dev):
        _lib.check(lib.pto_paged_attention(
            query.data_ptr(), key_cache.data_ptr(), value_cache.data_ptr(), block_table.data_ptr(),
            context_lens.data_ptr(), out.data_ptr(), dtype_code(out.dtype), batch, num_heads, kv_heads,
            head_dim, block_size, max_blocks, pool_blocks, q_len, scale, buf.data_ptr(), buf.numel(),
            _stream_ptr(dev)))
    return out


def paged_gather(src, indices, block_table, block_size: int, size: int | None = None, col_off: int = 0,
                 out: torch.Tensor | None = None):
    """out[i, :] = src[block_table[idx // bs] * bs + idx % bs, col_off : col_off + size]
    (pl.paged_gather, src/ir/op/tensor_ops/paged_gather.cpp:63-169).  Bit-exact copy."""
    dev = _need_cuda(src, indices, block_table)
    if src.dim() != 2:
        raise ValueError("src must be 2-D [rows, cols]")
    if indices.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise TypeError("indices and block_table must be int32")
    size = src.shape[1] - col_off if size is None else size
    if col_off < 0 or size < 0 or col_off + size > src.shape[1]:
        raise ValueError("column slice out of range")
    n = indices.numel()
    if out is None:
        out = torch.empty(n, size, dtype=src.dtype, device=dev)
    elif out.dtype != src.dtype or out.numel() != n * size:
        raise ValueError("out must have src's dtype and n_indices*size elements")
    buf = scratch(dev, 256)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_paged_gather(
            src.data_ptr(), src.shape[0], src.shape[1], src.element_size(), indices.data_ptr(), n,
            block_table.data_ptr(), block_table.numel(), block_size, col_off, size, out.data_ptr(),
            buf.data_ptr(), _stream_ptr(dev)))
    return out
