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
if hasattr(torch, "float8_e8m0fnu"):
    _DT[torch.float8_e8m0fnu] = _lib.PTO_UINT8          # E8M0 scale codes travel as bytes

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
    if code == 3:
        raise _lib.PtoError(1, f"index or row count outside its array, access skipped (site {site}, CTA {cta}, "
                               f"value {extra})")
    if code != 0:
        raise _lib.PtoError(2, f"device error word {code} (site {site}, CTA {cta}, value {extra})")


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


# ---------------------------------------------------------------------------
# tensor-core linear algebra and decoder-layer glue
# ---------------------------------------------------------------------------

def _err_ptr(dev) -> int:
    return scratch(dev, 256).data_ptr()


def pack_weight(w: torch.Tensor) -> torch.Tensor:
    """[K, N] fp32/bf16 (the ``x @ W`` layout) -> packed [N, K] bf16, once per weight."""
    dev = _need_cuda(w)
    if w.dim() != 2 or w.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError("pack_weight expects a 2-D fp32 or bf16 tensor")
    k, n = w.shape
    out = torch.empty(n, k, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_pack_weight(w.data_ptr(), dtype_code(w.dtype), out.data_ptr(), k, n,
                                               _stream_ptr(dev)))
    return out


def cast(x: torch.Tensor, dtype: torch.dtype, zero: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 <-> bf16 element cast; ``zero`` (contiguous, 16-byte aligned, a multiple of 16 bytes) is cleared by
    the same launch."""
    dev = _need_cuda(x)
    out = torch.empty(x.shape, dtype=dtype, device=dev)
    zb = 0
    if zero is not None:
        _need_cuda(zero)
        zb = zero.numel() * zero.element_size()
        if zb % 16 or zero.data_ptr() % 16:
            raise ValueError("cast: the tensor to clear must be 16-byte aligned and a multiple of 16 bytes")
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_cast_zero(x.data_ptr(), dtype_code(x.dtype), out.data_ptr(), dtype_code(dtype),
                                             x.numel(), zero.data_ptr() if zero is not None else None, zb,
                                             _stream_ptr(dev)))
    return out


def linear(x: torch.Tensor, w_packed: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False):
    """fp32 out[m, n] (+)= x[m, k] @ W with W packed [n, k] bf16, x bf16."""
    dev = _need_cuda(x, w_packed)
    if x.dtype != torch.bfloat16 or w_packed.dtype != torch.bfloat16:
        raise TypeError("linear: x and packed weight must be bfloat16")
    m, k = x.shape
    n, k2 = w_packed.shape
    if k != k2:
        raise ValueError(f"linear: x has k={k}, packed weight has k={k2}")
    if out is None:
        if accumulate:
            raise ValueError("linear: accumulate needs an existing output")
        out = torch.empty(m, n, dtype=torch.float32, device=dev)
    elif out.dtype != torch.float32 or tuple(out.shape) != (m, n) or not out.is_contiguous():
        raise ValueError("linear: out must be a contiguous fp32 [m, n] tensor")
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_linear(x.data_ptr(), w_packed.data_ptr(), out.data_ptr(), m, n, k,
                                          1 if accumulate else 0, _err_ptr(dev), _stream_ptr(dev)))
    return out


_ffn_ws: dict = {}


def ffn_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor, out: torch.Tensor | None = None,
               accumulate: bool = False):
    """fp32 out[m, n_out] (+)= bf16(silu(x Wg) * (x Wu)) Wd; packed weights
    (w_gate_up [2*inter, k] gate rows first, w_down [n_out, inter]); x bf16, or fp32 (rounded to bf16 operands by the
    operator itself: one launch for at most 128 rows)."""
    dev = _need_cuda(x, w_gate_up, w_down)
    if any(t.dtype != torch.bfloat16 for t in (w_gate_up, w_down)) or x.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("ffn_swiglu: packed weights must be bfloat16, x bfloat16 or float32")
    if not x.is_contiguous():
        raise ValueError("ffn_swiglu: x must be contiguous")
    m, k = x.shape
    inter = w_gate_up.shape[0] // 2
    n_out = w_down.shape[0]
    if w_gate_up.shape != (2 * inter, k) or w_down.shape != (n_out, inter):
        raise ValueError("ffn_swiglu: weight shapes do not match [2*inter, k] / [n_out, inter]")
    if out is None:
        if accumulate:
            raise ValueError("ffn_swiglu: accumulate needs an existing output")
        out = torch.empty(m, n_out, dtype=torch.float32, device=dev)
    elif out.dtype != torch.float32 or tuple(out.shape) != (m, n_out) or not out.is_contiguous():
        raise ValueError("ffn_swiglu: out must be a contiguous fp32 [m, n_out] tensor")
    lib = _lib.load()
    f32 = x.dtype == torch.float32
    need = lib.pto_ffn_swiglu_f32_workspace_bytes(m, k, inter) if f32 else lib.pto_ffn_swiglu_workspace_bytes(m, inter)
    key = (dev.index, _stream_ptr(dev))
    ws = _ffn_ws.get(key)
    if ws is None or ws.numel() < need:
        # zeroed once: the one-launch kernel for small batches keeps its call counter in the first bytes
        ws = _ffn_ws[key] = torch.zeros(need, dtype=torch.uint8, device=dev)
    entry = lib.pto_ffn_swiglu_f32 if f32 else lib.pto_ffn_swiglu
    with torch.cuda.device(dev):
        _lib.check(entry(x.data_ptr(), w_gate_up.data_ptr(), w_down.data_ptr(), out.data_ptr(), m, k,
                         inter, n_out, ws.data_ptr(), ws.numel(), 1 if accumulate else 0,
                         _err_ptr(dev), _stream_ptr(dev)))
    return out


def rms_norm(x: torch.Tensor, gamma: torch.Tensor | None, eps: float, out_dtype: torch.dtype = torch.bfloat16, *,
             copy_fp32: torch.Tensor | None = None, zero: torch.Tensor | None = None):
    """RMSNorm of the rows of x.  Optional side jobs of the same launch: ``copy_fp32`` (fp32, shape of x)
    receives x unchanged as fp32, ``zero`` (any contiguous tensor whose byte size is a multiple of 16) is
    cleared."""
    dev = _need_cuda(x) if gamma is None else _need_cuda(x, gamma)
    if gamma is not None and (gamma.dtype != torch.float32 or gamma.numel() != x.shape[-1]):
        raise ValueError("rms_norm: gamma must be fp32 with hidden elements")
    hidden = x.shape[-1]
    if copy_fp32 is not None:
        _need_cuda(copy_fp32)
        if copy_fp32.dtype != torch.float32 or copy_fp32.shape != x.shape or not copy_fp32.is_contiguous():
            raise ValueError("rms_norm: copy_fp32 must be a contiguous fp32 tensor of the shape of x")
    zero_bytes = 0
    if zero is not None:
        _need_cuda(zero)
        zero_bytes = zero.numel() * zero.element_size()
        if not zero.is_contiguous() or zero_bytes % 16 or zero.data_ptr() % 16:
            raise ValueError("rms_norm: the tensor to clear must be contiguous, 16-byte aligned, a multiple of 16 bytes")
    out = torch.empty(x.shape, dtype=out_dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_rms_norm_ex(
            x.data_ptr(), dtype_code(x.dtype), gamma.data_ptr() if gamma is not None else None, out.data_ptr(),
            dtype_code(out_dtype), x.numel() // hidden, hidden, float(eps),
            copy_fp32.data_ptr() if copy_fp32 is not None else None, zero.data_ptr() if zero is not None else None,
            zero_bytes, _stream_ptr(dev)))
    return out


def rope_kv_append(qkv, seq_lens, cos, sin, block_table, k_cache, v_cache, *, num_heads, kv_heads, head_dim,
                   block_size, q_out=None):
    """RoPE on Q/K at pos = seq_len - 1 + paged cache append; returns rotated Q (bf16)."""
    dev = _need_cuda(qkv, seq_lens, cos, sin, block_table, k_cache, v_cache)
    batch = seq_lens.numel()
    if qkv.dtype != torch.float32 or qkv.numel() != batch * (num_heads + 2 * kv_heads) * head_dim:
        raise ValueError("rope_kv_append: qkv must be fp32 [batch, (num_heads + 2*kv_heads) * head_dim]")
    if cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape != sin.shape or cos.shape[-1] != head_dim:
        raise ValueError("rope_kv_append: cos/sin must be fp32 [rows, head_dim]")
    if seq_lens.dtype != torch.int32 or block_table.dtype != torch.int32:
        raise TypeError("rope_kv_append: seq_lens and block_table must be int32")
    if k_cache.dtype != torch.bfloat16 or v_cache.dtype != torch.bfloat16:
        raise TypeError("rope_kv_append: caches must be bfloat16")
    rows = k_cache.numel() // head_dim
    pool_blocks = rows // (kv_heads * block_size)
    if q_out is None:
        q_out = torch.empty(batch * num_heads, head_dim, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_rope_kv_append(
            qkv.data_ptr(), seq_lens.data_ptr(), cos.data_ptr(), sin.data_ptr(), cos.shape[0],
            block_table.data_ptr(), block_table.numel() // max(batch, 1), k_cache.data_ptr(), v_cache.data_ptr(),
            q_out.data_ptr(), batch, num_heads, kv_heads, head_dim, block_size, pool_blocks, _err_ptr(dev),
            _stream_ptr(dev)))
    return q_out


def llama_mini(hidden, causal_mask, cos_emb, sin_emb, wq, wk, wv, w_dense, w_gate, w_up, w_down, w_lm) -> torch.Tensor:
    """The reference's minimal LLaMA forward pass (examples/models/08_llama_mini.py:384-483), fp32 -> logits [S, V]."""
    ts = (hidden, causal_mask, cos_emb, sin_emb, wq, wk, wv, w_dense, w_gate, w_up, w_down, w_lm)
    dev = _need_cuda(*ts)
    if any(t.dtype != torch.float32 or not t.is_contiguous() or t.dim() != 2 for t in ts):
        raise TypeError("llama_mini: all tensors must be contiguous 2-D float32")
    s, d = hidden.shape
    v = w_lm.shape[1]
    want = [(s, d), (s, s), (s, d // 2), (s, d // 2)] + [(d, d)] * 7 + [(d, v)]
    if [tuple(t.shape) for t in ts] != want:
        raise ValueError(f"llama_mini: shapes {[tuple(t.shape) for t in ts]} do not match {want}")
    out = torch.empty(s, v, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_llama_mini(*[t.data_ptr() for t in ts], out.data_ptr(), s, d, v, _stream_ptr(dev)))
    return out


def swiglu_act(gate_up: torch.Tensor) -> torch.Tensor:
    dev = _need_cuda(gate_up)
    rows, two_i = gate_up.shape
    out = torch.empty(rows, two_i // 2, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_swiglu_act(gate_up.data_ptr(), out.data_ptr(), rows, two_i // 2, _stream_ptr(dev)))
    return out


# ---------------------------------------------------------------------------
# mixture of experts
# ---------------------------------------------------------------------------

FP8 = torch.float8_e4m3fn


def moe_topk(scores: torch.Tensor, bias: torch.Tensor | None, topk: int, is_logits: bool = False):
    """(indices int32 [T, k], weights fp32 [T, k]); selection on score + bias, ties to the lower id."""
    dev = _need_cuda(scores) if bias is None else _need_cuda(scores, bias)
    if scores.dtype != torch.float32 or scores.dim() != 2:
        raise TypeError("moe_topk: scores must be fp32 [tokens, experts]")
    t, e = scores.shape
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != e):
        raise ValueError("moe_topk: bias must be fp32 [experts]")
    idx = torch.empty(t, topk, dtype=torch.int32, device=dev)
    w = torch.empty(t, topk, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_topk(scores.data_ptr(), bias.data_ptr() if bias is not None else None,
                                            1 if is_logits else 0, t, e, topk, idx.data_ptr(), w.data_ptr(),
                                            _stream_ptr(dev)))
    return idx, w


def quantize_rows(x: torch.Tensor):
    """(q e4m3 [rows, cols], scale fp32 [rows, cols/128]) with scale = amax/448 per 128 columns."""
    dev = _need_cuda(x)
    if x.dim() != 2 or x.shape[1] % 128 or x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("quantize_rows: x must be bf16/fp32 [rows, cols] with cols % 128 == 0")
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=FP8, device=dev)
    s = torch.empty(rows, cols // 128, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_quantize_rows(x.data_ptr(), dtype_code(x.dtype), q.data_ptr(), s.data_ptr(), rows,
                                                 cols, _stream_ptr(dev)))
    return q, s


def moe_dispatch_plan(expert_of: torch.Tensor, buckets: int):
    """counts [buckets], offsets [buckets+1], pos [routes], route_at [routes] (all int32).  An expert id
    outside [0, buckets) is never dereferenced: it sets the device error word (``check_device_status``)."""
    dev = _need_cuda(expert_of)
    if expert_of.dtype != torch.int32:
        raise TypeError("moe_dispatch_plan: expert ids must be int32")
    n = expert_of.numel()
    counts = torch.empty(buckets, dtype=torch.int32, device=dev)
    offsets = torch.empty(buckets + 1, dtype=torch.int32, device=dev)
    pos = torch.empty(n, dtype=torch.int32, device=dev)
    route_at = torch.empty(n, dtype=torch.int32, device=dev)
    tmp = torch.empty(n + buckets, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_dispatch_plan(expert_of.data_ptr(), n, buckets, counts.data_ptr(),
                                                     offsets.data_ptr(), pos.data_ptr(), route_at.data_ptr(),
                                                     tmp.data_ptr(), _err_ptr(dev), _stream_ptr(dev)))
    return counts, offsets, pos, route_at


def moe_recv_plan(recv_counts: torch.Tensor, capacity: int, slot_stride: int = 0):
    """Receiver plan from recv_counts int32 [world, L]: (counts [L], offsets [L+1], arrival_of [capacity],
    grouped_of [capacity]).  slot_stride > 0 lays expert e out at rows [e*slot_stride, (e+1)*slot_stride)."""
    dev = _need_cuda(recv_counts)
    if recv_counts.dtype != torch.int32 or recv_counts.dim() != 2:
        raise TypeError("moe_recv_plan: recv_counts must be int32 [world, local_experts]")
    world, L = recv_counts.shape
    counts = torch.empty(L, dtype=torch.int32, device=dev)
    offsets = torch.empty(L + 1, dtype=torch.int32, device=dev)
    arrival_of = torch.empty(max(capacity, 1), dtype=torch.int32, device=dev)
    grouped_of = torch.empty(max(capacity, 1), dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_recv_plan(recv_counts.data_ptr(), world, L, slot_stride, capacity,
                                                 counts.data_ptr(), offsets.data_ptr(), arrival_of.data_ptr(),
                                                 grouped_of.data_ptr(), _err_ptr(dev), _stream_ptr(dev)))
    return counts, offsets, arrival_of, grouped_of


def _row_bytes(t: torch.Tensor) -> int:
    return (t.numel() // t.shape[0]) * t.element_size() if t.shape[0] else 0


def gather_rows(sources: list, index: torch.Tensor | None, div: int = 1, rows: int | None = None):
    """dst_i[p] = src_i[index[p] // div] for up to three 2-D (or 1-D) tensors; bit-exact copies.  index -1
    gives a zero row; any other index outside the source sets the device error word."""
    import ctypes as C
    dev = _need_cuda(*sources) if index is None else _need_cuda(*sources, index)
    n = len(sources)
    if not 1 <= n <= 3:
        raise ValueError("gather_rows: 1..3 source tensors")
    rows = (index.numel() if index is not None else sources[0].shape[0]) if rows is None else rows
    outs = [torch.empty((rows,) + tuple(s.shape[1:]), dtype=s.dtype, device=dev) for s in sources]
    rb = [_row_bytes(s) for s in sources]
    if rows == 0 or any(b == 0 for b in rb):
        return outs
    src = (C.c_void_p * n)(*[s.data_ptr() for s in sources])
    dst = (C.c_void_p * n)(*[o.data_ptr() for o in outs])
    rbs = (C.c_int * n)(*rb)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_gather_rows(src, dst, rbs, n, index.data_ptr() if index is not None else None,
                                                   div, rows, min(s.shape[0] for s in sources), _err_ptr(dev),
                                                   _stream_ptr(dev)))
    return outs


def move_rows(parts: list, index: torch.Tensor | None, div: int, rows: int, src_rows: int):
    """Strided row mover behind payload packing: ``parts`` is a list of up to three
    (src_ptr, src_stride, dst_ptr, dst_stride, row_bytes) byte descriptions; dst row p of every part receives
    src row index[p] // div (identity without an index)."""
    import ctypes as C
    n = len(parts)
    if not 1 <= n <= 3:
        raise ValueError("move_rows: 1..3 parts")
    if rows == 0:
        return
    dev = torch.device("cuda", torch.cuda.current_device())
    src = (C.c_void_p * n)(*[p[0] for p in parts])
    sst = (C.c_int64 * n)(*[p[1] for p in parts])
    dst = (C.c_void_p * n)(*[p[2] for p in parts])
    dstr = (C.c_int64 * n)(*[p[3] for p in parts])
    rbs = (C.c_int * n)(*[p[4] for p in parts])
    _lib.check(_lib.load().pto_moe_move_rows(src, sst, dst, dstr, rbs, n, index.data_ptr() if index is not None else None,
                                             div, rows, src_rows, _err_ptr(dev), _stream_ptr(dev)))


def scale_rows(x: torch.Tensor, w: torch.Tensor, w_stride: int = 1, count: torch.Tensor | None = None,
               slot_stride: int = 0, out: torch.Tensor | None = None):
    """y[r] = bf16(fp32(x[r]) * w[r * w_stride]) (the reference's stand-in expert); with ``count`` only the first
    count[e] rows of every block of slot_stride rows are written."""
    dev = _need_cuda(x, w)
    if x.dtype != torch.bfloat16 or w.dtype != torch.float32 or x.dim() != 2:
        raise TypeError("scale_rows: x must be bf16 [rows, cols], w fp32")
    out = torch.zeros_like(x) if out is None else out
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_scale_rows(x.data_ptr(), w.data_ptr(), w_stride,
                                              count.data_ptr() if count is not None else None, slot_stride,
                                              x.shape[0], x.shape[1], out.data_ptr(), _stream_ptr(dev)))
    return out


def moe_expert_gemm(swiglu: bool, w: torch.Tensor, w_scale: torch.Tensor, x: torch.Tensor, x_scale: torch.Tensor,
                    offsets: torch.Tensor, route_w: torch.Tensor | None = None, out_rows: torch.Tensor | None = None):
    """Grouped FP8 GEMM over tokens sorted by expert.  w [E, rows, K] e4m3 (K-major), w_scale
    [E, rows/128, K/128]; x [R, K] e4m3, x_scale [R, K/128]; offsets int32 [E+1].
    swiglu: rows = 2*n_out (gate then up), returns bf16(silu(g)*u) [R, n_out];
    else returns bf16 [R, rows] scaled by route_w, row r written at out_rows[r] when a row map is given (rows that
    nothing maps to are left as allocated)."""
    dev = _need_cuda(w, w_scale, x, x_scale, offsets)
    e, w_rows, k = w.shape
    r = x.shape[0]
    n_out = w_rows // 2 if swiglu else w_rows
    if x.shape[1] != k or x_scale.shape != (r, k // 128) or w_scale.shape != (e, w_rows // 128, k // 128):
        raise ValueError("moe_expert_gemm: operand shapes do not match")
    if offsets.dtype != torch.int32 or offsets.numel() != e + 1:
        raise ValueError("moe_expert_gemm: offsets must be int32 [experts + 1]")
    out = torch.empty(r, n_out, dtype=torch.bfloat16, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_expert_gemm(
            1 if swiglu else 0, w.data_ptr(), w_scale.data_ptr(), e, w_rows, n_out, k, x.data_ptr(),
            x_scale.data_ptr(), offsets.data_ptr(), r, route_w.data_ptr() if route_w is not None else None,
            out_rows.data_ptr() if out_rows is not None else None, out.data_ptr(), _err_ptr(dev), _stream_ptr(dev)))
    return out


def moe_combine(rows: torch.Tensor, pos: torch.Tensor, shared: torch.Tensor | None, tokens: int, topk: int,
                want_f32: bool = False):
    dev = _need_cuda(rows, pos) if shared is None else _need_cuda(rows, pos, shared)
    hidden = rows.shape[1]
    y = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
    y32 = torch.empty(tokens, hidden, dtype=torch.float32, device=dev) if want_f32 else None
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_combine(rows.data_ptr(), pos.data_ptr(),
                                               shared.data_ptr() if shared is not None else None, tokens, topk, hidden,
                                               rows.shape[0], y.data_ptr(), y32.data_ptr() if want_f32 else None,
                                               _stream_ptr(dev)))
    return (y, y32) if want_f32 else y


def moe_push_rows(rows: torch.Tensor, recv_counts: torch.Tensor, dst_base: torch.Tensor, back: list, flags: list,
                  my_rank: int, step: int, done_counter: torch.Tensor) -> None:
    """The expert-parallel layer's return path as a call of its own: ``rows`` [n, cols] (arrival order, recv_counts
    int32 [world, local_experts] rows from each source) go block by block to ``back[r][dst_base[r]:]``, then
    ``flags[r][my_rank] = step``.  ``back`` / ``flags``: one tensor per rank, of this process (tensors of other ranks
    would be ones mapped from their CUDA IPC handles)."""
    import ctypes as C
    dev = _need_cuda(rows, recv_counts, dst_base, done_counter, *back, *flags)
    world, local_experts = recv_counts.shape
    if len(back) != world or len(flags) != world:
        raise ValueError("moe_push_rows: one result buffer and one flag array per rank")
    row_bytes = rows.shape[1] * rows.element_size()
    if any(b.shape[1:] != rows.shape[1:] or b.dtype != rows.dtype or not b.is_contiguous() for b in back):
        raise ValueError("moe_push_rows: result buffers must be contiguous with the rows' width and dtype")
    bp = (C.c_void_p * world)(*[b.data_ptr() for b in back])
    fp = (C.c_void_p * world)(*[f.data_ptr() for f in flags])
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_push_rows(rows.data_ptr(), row_bytes, recv_counts.data_ptr(), world, local_experts,
                                                 dst_base.data_ptr(), bp, fp, my_rank, step, min(b.shape[0] for b in back),
                                                 rows.shape[0], done_counter.data_ptr(), _err_ptr(dev), _stream_ptr(dev)))


def moe_wait_flags(flags: torch.Tensor, world: int, step: int) -> None:
    """Waits on the device (at most two seconds) until ``flags[r] >= step`` for every rank; a rank that does not show
    ends up in the device error word (``check_device_status``)."""
    dev = _need_cuda(flags)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_moe_wait_flags(flags.data_ptr(), world, step, _err_ptr(dev), _stream_ptr(dev)))


# ---------------------------------------------------------------------------
# MX block-scaled FP8 matmul
# ---------------------------------------------------------------------------

MX_SCALE_LOGICAL, MX_SCALE_A_ZZ, MX_SCALE_B_NN = 0, 1, 2


def transpose_u8(x: torch.Tensor) -> torch.Tensor:
    """[rows, cols] of one-byte elements -> [cols, rows] (operand re-layout for ``matmul_mx``)."""
    dev = _need_cuda(x)
    if x.dim() != 2 or x.element_size() != 1:
        raise TypeError("transpose_u8: a 2-D tensor of one-byte elements is expected")
    out = torch.empty(x.shape[1], x.shape[0], dtype=x.dtype, device=dev)
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_transpose_u8(x.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], _stream_ptr(dev)))
    return out


def matmul_mx(a: torch.Tensor, a_scale: torch.Tensor, b_t: torch.Tensor, b_scale: torch.Tensor, *,
              acc: torch.Tensor | None = None, out: torch.Tensor | None = None,
              a_scale_layout: int = MX_SCALE_LOGICAL, b_scale_layout: int = MX_SCALE_LOGICAL) -> torch.Tensor:
    """fp32 out[m, n] = (acc +) MX matmul of a e4m3 [m, k] and b_t e4m3 [n, k] (K contiguous) with E8M0 scale
    codes a_scale uint8 [m, k/32], b_scale uint8 [k/32, n] (tile.matmul_mx / matmul_mx_acc,
    src/ir/op/tile_ops/matmul_mx.cpp:321-345)."""
    dev = _need_cuda(a, a_scale, b_t, b_scale)
    if a.element_size() != 1 or b_t.element_size() != 1 or a_scale.element_size() != 1 or b_scale.element_size() != 1:
        raise TypeError("matmul_mx: operands are e4m3 (one byte) and scales E8M0 codes (one byte)")
    m, k = a.shape
    n, k2 = b_t.shape
    if k != k2 or k % 32:
        raise ValueError("matmul_mx: both operands need the same K, a multiple of 32")
    if a_scale.numel() != m * (k // 32) or b_scale.numel() != (k // 32) * n:
        raise ValueError("matmul_mx: scale tensors must hold m*k/32 and (k/32)*n codes")
    if out is None:
        out = torch.empty(m, n, dtype=torch.float32, device=dev)
    elif out.dtype != torch.float32 or tuple(out.shape) != (m, n) or not out.is_contiguous():
        raise ValueError("matmul_mx: out must be a contiguous fp32 [m, n] tensor")
    if acc is not None:
        _need_cuda(acc)
        if acc.dtype != torch.float32 or tuple(acc.shape) != (m, n):
            raise ValueError("matmul_mx: acc must be fp32 [m, n]")
    with torch.cuda.device(dev):
        _lib.check(_lib.load().pto_matmul_mx(a.data_ptr(), a_scale.data_ptr(), a_scale_layout, b_t.data_ptr(),
                                             b_scale.data_ptr(), b_scale_layout,
                                             acc.data_ptr() if acc is not None else None, out.data_ptr(), m, n, k,
                                             _err_ptr(dev), _stream_ptr(dev)))
    return out
