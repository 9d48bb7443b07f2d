"""Oracle for the decoder-layer glue and the whole decode layer
(test infrastructure, not product code).

Restates
  RMSNorm   tests/st/examples/02_intermediate/test_rms_norm.py:35-37 (fp32),
            test_qwen3_decode_scope3_mixed.py:278-280 (bf16 round at the end),
            examples/models/qwen3_jit/kernels/rmsnorm.py:27-89
  RoPE      tests/st/examples/03_llm_models/test_llama_7b_mini_1h.py:83-95 (tables),
            :146-159 (rotate-half); cache write position and bf16 rounding
            examples/models/qwen3_jit/kernels/attention.py:53-79
  layer     examples/models/qwen3_jit/qwen3_decode.py:50-112 (order of scopes),
            test_qwen3_decode_scope3_mixed.py:256-287 (scope-3 rounding points)
The reference example leaves attention between scope 2 and 3 as a placeholder
(qwen3_decode.py:95-99); here the paged-attention oracle fills it, bf16 output.
"""

from __future__ import annotations

import torch

from . import paged_attention as pa


def rms_norm(x, gamma, eps, out_dtype=None):
    """x * rsqrt(mean(x^2) + eps) * gamma with fp32 statistics
    (test_qwen3_decode_scope3_mixed.py:278-280)."""
    xf = x.float()
    var = xf.pow(2).mean(dim=-1, keepdim=True)
    y = xf * torch.rsqrt(var + eps) * gamma.float().reshape(1, -1)
    return y if out_dtype is None else y.to(out_dtype)


def rms_norm_sqrt_div(x, gamma, eps):
    """The fp32 form of test_rms_norm.py:35-37: (x / sqrt(mean_sq + eps)) * gamma."""
    mean_sq = (x**2).sum(dim=-1, keepdim=True) / x.shape[-1]
    return (x / torch.sqrt(mean_sq + eps)) * gamma


def rope_tables(max_seq, head_dim, theta):
    """cos/sin tables [max_seq, head_dim] fp32, the half table repeated twice;
    theta_i = theta^(-2i/head_dim) as in test_llama_7b_mini_1h.py:83-95."""
    half = head_dim // 2
    pos = torch.arange(max_seq).float().unsqueeze(1)
    freqs = torch.arange(half).float()
    inv = 1.0 / (float(theta) ** (2 * freqs / head_dim))
    ang = pos * inv.unsqueeze(0)
    return torch.cat([torch.cos(ang)] * 2, dim=-1), torch.cat([torch.sin(ang)] * 2, dim=-1)


def rope_rotate(x, cos_row, sin_row):
    """Rotate-half on the last dim (attention.py:69-70; test_llama_7b_mini_1h.py:146-159).
    x [..., D]; cos_row/sin_row broadcastable [..., D]."""
    half = x.shape[-1] // 2
    lo, hi = x[..., :half], x[..., half:]
    c_lo, c_hi = cos_row[..., :half], cos_row[..., half:]
    s_lo, s_hi = sin_row[..., :half], sin_row[..., half:]
    return torch.cat([lo * c_lo - hi * s_lo, hi * c_hi + lo * s_hi], dim=-1)


def rope_kv_append(q_proj, k_proj, v_proj, seq_lens, cos, sin, k_cache, v_cache, block_table,
                   *, num_heads, kv_heads, head_dim, block_size):
    """RoPE on Q and K at pos = seq_len - 1, bf16 rounding, and the write of the
    rotated K row and the V row into the paged cache at that position
    (attention.py:53-79).  The reference addresses a contiguous cache row
    b*KVH*MAX_SEQ + ki*MAX_SEQ + pos; here the row is found through the block
    table: ((block_table[b, pos // bs] * kv_heads + ki) * bs + pos % bs).
    Returns q_rot bf16 [batch * num_heads, head_dim]; caches updated in place."""
    batch = q_proj.shape[0]
    pos = seq_lens.long() - 1
    c = cos[pos].unsqueeze(1)  # [batch, 1, D]
    s = sin[pos].unsqueeze(1)
    q = rope_rotate(q_proj.float().reshape(batch, num_heads, head_dim), c, s).bfloat16()
    k = rope_rotate(k_proj.float().reshape(batch, kv_heads, head_dim), c, s).bfloat16()
    v = v_proj.float().reshape(batch, kv_heads, head_dim).bfloat16()
    bt = block_table.reshape(batch, -1).long()
    blk = bt[torch.arange(batch), pos // block_size]
    for ki in range(kv_heads):
        row = (blk * kv_heads + ki) * block_size + pos % block_size
        k_cache[row] = k[:, ki]
        v_cache[row] = v[:, ki]
    return q.reshape(batch * num_heads, head_dim)


def decoder_layer(t: dict, *, num_heads, kv_heads, head_dim, block_size, eps, scale):
    """One decode step of a Llama-style layer; every rounding point follows
    qwen3_decode.py:50-112 and test_qwen3_decode_scope3_mixed.py:269-287.

    t holds: hidden [B,H] bf16, input_rms_weight/post_rms_weight [1,H] fp32,
    wq [H, Hq*D], wk/wv [H, Hkv*D], wo [Hq*D, H], w_gate/w_up [H, I], w_down [I, H]
    (bf16), seq_lens int32 [B], rope_cos/rope_sin [S, D] fp32, k_cache/v_cache
    (paged, updated in place), block_table int32 [B, max_blocks].
    Returns bf16 [B, H]."""
    hidden = t["hidden"]
    normed = rms_norm(hidden, t["input_rms_weight"], eps, torch.bfloat16)
    nf = normed.float()
    q_proj = torch.matmul(nf, t["wq"].float())
    k_proj = torch.matmul(nf, t["wk"].float())
    v_proj = torch.matmul(nf, t["wv"].float())
    q_rot = rope_kv_append(q_proj, k_proj, v_proj, t["seq_lens"], t["rope_cos"], t["rope_sin"],
                           t["k_cache"], t["v_cache"], t["block_table"], num_heads=num_heads,
                           kv_heads=kv_heads, head_dim=head_dim, block_size=block_size)
    attn = pa.paged_attention(q_rot, t["k_cache"], t["v_cache"], t["block_table"], t["seq_lens"],
                              num_heads=num_heads, head_dim=head_dim, block_size=block_size,
                              scale=scale, kv_heads=kv_heads).bfloat16()
    attn = attn.reshape(hidden.shape[0], num_heads * head_dim)
    resid1 = torch.matmul(attn.float(), t["wo"].float()) + hidden.float()
    post = rms_norm(resid1, t["post_rms_weight"], eps, torch.bfloat16)
    pf = post.float()
    gate = torch.matmul(pf, t["w_gate"].float())
    up = torch.matmul(pf, t["w_up"].float())
    act = (gate * torch.sigmoid(gate) * up).bfloat16()
    down = torch.matmul(act.float(), t["w_down"].float())
    return (down + resid1).bfloat16()
