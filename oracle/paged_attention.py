"""Oracle for paged-attention decode (test infrastructure, not product code).

Restates the reference golden
  examples/models/04_paged_attention.py:473-541   (canonical rounding order)
  examples/models/09_paged_attention_spmd.py:579-653 (empty-sequence guard)
  tests/st/runtime/framework_and_models/test_paged_attention.py:542-596 (same)

Order of operations per KV block, kept exactly: S = (Q K^T) * scale in fp32,
positions >= valid_len set to -inf, m = rowmax(S) clamped at -1e30,
P = exp(S - m) with masked entries 0, P rounded to bf16, l = rowsum(rounded P),
O_blk = P_bf16 V in fp32, then the online-softmax merge of (m, l, O) in fp32 and
a final O / l (0 where l == 0).

Extensions the reference does not contain -- PARITY UNPINNED, this file is their
only definition:
  * kv_heads > 1 (GQA): query head h reads KV head h // (num_heads // kv_heads);
    the pools are laid out [(block, kv_head, token), head_dim], which for
    kv_heads == 1 is the reference's [(block, token), head_dim].
  * q_len > 1 (speculative verify): query rows are ordered (sequence, draft j,
    head); draft token j sees the first ctx_len - q_len + j + 1 keys, where
    ctx_len already counts the q_len draft tokens stored in the cache.
"""

from __future__ import annotations

import struct

import torch


def pack_config(batch, num_heads, kv_heads, head_dim, block_size, max_blocks, scale):
    """The int64[7] config tensor of 04_paged_attention.py:287 (scale as fp32 bits)."""
    bits = struct.unpack("I", struct.pack("f", float(scale)))[0]
    return torch.tensor(
        [batch, num_heads, kv_heads, head_dim, block_size, max_blocks, bits], dtype=torch.int64
    )


def unpack_scale(config) -> float:
    """Inverse of the scale packing (04_paged_attention.py:489-491)."""
    bits = int(config[6].item()) & 0xFFFFFFFF
    return struct.unpack("f", struct.pack("I", bits))[0]


def paged_attention(
    query: torch.Tensor,
    key_cache: torch.Tensor,
    value_cache: torch.Tensor,
    block_table: torch.Tensor,
    context_lens: torch.Tensor,
    *,
    num_heads: int,
    head_dim: int,
    block_size: int,
    scale: float,
    kv_heads: int = 1,
    q_len: int = 1,
    q_tile: int = 16,
) -> torch.Tensor:
    """Return fp32 out[batch * q_len * num_heads, head_dim].

    query        [batch * q_len * num_heads, head_dim]  (any float dtype)
    key_cache    [pool_blocks * kv_heads * block_size, head_dim]
    value_cache  same shape
    block_table  int32 [batch, max_blocks] or flat
    context_lens int32 [batch]
    """
    batch = int(context_lens.numel())
    group = num_heads // kv_heads
    assert group * kv_heads == num_heads
    rows = q_len * group
    q = query.float().reshape(batch, q_len, num_heads, head_dim)
    kc = key_cache.reshape(-1, kv_heads, block_size, head_dim)
    vc = value_cache.reshape(-1, kv_heads, block_size, head_dim)
    bt = block_table.reshape(batch, -1).long()
    ctx = context_lens.long()
    out = torch.zeros(batch, q_len, num_heads, head_dim, dtype=torch.float32)
    if batch == 0:
        return out.reshape(0, head_dim)
    max_bn = int((int(ctx.max().item()) + block_size - 1) // block_size)
    pos = torch.arange(block_size).reshape(1, 1, block_size)
    # keys visible to each row of a (sequence, kv head) item: [batch, rows]
    draft = torch.arange(rows) // group
    limit = (ctx.reshape(batch, 1) - q_len + draft.reshape(1, rows) + 1).clamp(min=0)
    limit = torch.where(ctx.reshape(batch, 1) > 0, limit, torch.zeros_like(limit))

    for kvh in range(kv_heads):
        h0 = kvh * group
        q_item = q[:, :, h0 : h0 + group, :].reshape(batch, rows, head_dim)
        o_item = torch.zeros(batch, rows, head_dim, dtype=torch.float32)
        for r0 in range(0, rows, q_tile):
            qi = q_item[:, r0 : r0 + q_tile, :]
            lim = limit[:, r0 : r0 + q_tile]
            n = qi.shape[1]
            oi = torch.zeros(batch, n, head_dim, dtype=torch.float32)
            li = torch.zeros(batch, n, 1, dtype=torch.float32)
            mi = torch.zeros(batch, n, 1, dtype=torch.float32)
            for bn in range(max_bn):
                valid = (lim - bn * block_size).clamp(min=0, max=block_size)  # [batch, n]
                if not bool((valid > 0).any()):
                    break
                blk = bt[:, bn]
                kj = kc[blk, kvh].float()  # [batch, block_size, head_dim]
                vj = vc[blk, kvh].float()
                sij = torch.bmm(qi, kj.transpose(1, 2)) * scale
                mask = pos < valid.unsqueeze(-1)  # [batch, n, block_size]
                sij = sij.masked_fill(~mask, float("-inf"))
                mij = sij.max(dim=-1, keepdim=True)[0].clamp(min=-1e30)
                pij = torch.exp(sij - mij).masked_fill(~mask, 0.0)
                pij = pij.to(torch.bfloat16).to(torch.float32)
                lij = pij.sum(dim=-1, keepdim=True)
                oi_new = torch.bmm(pij, vj)
                if bn == 0:
                    oi, li, mi = oi_new, lij, mij
                else:
                    mi_new = torch.maximum(mi, mij)
                    alpha = torch.exp(mi - mi_new)
                    beta = torch.exp(mij - mi_new)
                    li = alpha * li + beta * lij
                    oi = alpha * oi + beta * oi_new
                    mi = mi_new
            o_item[:, r0 : r0 + n, :] = torch.where(li > 0, oi / li, torch.zeros_like(oi))
        out[:, :, h0 : h0 + group, :] = o_item.reshape(batch, q_len, group, head_dim)
    return out.reshape(batch * q_len * num_heads, head_dim)


def golden(tensors: dict, params: dict | None = None) -> None:
    """Same call shape as the reference's ``golden(tensors, params)``: reads the
    int64 config tensor (04_paged_attention.py:287) and fills ``tensors['out']``."""
    cfg = tensors["config"]
    batch, num_heads, kv_heads = int(cfg[0]), int(cfg[1]), int(cfg[2])
    head_dim, block_size = int(cfg[3]), int(cfg[4])
    if "scale" in tensors:  # SPMD variant carries the scale as a [1] fp32 tensor
        scale = float(tensors["scale"][0].item())
    else:
        scale = unpack_scale(cfg)
    out = paged_attention(
        tensors["query"],
        tensors["key_cache"],
        tensors["value_cache"],
        tensors["block_table"],
        tensors["context_lens"],
        num_heads=num_heads,
        head_dim=head_dim,
        block_size=block_size,
        scale=scale,
        kv_heads=max(kv_heads, 1),
        q_len=int((params or {}).get("q_len", 1)),
    )
    tensors["out"][:] = out.reshape(tensors["out"].shape).to(tensors["out"].dtype)
    assert batch == tensors["context_lens"].numel()


def kv_bytes(context_lens: torch.Tensor, kv_heads: int, head_dim: int, elem: int = 2) -> int:
    """Algorithmic KV bytes one decode pass must read: K and V rows of every
    visible token of every sequence and KV head."""
    return int(context_lens.long().sum().item()) * kv_heads * head_dim * elem * 2
