"""Seeded synthetic inputs for the five benchmark workloads and their scaled-down
parity cases (test infrastructure, not product code).

Generation order and distributions follow the reference examples where they
exist: examples/models/01_ffn.py:155-160 (seed 0; x, W_gate, W_up, W_down in that
order), examples/models/04_paged_attention.py:544-584 (bf16 randn Q / K / V, int32
block table and context lengths).  Differences asked for by the workload
definitions: block tables are a random permutation of a pool sized to total need
plus 10 % (the reference draws block ids with replacement, :568-570), context
lengths are uniform in a range, several KV heads, bf16 output.
"""

from __future__ import annotations

import math

import torch

from . import layer as _layer
from . import moe as _moe


def _gen(seed):
    return torch.Generator().manual_seed(seed)


def ffn_inputs(m=128, k=1024, inter=4096, seed=0, w_std=0.02):
    g = _gen(seed)
    x = torch.randn(m, k, generator=g)
    wg = torch.randn(k, inter, generator=g) * w_std
    wu = torch.randn(k, inter, generator=g) * w_std
    wd = torch.randn(inter, k, generator=g) * w_std
    return x, wg, wu, wd


def paged_attention_inputs(batch=64, num_heads=32, kv_heads=8, head_dim=128, block_size=128,
                           ctx_lo=1024, ctx_hi=8192, q_len=1, seed=0, context_lens=None,
                           pool_slack=0.10, kv_dtype=torch.bfloat16):
    """Returns a dict with query, key_cache, value_cache, block_table [batch, max_blocks],
    context_lens, scale and the geometry."""
    g = _gen(seed)
    if context_lens is None:
        ctx = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=g, dtype=torch.int32)
    else:
        ctx = torch.as_tensor(context_lens, dtype=torch.int32)
        batch = ctx.numel()
    n_blk = (ctx.long() + block_size - 1) // block_size
    total = int(n_blk.sum())
    pool_blocks = max(1, math.ceil(total * (1.0 + pool_slack)))
    max_blocks = max(1, int(n_blk.max()) if batch else 1)
    perm = torch.randperm(pool_blocks, generator=g).to(torch.int32)
    bt = torch.zeros(batch, max_blocks, dtype=torch.int32)
    o = 0
    for b in range(batch):
        nb = int(n_blk[b])
        bt[b, :nb] = perm[o : o + nb]
        o += nb
    rows = pool_blocks * kv_heads * block_size
    q = torch.randn(batch * q_len * num_heads, head_dim, generator=g).to(kv_dtype)
    kc = torch.empty(rows, head_dim, dtype=kv_dtype)
    vc = torch.empty(rows, head_dim, dtype=kv_dtype)
    chunk = 1 << 16
    for r0 in range(0, rows, chunk):  # chunked so the fp32 staging stays small
        r1 = min(rows, r0 + chunk)
        kc[r0:r1] = torch.randn(r1 - r0, head_dim, generator=g).to(kv_dtype)
        vc[r0:r1] = torch.randn(r1 - r0, head_dim, generator=g).to(kv_dtype)
    return dict(query=q, key_cache=kc, value_cache=vc, block_table=bt, context_lens=ctx,
                scale=1.0 / math.sqrt(head_dim), batch=batch, num_heads=num_heads,
                kv_heads=kv_heads, head_dim=head_dim, block_size=block_size, q_len=q_len,
                pool_blocks=pool_blocks, max_blocks=max_blocks)


def decoder_layer_inputs(batch=32, hidden=4096, num_heads=32, kv_heads=8, head_dim=128,
                         inter=14336, ctx=4096, block_size=128, theta=500000.0, seed=0,
                         w_std=0.02):
    g = _gen(seed)

    def w(*shape):
        return (torch.randn(*shape, generator=g) * w_std).bfloat16()

    t = dict(
        hidden=torch.randn(batch, hidden, generator=g).bfloat16(),
        input_rms_weight=torch.ones(1, hidden),
        post_rms_weight=torch.ones(1, hidden),
        wq=w(hidden, num_heads * head_dim), wk=w(hidden, kv_heads * head_dim),
        wv=w(hidden, kv_heads * head_dim), wo=w(num_heads * head_dim, hidden),
        w_gate=w(hidden, inter), w_up=w(hidden, inter), w_down=w(inter, hidden),
    )
    pa = paged_attention_inputs(batch=batch, num_heads=num_heads, kv_heads=kv_heads,
                                head_dim=head_dim, block_size=block_size, seed=seed + 1,
                                context_lens=[ctx] * batch)
    max_seq = ((ctx + block_size - 1) // block_size) * block_size
    cos, sin = _layer.rope_tables(max_seq, head_dim, theta)
    t.update(seq_lens=pa["context_lens"], rope_cos=cos, rope_sin=sin, k_cache=pa["key_cache"],
             v_cache=pa["value_cache"], block_table=pa["block_table"])
    geom = dict(num_heads=num_heads, kv_heads=kv_heads, head_dim=head_dim, block_size=block_size,
                eps=1e-5, scale=1.0 / math.sqrt(head_dim))
    return t, geom


def moe_inputs(tokens=4096, hidden=7168, inter=2048, n_experts=256, topk=8, shared=True, seed=0,
               w_std=0.02):
    """Tokens, gate, bias and FP8 block-quantised expert weights (stacked)."""
    g = _gen(seed)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    gate_w = (torch.randn(hidden, n_experts, generator=g) * w_std).bfloat16()
    bias = torch.rand(n_experts, generator=g) * 0.2 - 0.1

    def one_expert():
        wg, sg = _moe.quantize_weight_blocks(torch.randn(hidden, inter, generator=g) * w_std)
        wu, su = _moe.quantize_weight_blocks(torch.randn(hidden, inter, generator=g) * w_std)
        wd, sd = _moe.quantize_weight_blocks(torch.randn(inter, hidden, generator=g) * w_std)
        return dict(wg=wg, sg=sg, wu=wu, su=su, wd=wd, sd=sd)

    exps = [one_expert() for _ in range(n_experts)]
    routed = {k: torch.stack([e[k] for e in exps]) for k in exps[0]}
    sh = one_expert() if shared else None
    return dict(x=x, gate_w=gate_w, bias=bias, routed=routed, shared=sh, topk=topk)
