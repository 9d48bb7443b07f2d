"""GPU parity on the attention geometries the reference's own system tests pin (single KV head,
q_len 1, fp32 output), generated the way the reference's build_tensors does it (block ids drawn
with replacement).  Shapes: tests/st/runtime/framework_and_models/test_paged_attention.py:843-887,
test_dynamic_paged_attention.py:220-229, test_paged_attention_spmd.py:178-186,
test_paged_attention_multi_config.py:689-718, test_batch_paged_attention.py:1090-1094.  The
256-sequence cases run with 16 sequences so that the CPU oracle stays in seconds; every other
dimension is the reference's."""

import pytest
import torch

from oracle import paged_attention as opa

pytestmark = pytest.mark.gpu

# (batch, heads, head_dim, block_size, context (int or per-sequence list), max_model_len, scale)
CASES = [
    (64, 16, 128, 128, 8192, 32768, 1.0),
    (64, 16, 128, 128, 8100, 32768, 1.0),
    (16, 16, 128, 128, 8192, 32768, 1.0),
    (16, 64, 128, 64, 8192, 32768, 1.0),
    (8, 64, 256, 64, 2048, 32768, 1.0),
    (4, 16, 128, 128, [512, 4096, 8192, 768], 32768, 1.0),
    (2, 64, 256, 128, 64, 4096, 0.0625),
    (2, 64, 256, 128, 50, 4096, 0.0625),
    (2, 64, 256, 128, 100 + 64, 4096, 0.0625),
    (2, 64, 256, 64, 1000, 4096, 0.0625),
    (2, 64, 128, 128, 700, 4096, 0.0884),
    (2, 64, 128, 64, 500, 4096, 0.0884),
    (2, 16, 16, 16, 64, 256, 1.0),
]


@pytest.mark.parametrize("batch,heads,hd,bs,ctx,max_len,scale", CASES)
def test_reference_pinned_geometry(batch, heads, hd, bs, ctx, max_len, scale):
    from pypto_b200 import ops
    g = torch.Generator().manual_seed(batch * 1000 + heads + hd + bs)
    max_blocks = max_len // bs
    ctx_t = torch.tensor(ctx if isinstance(ctx, list) else [ctx] * batch, dtype=torch.int32)
    need = int(((ctx_t.long() + bs - 1) // bs).max())
    pool_blocks = max(batch * need, 1)              # a pool as large as the blocks actually addressed
    bt = torch.randint(0, pool_blocks, (batch, max_blocks), generator=g, dtype=torch.int32)
    q = torch.randn(batch * heads, hd, generator=g).bfloat16()
    kc = torch.randn(pool_blocks * bs, hd, generator=g).bfloat16()
    vc = torch.randn(pool_blocks * bs, hd, generator=g).bfloat16()
    exp = opa.paged_attention(q, kc, vc, bt, ctx_t, num_heads=heads, head_dim=hd, block_size=bs, scale=scale)
    got = ops.paged_attention(q.cuda(), kc.cuda(), vc.cuda(), bt.cuda(), ctx_t.cuda(), num_heads=heads, kv_heads=1,
                              head_dim=hd, block_size=bs, scale=scale, out_dtype=torch.float32)
    torch.cuda.synchronize()
    ops.check_device_status()
    got = got.cpu()
    assert torch.isfinite(got).all()
    bad = (got - exp).abs() > 4e-3 + 2e-2 * exp.abs()      # rtol 2e-2 of test_paged_attention.py:490-491
    assert not bad.any(), f"{int(bad.sum())} of {bad.numel()} off, max abs diff {(got - exp).abs().max():.4g}"
