"""GPU parity for the decoder-layer glue (RMSNorm, RoPE + paged KV append) and the whole
decode layer against the oracle (rounding points of qwen3_decode.py:50-112)."""

import pytest
import torch

import oracle
from oracle import layer as olayer

pytestmark = pytest.mark.gpu


def _ops():
    from pypto_b200 import ops
    return ops


@pytest.mark.parametrize("rows,hidden,in_dtype", [(32, 64, torch.float32), (16, 4096, torch.bfloat16),
                                                  (5, 1000, torch.float32)])
def test_rms_norm(rows, hidden, in_dtype):
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(rows, hidden, generator=g).to(in_dtype)
    gamma = torch.randn(1, hidden, generator=g)
    got32 = _ops().rms_norm(x.cuda(), gamma.reshape(-1).cuda(), 1e-5, torch.float32).cpu()
    assert torch.allclose(got32, olayer.rms_norm(x, gamma, 1e-5), rtol=1e-5, atol=1e-5)   # test_rms_norm.py:39
    got16 = _ops().rms_norm(x.cuda(), gamma.reshape(-1).cuda(), 1e-5, torch.bfloat16).cpu()
    exp16 = olayer.rms_norm(x, gamma, 1e-5, torch.bfloat16)
    assert (got16.float() - exp16.float()).abs().max() <= 2 ** -7 * exp16.float().abs().max()


def test_rope_kv_append_rows_and_values():
    heads, kvh, d, bs = 8, 2, 128, 16
    pa = oracle.inputs.paged_attention_inputs(num_heads=heads, kv_heads=kvh, block_size=bs,
                                              context_lens=[1, 16, 17, 300], seed=6)
    batch = 4
    g = torch.Generator().manual_seed(1)
    qkv = torch.randn(batch, (heads + 2 * kvh) * d, generator=g)
    cos, sin = olayer.rope_tables(320, d, 500000.0)
    kc, vc = pa["key_cache"].clone(), pa["value_cache"].clone()
    q_exp = olayer.rope_kv_append(qkv[:, :heads * d], qkv[:, heads * d:(heads + kvh) * d], qkv[:, (heads + kvh) * d:],
                                  pa["context_lens"], cos, sin, kc, vc, pa["block_table"], num_heads=heads,
                                  kv_heads=kvh, head_dim=d, block_size=bs)
    kd, vd = pa["key_cache"].cuda(), pa["value_cache"].cuda()
    q_got = _ops().rope_kv_append(qkv.cuda(), pa["context_lens"].cuda(), cos.cuda(), sin.cuda(),
                                  pa["block_table"].cuda(), kd, vd, num_heads=heads, kv_heads=kvh, head_dim=d,
                                  block_size=bs)
    torch.cuda.synchronize()
    _ops().check_device_status()
    changed = (kd.cpu() != pa["key_cache"]).any(dim=1)
    assert torch.equal(changed, (kc != pa["key_cache"]).any(dim=1))      # exactly the appended rows
    assert torch.equal(vd.cpu().view(torch.int16), vc.view(torch.int16))      # V rows are a pure bf16 round
    for got, exp in ((kd.cpu(), kc), (q_got.cpu(), q_exp)):
        assert (got.float() - exp.float()).abs().max() <= 2 ** -7 * exp.float().abs().max()


def _layer_case(**kw):
    from pypto_b200.layers import DecoderLayer
    t, geom = oracle.inputs.decoder_layer_inputs(**kw)
    ref = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in t.items()}
    exp = olayer.decoder_layer(ref, **geom)
    dev = {k: v.cuda() for k, v in t.items()}
    layer = DecoderLayer(dev, **geom)
    got = layer.step(dev["hidden"], dev["seq_lens"], dev["block_table"], dev["k_cache"], dev["v_cache"])
    torch.cuda.synchronize()
    _ops().check_device_status()
    return got.cpu(), exp, dev, ref


def test_decoder_layer_small():
    got, exp, dev, ref = _layer_case(batch=4, hidden=512, num_heads=8, kv_heads=2, head_dim=128, inter=1024,
                                     ctx=300, seed=3)
    err = (got.float() - exp.float()).abs().max().item()
    assert err <= 2e-2 * exp.float().abs().max().item(), err
    assert (dev["k_cache"].cpu().float() - ref["k_cache"].float()).abs().max() <= 0.05


def test_decoder_layer_full_size():
    """hidden 4096, 32/8 heads, head_dim 128, FFN 14336, batch 32, 4096-token paged caches."""
    got, exp, _dev, _ref = _layer_case()
    rel = ((got.float() - exp.float()).norm() / exp.float().norm()).item()
    err = (got.float() - exp.float()).abs().max().item()
    assert rel < 1e-2 and err <= 2e-2 * exp.float().abs().max().item(), (rel, err)


def test_rms_norm_side_jobs_copy_and_clear():
    """The fused form gives the same rows as the plain one, leaves x as fp32 in `copy_fp32` and clears `zero`."""
    ops = _ops()
    torch.manual_seed(1)
    x = torch.randn(32, 4096).bfloat16().cuda()
    gamma = (torch.rand(4096) + 0.5).cuda()
    plain = ops.rms_norm(x, gamma, 1e-5, torch.bfloat16)
    copy = torch.full((32, 4096), float("nan"), device="cuda")
    acc = torch.full((32, 6144), 3.0, device="cuda")
    fused = ops.rms_norm(x, gamma, 1e-5, torch.bfloat16, copy_fp32=copy, zero=acc)
    assert torch.equal(fused, plain)
    assert torch.equal(copy, x.float())
    assert not acc.any()
    with pytest.raises(ValueError):
        ops.rms_norm(x, gamma, 1e-5, torch.bfloat16, copy_fp32=torch.empty(32, 4096, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        ops.rms_norm(x, gamma, 1e-5, torch.bfloat16, zero=torch.empty(3, device="cuda"))
