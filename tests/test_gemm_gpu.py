"""GPU parity for the tcgen05 GEMM paths: linear (decode and prefill orientation, split-K,
accumulate), the fused SwiGLU FFN, against fp32 torch on the same bf16-rounded operands and
against the oracle's FFN.  bf16 bar of the workload definition: relative 2e-2; the GEMMs
themselves accumulate in fp32, so they are held to 2e-3 of the output scale."""

import pytest
import torch

import oracle
from oracle import ffn as offn

pytestmark = pytest.mark.gpu


def _ops():
    from pypto_b200 import ops
    return ops


def _check(got, exp, rel, what):
    got, exp = got.float().cpu(), exp.float().cpu()
    assert torch.isfinite(got).all(), what
    scale = exp.abs().max().item() + 1e-12
    err = (got - exp).abs().max().item()
    assert err <= rel * scale, f"{what}: max abs err {err:.4g} vs scale {scale:.4g}"


@pytest.mark.parametrize("m,n,k", [(1, 128, 64), (7, 300, 200), (32, 4096, 1024), (100, 512, 4096),
                                   (256, 1000, 520), (300, 384, 256), (1024, 1024, 512), (640, 200, 1096)])
def test_linear_matches_fp32_matmul(m, n, k):
    ops = _ops()
    g = torch.Generator().manual_seed(m * 7 + n)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(k, n, generator=g) * 0.05).bfloat16()
    exp = x.float() @ w.float()
    wp = ops.pack_weight(w.cuda())
    assert torch.equal(wp.cpu(), w.t().contiguous())
    got = ops.linear(x.cuda(), wp)
    torch.cuda.synchronize()
    ops.check_device_status()
    _check(got, exp, 2e-3, f"linear {m}x{n}x{k}")
    # accumulate on top of an existing fp32 tensor (the residual form)
    base = torch.randn(m, n, generator=g)
    acc = base.cuda().clone()
    ops.linear(x.cuda(), wp, out=acc, accumulate=True)
    _check(acc, exp + base, 2e-3, f"linear accumulate {m}x{n}x{k}")


def test_large_m_256_row_tiles():
    """Sizes that take the 256-row CTA tile (two A tiles share the B tile, all 512 TMEM columns
    in use), with a ragged last tile."""
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    m, n, k = 8000, 4096, 2048
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(k, n, generator=g) * 0.05).bfloat16()
    got = ops.linear(x.cuda(), ops.pack_weight(w.cuda()))
    torch.cuda.synchronize()
    ops.check_device_status()
    _check(got, x.float() @ w.float(), 2e-3, "linear 8000x4096x2048")
    from pypto_b200.layers import SwiGLUFFN
    xf, wg, wu, wd = oracle.inputs.ffn_inputs(5000, 2048, 2048, seed=6)
    xb, wgb, wub, wdb = xf.bfloat16(), wg.bfloat16(), wu.bfloat16(), wd.bfloat16()
    got = SwiGLUFFN(wgb.cuda(), wub.cuda(), wdb.cuda())(xb.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()
    _check(got, offn.ffn_swiglu_bf16(xb, wgb, wub, wdb), 5e-3, "ffn 5000x2048x2048")


@pytest.mark.parametrize("m,n,k", [(1300, 3400, 264), (2048, 19200, 64), (4096, 4736, 1024)])
def test_linear_on_cta_pairs_with_ragged_edges(m, n, k):
    """Shapes that run on CTA pairs (256 x 256 tiles, tcgen05.mma.cta_group::2): row, column and K tails, a single
    K block per tile (every hand-off of the pair once per tile), and many tiles per pair."""
    ops = _ops()
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(k, n, generator=g) * 0.05).bfloat16()
    got = ops.linear(x.cuda(), ops.pack_weight(w.cuda()))
    torch.cuda.synchronize()
    ops.check_device_status()
    _check(got, x.float() @ w.float(), 2e-3, f"linear on pairs {m}x{n}x{k}")


def test_pack_weight_from_fp32_rounds_to_bf16():
    w = torch.randn(96, 40)
    wp = _ops().pack_weight(w.cuda())
    assert torch.equal(wp.cpu(), w.bfloat16().t().contiguous())


@pytest.mark.parametrize("m,k,inter", [(32, 512, 1024), (4, 256, 384), (128, 1024, 4096), (512, 512, 1024),
                                       (1000, 256, 2048)])
def test_ffn_swiglu_matches_oracle(m, k, inter):
    from pypto_b200.layers import SwiGLUFFN
    x, wg, wu, wd = oracle.inputs.ffn_inputs(m, k, inter, seed=m)
    xb, wgb, wub, wdb = x.bfloat16(), wg.bfloat16(), wu.bfloat16(), wd.bfloat16()
    exp = offn.ffn_swiglu_bf16(xb, wgb, wub, wdb)
    f = SwiGLUFFN(wgb.cuda(), wub.cuda(), wdb.cuda())
    got = f(xb.cuda())
    torch.cuda.synchronize()
    _ops().check_device_status()
    _check(got, exp, 5e-3, f"ffn {m}x{k}x{inter}")


def test_ffn_reference_example_config_fp32_inputs():
    """The FFN workload: x[128,1024] N(0,1), W ~ N(0, 0.02^2), fp32 as specified, seed 0; result
    held to relative 2e-2 against the fp32 expression of examples/models/01_ffn.py:174-176."""
    from pypto_b200.layers import SwiGLUFFN
    x, wg, wu, wd = oracle.inputs.ffn_inputs(128, 1024, 4096, seed=0)
    exp = offn.ffn_swiglu(x, wg, wu, wd)
    got = SwiGLUFFN(wg.cuda(), wu.cuda(), wd.cuda())(x.cuda())
    torch.cuda.synchronize()
    _ops().check_device_status()
    _check(got, exp, 2e-2, "ffn fp32-specified workload")
    rel = ((got.cpu() - exp).norm() / exp.norm()).item()
    assert rel < 1e-2, rel


@pytest.mark.parametrize("m", [128, 57, 300])
def test_ffn_takes_fp32_x_and_casts_it_itself(m):
    """pto_ffn_swiglu_f32: x in fp32 as `ffn_swiglu` receives it (01_ffn.py:155-160).  At most 128 rows: ONE launch whose
    CTAs cast x (each its share) and clear the output before the first GEMM; more rows: a cast kernel ahead of the
    GEMM chain.  Same numbers as casting first, bit for bit; the accumulate form adds onto a residual."""
    ops = _ops()
    from pypto_b200.layers import SwiGLUFFN
    x, wg, wu, wd = oracle.inputs.ffn_inputs(m, 1024, 4096, seed=m)
    f = SwiGLUFFN(wg.cuda(), wu.cuda(), wd.cuda())
    xd = x.cuda()
    out = torch.full((m, 1024), 7.0, device="cuda")                  # stale contents must be cleared
    got = ops.ffn_swiglu(xd, f.w_gate_up, f.w_down, out=out)
    again = ops.ffn_swiglu(xd, f.w_gate_up, f.w_down, out=out)       # counters of the call before are back at zero
    torch.cuda.synchronize()
    ops.check_device_status()
    exp = offn.ffn_swiglu(x, wg, wu, wd)
    _check(got, exp, 2e-2, f"ffn fp32 x, m = {m}")
    ref = ops.ffn_swiglu(ops.cast(xd, torch.bfloat16), f.w_gate_up, f.w_down)
    if m <= 128:                                                      # stream-K partial sums meet in any order
        assert (got - ref).abs().max() <= 1e-3 * exp.abs().max() and (again - ref).abs().max() <= 1e-3 * exp.abs().max()
    resid = torch.randn(m, 1024, device="cuda")
    acc = ops.ffn_swiglu(xd, f.w_gate_up, f.w_down, out=resid.clone(), accumulate=True)
    torch.cuda.synchronize()
    _check(acc - resid, exp, 2e-2, f"ffn fp32 x accumulate, m = {m}")


def test_ffn_64x64_reference_shape():
    """64x64 fp32, N(0,1) weights, the shapes of 01_ffn.py:157-160 (rtol/atol 3e-3 there is for
    fp32 operands; bf16 operands are held to 2e-2 of the output scale)."""
    from pypto_b200.layers import SwiGLUFFN
    x, wg, wu, wd = oracle.inputs.ffn_inputs(64, 64, 64, seed=0, w_std=1.0)
    exp = offn.ffn_swiglu(x, wg, wu, wd)
    got = SwiGLUFFN(wg.cuda(), wu.cuda(), wd.cuda())(x.cuda())
    _check(got, exp, 2e-2, "ffn 64x64")


@pytest.mark.parametrize("m,k,inter,n_out", [(1, 256, 128, 256), (33, 1024, 4096, 1024), (128, 1024, 4096, 1024),
                                             (32, 512, 14336, 520), (100, 200, 192, 68)])
def test_one_launch_ffn_repeated_calls_and_residual(m, k, inter, n_out):
    """At most 128 rows: both GEMMs in one cooperative launch whose CTAs hand the activation over through
    counters kept in the workspace.  Several calls in a row on one workspace (the counters only grow and the
    call number advances on the device), different inputs each time, with and without a residual in the output;
    ragged K, output width and token count."""
    ops = _ops()
    g = torch.Generator().manual_seed(m + inter)
    wg = (torch.randn(k, inter, generator=g) * 0.05).bfloat16()
    wu = (torch.randn(k, inter, generator=g) * 0.05).bfloat16()
    wd = (torch.randn(inter, n_out, generator=g) * 0.05).bfloat16()
    w_gu = ops.pack_weight(torch.cat([wg, wu], dim=1).contiguous().cuda())
    w_d = ops.pack_weight(wd.cuda())
    for rep in range(4):
        x = torch.randn(m, k, generator=g).bfloat16()
        act = (x.float() @ wg.float())
        act = (act * torch.sigmoid(act) * (x.float() @ wu.float())).bfloat16()
        exp = act.float() @ wd.float()
        if rep % 2:
            base = torch.randn(m, n_out, generator=g)
            out = base.cuda().clone()
            ops.ffn_swiglu(x.cuda(), w_gu, w_d, out=out, accumulate=True)
            exp = exp + base
        else:
            out = ops.ffn_swiglu(x.cuda(), w_gu, w_d)
        torch.cuda.synchronize()
        ops.check_device_status()
        _check(out, exp, 5e-3, f"one-launch ffn {m}x{k}x{inter}x{n_out} call {rep}")
