"""GPU parity of the MX block-scaled FP8 matmul: the reference's own known-answer case (integer-valued e4m3
data, E8M0 codes 126..129, rtol = atol = 0, tests/st/runtime/ops/test_matmul_mx.py:154-165, 283) through the
C ABI in both scale layouts, the accumulate form, and ragged / large shapes against the oracle."""

import pytest
import torch

from oracle import matmul_mx as omx

pytestmark = pytest.mark.gpu

FP8 = torch.float8_e4m3fn


def _ops():
    from pypto_b200 import ops
    return ops


def test_reference_known_answer_case_is_exact_in_both_scale_layouts(golden):
    ops = _ops()
    t = golden("matmul_mx")
    a = t["a"].cuda().view(FP8)
    b_t = ops.transpose_u8(t["b"].cuda()).view(FP8)                     # [K, N] as the reference passes it -> [N, K]
    assert torch.equal(b_t.cpu().view(torch.uint8), t["b"].t().contiguous())
    out = ops.matmul_mx(a, t["a_scale_codes"].cuda(), b_t, t["b_scale_codes"].cuda())
    out_phys = ops.matmul_mx(a, t["a_scale_packed"].cuda(), b_t, t["b_scale_packed"].cuda(),
                             a_scale_layout=ops.MX_SCALE_A_ZZ, b_scale_layout=ops.MX_SCALE_B_NN)
    acc = ops.matmul_mx(a, t["a_scale_codes"].cuda(), b_t, t["b_scale_codes"].cuda(), acc=out)    # matmul_mx_acc
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.equal(out.cpu(), t["out"])            # rtol = atol = 0, as the reference's RunConfig demands
    assert torch.equal(out_phys.cpu(), t["out"])
    assert torch.equal(acc.cpu(), t["out_acc"])
    inplace = out.clone()
    ops.matmul_mx(a, t["a_scale_codes"].cuda(), b_t, t["b_scale_codes"].cuda(), acc=inplace, out=inplace)
    assert torch.equal(inplace.cpu(), t["out_acc"])


@pytest.mark.parametrize("m,n,k", [(64, 128, 128), (200, 384, 352), (129, 130, 32), (1, 128, 1024), (4096, 4096, 512),
                                   (2100, 4232, 1056)])
def test_integer_operands_are_exact_at_ragged_and_large_shapes(m, n, k):
    """Same recipe as the reference's case at other shapes: row/column/K tails (TMA zero fill, neutral scale
    codes outside the matrix), many tiles per CTA, and the 256 x 224 tiles that large problems with K >= 1024
    run on SM pairs (the last shape has tails in all three dimensions there)."""
    ops = _ops()
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randint(-2, 3, (m, k), generator=g).to(FP8)
    b = torch.randint(-2, 3, (k, n), generator=g).to(FP8)
    sa = torch.randint(126, 130, (m, k // 32), generator=g).to(torch.uint8)
    sb = torch.randint(126, 130, (k // 32, n), generator=g).to(torch.uint8)
    exp = omx.matmul_mx(a, sa, b, sb)
    b_t = ops.transpose_u8(b.cuda().view(torch.uint8)).view(FP8)
    out = ops.matmul_mx(a.cuda(), sa.cuda(), b_t, sb.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.equal(out.cpu(), exp)


@pytest.mark.parametrize("m,n,k", [(256, 512, 512), (144, 272, 256), (4096, 2048, 1024), (2064, 4240, 1024)])
def test_physical_scale_layouts_are_exact_at_larger_shapes(m, n, k):
    """The reference's packed scale layouts (MX_A_ZZ, MX_B_NN; test_matmul_mx.py:38-117) on tiles that lie inside the
    matrix (wide scale loads) and on tiles with row and column tails (byte loads), against the same golden."""
    ops = _ops()
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randint(-2, 3, (m, k), generator=g).to(FP8)
    b = torch.randint(-2, 3, (k, n), generator=g).to(FP8)
    sa = torch.randint(125, 131, (m, k // 32), generator=g).to(torch.uint8)
    sb = torch.randint(125, 131, (k // 32, n), generator=g).to(torch.uint8)
    exp = omx.matmul_mx(a, sa, b, sb)
    b_t = ops.transpose_u8(b.cuda().view(torch.uint8)).view(FP8)
    out = ops.matmul_mx(a.cuda(), omx.pack_a_scale(sa).cuda(), b_t, omx.pack_b_scale(sb).cuda(),
                        a_scale_layout=ops.MX_SCALE_A_ZZ, b_scale_layout=ops.MX_SCALE_B_NN)
    mixed = ops.matmul_mx(a.cuda(), sa.cuda(), b_t, omx.pack_b_scale(sb).cuda(), b_scale_layout=ops.MX_SCALE_B_NN)
    twice = ops.matmul_mx(a.cuda(), sa.cuda(), b_t, sb.cuda(), acc=out)        # matmul_mx_acc on the same tiles
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.equal(out.cpu(), exp)
    assert torch.equal(mixed.cpu(), exp)
    assert torch.equal(twice.cpu(), exp + exp)


def test_quantised_gaussian_operands_match_the_fp64_golden():
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    m, n, k = 384, 512, 2048
    a, sa = omx.quantize_mx(torch.randn(m, k, generator=g), dim=1)
    b, sb = omx.quantize_mx(torch.randn(k, n, generator=g) * 0.02, dim=0)
    exp = omx.matmul_mx(a, sa, b, sb)
    out = ops.matmul_mx(a.cuda(), sa.cuda(), ops.transpose_u8(b.cuda().view(torch.uint8)).view(FP8), sb.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()
    rel = ((out.cpu() - exp).norm() / exp.norm()).item()
    assert rel < 1e-5, rel        # fp32 accumulation of exact products against the fp64 golden


def test_argument_checks():
    from pypto_b200 import _lib
    ops = _ops()
    a = torch.zeros(16, 48, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError):
        ops.matmul_mx(a, a[:, :1], a, a[:1])                # K not a multiple of 32
    a = torch.zeros(24, 64, dtype=torch.uint8, device="cuda")
    s = torch.zeros(24, 2, dtype=torch.uint8, device="cuda")
    with pytest.raises(_lib.PtoError):
        ops.matmul_mx(a, s, a, s.t().contiguous(), a_scale_layout=ops.MX_SCALE_A_ZZ)    # m % 16 != 0
