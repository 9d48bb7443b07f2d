"""Oracle for the MX block-scaled FP8 matmul (test infrastructure, not product code).

Restates the golden of the reference's MX matmul test
(tests/st/runtime/ops/test_matmul_mx.py:119-131): operands are e4m3 values with one E8M0
scale code per group of 32 elements along K (value * 2**(code - 127)); the product is
taken in float64 and returned as float32.  ``matmul_mx_acc`` adds the product to a base
tile (src/ir/op/tile_ops/matmul_mx.cpp:321-345; the test expects ``2 * base`` when the
base is the product itself, test_matmul_mx.py:314-315).

The reference hands the kernel its scale tensors in two physical layouts, MX_A_ZZ for the
left operand and MX_B_NN for the right one (test_matmul_mx.py:38-101); ``pack_*`` /
``unpack_*`` restate those permutations.  Pinned bit-for-bit against
tests/golden/matmul_mx.pt, which the extracted reference functions produced.
"""

from __future__ import annotations

import torch

GROUP = 32          # elements of K that share one scale (MX_GROUP_SIZE)
SCALE_BLOCK = 16    # rows (A) / columns (B) per physical scale block
SCALE_C0 = 2        # K groups per physical scale block


def decode_scale(codes: torch.Tensor) -> torch.Tensor:
    """E8M0 code -> float64 scale 2**(code - 127)."""
    return torch.pow(2.0, codes.to(torch.float64) - 127)


def matmul_mx(a, a_scale_codes, b, b_scale_codes, acc=None):
    """a [M, K], b [K, N] (any dtype holding e4m3-representable values); a_scale_codes uint8
    [M, K/32]; b_scale_codes uint8 [K/32, N].  Returns fp32 [M, N] (+ acc)."""
    k = a.shape[1]
    kg = torch.arange(k) // GROUP
    a_s = a.to(torch.float64) * decode_scale(a_scale_codes)[:, kg]
    b_s = b.to(torch.float64) * decode_scale(b_scale_codes)[kg, :]
    out = torch.matmul(a_s, b_s).to(torch.float32)
    return out if acc is None else out + acc


def pack_a_scale(codes: torch.Tensor) -> torch.Tensor:
    """Logical [M, K/32] -> MX_A_ZZ physical order (same shape)."""
    m, g = codes.shape
    return codes.reshape(m // SCALE_BLOCK, SCALE_BLOCK, g // SCALE_C0, SCALE_C0).permute(0, 2, 1, 3) \
        .contiguous().reshape(m, g)


def unpack_a_scale(packed: torch.Tensor) -> torch.Tensor:
    m, g = packed.shape
    return packed.reshape(m // SCALE_BLOCK, g // SCALE_C0, SCALE_BLOCK, SCALE_C0).permute(0, 2, 1, 3) \
        .contiguous().reshape(m, g)


def pack_b_scale(codes: torch.Tensor) -> torch.Tensor:
    """Logical [K/32, N] -> MX_B_NN physical order (same shape)."""
    g, n = codes.shape
    return codes.reshape(g // SCALE_C0, SCALE_C0, n // SCALE_BLOCK, SCALE_BLOCK).permute(2, 0, 3, 1) \
        .contiguous().reshape(g, n)


def unpack_b_scale(packed: torch.Tensor) -> torch.Tensor:
    g, n = packed.shape
    return packed.reshape(n // SCALE_BLOCK, g // SCALE_C0, SCALE_BLOCK, SCALE_C0).permute(1, 3, 0, 2) \
        .contiguous().reshape(g, n)


def quantize_mx(x: torch.Tensor, dim: int):
    """Quantise a float matrix to e4m3 with one power-of-two scale per 32 elements along ``dim``
    (the OCP MX rule: shared exponent = floor(log2(amax)) - 8, 8 = emax of e4m3).  Returns
    (values e4m3, codes uint8 with the group axis in place of ``dim``).  Used to make
    realistic inputs at benchmark sizes; the reference test draws integers instead."""
    xm = x.float().movedim(dim, -1)
    shp = xm.shape
    g = xm.reshape(*shp[:-1], shp[-1] // GROUP, GROUP)
    amax = g.abs().amax(dim=-1)
    e = torch.where(amax > 0, torch.floor(torch.log2(amax)) - 8, torch.zeros_like(amax)).clamp(-127, 127)
    q = (g / torch.pow(2.0, e).unsqueeze(-1)).clamp(-448, 448).reshape(shp).to(torch.float8_e4m3fn)
    codes = (e + 127).to(torch.uint8)
    return q.movedim(-1, dim).contiguous(), codes.movedim(-1, dim).contiguous()
