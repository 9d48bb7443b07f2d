"""GPU parity for the block-table gather: bit-exact against the oracle and the
reference's closed-form fixture (tests/st/runtime/ops/test_paged_gather.py:42-74)."""

import pytest
import torch

from oracle import gather

pytestmark = pytest.mark.gpu


def _ops():
    from pypto_b200 import ops
    return ops


def test_reference_fixture_bit_exact(golden):
    t = golden("paged_gather")
    got = _ops().paged_gather(t["src"].cuda(), t["indices"].cuda(), t["block_table"].cuda(),
                              t["block_size"], t["size"]).cpu()
    assert torch.equal(got.view(torch.int16), t["out"].view(torch.int16))


@pytest.mark.parametrize("dtype,cols,off,size", [(torch.bfloat16, 128, 0, 128), (torch.float32, 96, 32, 48),
                                                 (torch.uint8, 100, 3, 77), (torch.int64, 16, 0, 16)])
def test_random_gathers_bit_exact(dtype, cols, off, size):
    g = torch.Generator().manual_seed(cols)
    bs, nblk = 16, 40
    src = torch.randint(0, 255, (bs * nblk, cols * torch.empty(0, dtype=dtype).element_size()),
                        generator=g, dtype=torch.uint8).view(dtype).reshape(bs * nblk, cols)
    bt = torch.randperm(nblk, generator=g).to(torch.int32)
    idx = torch.randint(0, bs * nblk, (1000,), generator=g, dtype=torch.int32)
    exp = gather.paged_gather(src, idx, bt, bs, size, off)
    got = _ops().paged_gather(src.cuda(), idx.cuda(), bt.cuda(), bs, size, off).cpu()
    assert torch.equal(got.view(torch.uint8), exp.contiguous().view(torch.uint8))


def test_empty_index_list():
    src = torch.zeros(32, 8, device="cuda")
    out = _ops().paged_gather(src, torch.zeros(0, dtype=torch.int32, device="cuda"),
                              torch.zeros(2, dtype=torch.int32, device="cuda"), 16)
    assert out.shape == (0, 8)


def test_index_past_table_is_reported_and_row_zeroed():
    ops = _ops()
    src = torch.ones(32, 8, device="cuda")
    idx = torch.tensor([3, 500], dtype=torch.int32, device="cuda")
    out = ops.paged_gather(src, idx, torch.tensor([1, 0], dtype=torch.int32, device="cuda"), 16)
    torch.cuda.synchronize()
    assert ops.device_status()[0] == 2
    assert out[0].sum() == 8 and out[1].sum() == 0
