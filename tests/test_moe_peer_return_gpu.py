"""GPU (one device): the peer-memory return path of the expert-parallel layer, its ranks emulated on ONE GPU -- every
"rank" is a set of buffers of this process and the push kernels run one after another on one stream, so nothing ever
waits for a kernel that has not run yet.  (On real ranks the same kernels store into buffers mapped from the other
processes' CUDA IPC handles; tests/test_moe_ep_gpu.py covers that on 2, 4 and 8 GPUs.)"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from pypto_b200 import ops
    return ops


def _case(world, local_experts, cols, seed):
    """Counts counts[d][s][e] = rows rank s sends to local expert e of rank d, and what every rank must end up with."""
    g = torch.Generator().manual_seed(seed)
    counts = torch.randint(0, 7, (world, world, local_experts), generator=g, dtype=torch.int32)
    counts[1 % world, 0] = 0                                   # a pair that exchanges nothing
    # rank s keeps its routes sorted by (destination rank, expert): the block for rank d starts at base[s][d]
    per_dst = counts.sum(dim=2).t().contiguous()               # [s][d]
    base = torch.zeros(world, world, dtype=torch.int64)
    base[:, 1:] = per_dst.cumsum(dim=1)[:, :-1]
    total_sorted = per_dst.sum(dim=1)                          # rows of rank s
    # result rows as rank d holds them: arrival order = source after source; value encodes (d, s, j)
    cap = int(total_sorted.max()) + 3                          # every rank's result buffer holds the same number of rows
    arrival, expected = [], [torch.zeros(cap, cols, dtype=torch.bfloat16) for s in range(world)]
    for d in range(world):
        blocks = []
        for s in range(world):
            n = int(per_dst[s, d])
            blk = (torch.arange(n, dtype=torch.float32)[:, None] + 100 * s + 1000 * d + torch.arange(cols)[None, :] * 0.25)
            blk = blk.bfloat16()
            blocks.append(blk)
            expected[s][int(base[s, d]): int(base[s, d]) + n] = blk
        arrival.append(torch.cat(blocks) if blocks else torch.zeros(0, cols, dtype=torch.bfloat16))
    return counts, base, arrival, expected


@pytest.mark.parametrize("world,local_experts,cols", [(2, 3, 64), (4, 2, 7168), (8, 4, 256)])
def test_blocks_land_at_their_sources_offsets_and_flags_follow(world, local_experts, cols):
    ops = _ops()
    counts, base, arrival, expected = _case(world, local_experts, cols, seed=world)
    back = [torch.zeros_like(e).cuda() for e in expected]                      # rows past a rank's own stay zero
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(world)]
    done = torch.zeros(64, dtype=torch.int32, device="cuda")
    for step in (1, 2):                                                        # flags only ever count up
        for b in back:
            b.zero_()
        for d in range(world):
            dst_base = base[:, d].to(torch.int32).cuda()                       # what every source asked rank d for
            rows = arrival[d].cuda() if arrival[d].shape[0] else torch.zeros(1, cols, dtype=torch.bfloat16, device="cuda")
            ops.moe_push_rows(rows, counts[d].cuda(), dst_base, back, flags, d, step, done)
        for r in range(world):
            ops.moe_wait_flags(flags[r], world, step)
        torch.cuda.synchronize()
        ops.check_device_status()
        for s in range(world):
            assert torch.equal(back[s].cpu(), expected[s]), (step, s)
            assert flags[s][:world].tolist() == [step] * world
        assert int(done[0]) == 0


def test_a_block_that_does_not_fit_is_refused_not_written():
    ops = _ops()
    counts = torch.tensor([[4]], dtype=torch.int32).cuda()                     # one rank, one expert, four rows
    rows = torch.ones(4, 64, dtype=torch.bfloat16, device="cuda")
    back = [torch.zeros(5, 64, dtype=torch.bfloat16, device="cuda")]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda")]
    done = torch.zeros(64, dtype=torch.int32, device="cuda")
    ops.moe_push_rows(rows, counts, torch.tensor([3], dtype=torch.int32).cuda(), back, flags, 0, 1, done)   # rows 3..6 of 5
    torch.cuda.synchronize()
    code, site, _, _ = ops.device_status()
    assert (code, site) == (3, 65)
    assert back[0][:3].abs().sum() == 0 and back[0][3:5].float().sum() == 2 * 64     # the rows that fit were written


def test_a_rank_that_never_shows_ends_in_the_error_word():
    """A flag that nothing raises: the wait gives up after its two seconds, the error word names the rank, the
    context stays usable."""
    ops = _ops()
    flags = torch.zeros(64, dtype=torch.int32, device="cuda")
    flags[0] = 5
    ops.moe_wait_flags(flags, 2, 5)                                             # rank 1 never raised its flag
    torch.cuda.synchronize()
    code, site, _, detail = ops.device_status()
    assert (code, site, detail) == (1, 66, 1)
    flags[1] = 5
    ops.moe_wait_flags(flags, 2, 5)
    torch.cuda.synchronize()
    ops.check_device_status()
