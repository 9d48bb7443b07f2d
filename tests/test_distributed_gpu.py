"""The reference's expert-parallel program through ``compiled(...)`` of the level-3 launch surface: the
committed fixtures of its own goldens (_compute_golden_recv / _compute_golden_routed,
tests/st/distributed/test_l3_ep_dispatch_combine.py:562-629) on 2 and 4 GPUs, compared the way the reference
compares (:690-725: counts, rows and route ids bit for bit; routed_y within two bf16 ulps), plus a one-rank run
(all experts local) and resident rank-sharded inputs on a prepared worker."""

import pytest
import torch

import ep_program
from oracle import ep as oep

pytestmark = pytest.mark.gpu


def _check(args, exp):
    _ind, _x, _w, _i, recv_x, recv_w, recv_idx, recv_count, recv_y, routed = args
    n, L, R = recv_w.shape
    assert torch.equal(recv_count.squeeze(-1), exp["count"])
    rx, ry = recv_x.reshape(n, L, R, -1), recv_y.reshape(n, L, R, -1)
    for r in range(n):
        for e in range(L):
            c = int(exp["count"][r, e])
            assert torch.equal(rx[r, e, :c].view(torch.int16), exp["recv_x"][r, e, :c].view(torch.int16))
            assert torch.equal(recv_w[r, e, :c], exp["recv_w"][r, e, :c])
            assert torch.equal(recv_idx[r, e, :c], exp["recv_idx"][r, e, :c])
            assert torch.equal(ry[r, e, :c].view(torch.int16),
                               oep.standin_expert(exp["recv_x"][r, e, :c], exp["recv_w"][r, e, :c]).view(torch.int16))
            assert torch.count_nonzero(rx[r, e, c:].float()) == 0          # unused slots stay zero
    assert torch.allclose(routed, exp["routed"], atol=2.0 ** -6, rtol=2.0 ** -6)


def _compiled(n, t):
    from pypto_b200 import ir
    from pypto_b200.ir import DistributedConfig
    prog = ep_program.build(n, t["t"], t["topk"], t["d"], t["l"], t["r"])
    return ir.compile(prog, platform="b200", distributed_config=DistributedConfig(device_ids=list(range(n))))


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_reference_ep_fixture_through_the_distributed_call(golden, n_ranks):
    if torch.cuda.device_count() < n_ranks:
        pytest.skip(f"needs {n_ranks} GPUs")
    t = golden(f"ep_{n_ranks}")
    args = ep_program.host_tensors(t["x"], t["weights"], t["indices"], t["l"], t["r"])
    _compiled(n_ranks, t)(*args)
    _check(args, t)


def test_single_rank_program_and_resident_inputs(golden):
    """World size 1 (every expert local): same child-process machinery, same padded receive layout, on one GPU.
    The golden comes from the oracle's restatement of the reference's dispatch (pinned against the 2- and
    4-rank fixtures on CPU).  Second dispatch with the inputs resident on the worker."""
    t = golden("ep_2")
    L2, R = 2 * t["l"], 2 * t["r"]                        # rank 0's tokens over all 8 experts, local now
    x, w, ind = t["x"][:1], t["weights"][:1], t["indices"][:1]
    rx, rw, ri, _rs, cnt = oep.dispatch(x, ind, w, L2, R)
    exp = dict(count=cnt, recv_x=rx, recv_w=rw, recv_idx=ri, routed=t["routed"][:1])
    args = ep_program.host_tensors(x, w, ind, L2, R)
    c = _compiled(1, dict(t, l=L2, r=R))
    with c.prepare() as worker:
        worker(*args)
        _check(args, exp)
        stacked = [worker.alloc_stacked_tensor(a) for a in args[:4]]
        outs = [torch.zeros_like(a) for a in args[4:]]
        worker.run(c, *stacked, *outs)
        _check(args[:4] + outs, exp)
        back = torch.empty_like(args[1])
        worker.copy_stacked_from(stacked[1], back)
        assert torch.equal(back.view(torch.int16), args[1].view(torch.int16))
        worker.free_stacked_tensor(stacked[0])
        with pytest.raises(ValueError):
            worker.run(c, *stacked, *outs)
