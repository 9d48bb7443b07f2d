"""world_size-2 and -4 gloo runs (CPU) of the expert-parallel host logic: count exchange, split
sizes, all-to-all-v of rows, arrival-order expert ids.  The device kernels are replaced by
torch CPU sorts here; the exchanged rows must land exactly where the reference's dispatch
golden puts them (fixtures from _compute_golden_recv)."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pypto_b200 import moe

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        t = torch.load(os.path.join(GOLDEN, f"ep_{world}.pt"), weights_only=True)
        L, K = t["l"], t["topk"]
        eid = t["indices"][rank].reshape(-1).long()
        order = torch.sort(eid, stable=True)[1]                 # (global expert, route) order
        counts = torch.bincount(eid, minlength=world * L).to(torch.int32)
        send_counts = counts.view(world, L)
        recv_counts = moe.exchange_counts(send_counts, None)
        in_split, out_split = send_counts.sum(1).tolist(), recv_counts.sum(1).tolist()
        x_s = t["x"][rank][order // K]
        id_s = order.to(torch.int32).reshape(-1, 1)
        x_r = moe.exchange_rows(x_s, sum(out_split), out_split, in_split, None)
        id_r = moe.exchange_rows(id_s, sum(out_split), out_split, in_split, None)
        e_r = moe.arrival_expert_ids(recv_counts)
        regroup = torch.sort(e_r.long(), stable=True)[1]        # (local expert, source, route)
        x_g, id_g = x_r[regroup], id_r[regroup, 0]
        cnt = torch.bincount(e_r.long(), minlength=L)
        ok = torch.equal(cnt.to(torch.int32), t["count"][rank])
        o = 0
        for e in range(L):
            n = int(cnt[e])
            ok &= torch.equal(x_g[o:o + n].view(torch.int16), t["recv_x"][rank, e, :n].view(torch.int16))
            ok &= torch.equal(id_g[o:o + n], t["recv_idx"][rank, e, :n])
            o += n
        # the way back: rows return to the senders' sorted order
        back = moe.exchange_rows(x_r, sum(in_split), in_split, out_split, None)
        ok &= torch.equal(back.view(torch.int16), x_s.view(torch.int16))
        result_q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ep_exchange_host_logic_over_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    results = dict(q.get(timeout=5) for _ in range(world))
    assert all(results.values()), results
