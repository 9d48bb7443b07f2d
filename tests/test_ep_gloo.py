"""world_size-2 and -4 gloo runs (CPU) of the expert-parallel exchange: the host arithmetic of the product path
(``pypto_b200.moe.split_sizes``) driving a communicator with the interface of ``pypto_b200.comm.Communicator``
(gloo stands in for NCCL here), with the device plan kernels restated as torch CPU sorts.  The exchanged rows
must land exactly where the reference's dispatch golden puts them (fixtures from _compute_golden_recv), and
return to their senders in sorted order."""

import os
import queue
import socket
import traceback

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


class GlooComm:
    """The two collectives of pypto_b200.comm.Communicator over torch.distributed (CPU tensors)."""

    def __init__(self):
        self.rank, self.world = dist.get_rank(), dist.get_world_size()

    def all_to_all(self, send, recv):
        dist.all_to_all_single(recv, send)

    def all_to_all_v(self, send, send_rows, recv, recv_rows):
        dist.all_to_all_single(recv[:sum(recv_rows)], send[:sum(send_rows)], list(recv_rows), list(send_rows))


def _worker(rank, world, port, result_q):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        comm = GlooComm()
        t = torch.load(os.path.join(GOLDEN, f"ep_{world}.pt"), weights_only=True)
        L, K = t["l"], t["topk"]
        eid = t["indices"][rank].reshape(-1).long()
        # dispatch plan (moe_dispatch_plan restated): routes sorted by global expert, ties by route id
        route_at = torch.sort(eid, stable=True)[1]
        counts = torch.bincount(eid, minlength=world * L).to(torch.int32)
        offsets = torch.cat([torch.zeros(1, dtype=torch.int32), counts.cumsum(0).to(torch.int32)])
        send_counts = counts.view(world, L).contiguous()
        recv_counts = torch.empty_like(send_counts)
        comm.all_to_all(send_counts, recv_counts)
        send_rows, recv_rows = moe.split_sizes(offsets.tolist(), recv_counts.reshape(-1).tolist(), world, L)
        assert send_rows == send_counts.sum(1).tolist() and recv_rows == recv_counts.sum(1).tolist()
        # payload rows: x row and route id side by side, as bytes
        x_s = t["x"][rank][route_at // K]
        payload = torch.cat([x_s.view(torch.uint8), route_at.to(torch.int32).reshape(-1, 1).view(torch.uint8)], dim=1)
        arrived = sum(recv_rows)
        recv = torch.empty(arrived, payload.shape[1], dtype=torch.uint8)
        comm.all_to_all_v(payload.contiguous(), send_rows, recv, recv_rows)
        # receive plan (moe_recv_plan restated): arrival rows are source-major, local-expert-minor
        e_r = torch.repeat_interleave(torch.arange(L).repeat(world), recv_counts.reshape(-1).long())
        arrival_of = torch.sort(e_r, stable=True)[1]            # grouped row -> arrival row
        grouped = recv[arrival_of]
        d_bytes = t["x"].shape[2] * 2
        x_g = grouped[:, :d_bytes].contiguous().view(torch.int16)
        id_g = grouped[:, d_bytes:].contiguous().view(torch.int32)[:, 0]
        cnt = torch.bincount(e_r, minlength=L)
        ok = torch.equal(cnt.to(torch.int32), t["count"][rank])
        o = 0
        for e in range(L):
            n = int(cnt[e])
            ok &= torch.equal(x_g[o:o + n], t["recv_x"][rank, e, :n].view(torch.int16))
            ok &= torch.equal(id_g[o:o + n], t["recv_idx"][rank, e, :n])
            o += n
        # the way back: arrival-order rows return to the senders' sorted order
        back = torch.empty_like(payload)
        comm.all_to_all_v(recv, recv_rows, back, send_rows)
        ok &= torch.equal(back, payload)
        result_q.put((rank, "ok", bool(ok)))
        dist.destroy_process_group()
    except BaseException:
        result_q.put((rank, "error", traceback.format_exc()))
        os._exit(1)


@pytest.mark.parametrize("world", [2, 4])
def test_ep_exchange_host_logic_over_gloo(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    results = {}
    try:
        for p in procs:
            p.start()
        for _ in range(world):
            try:
                rank, status, payload = q.get(timeout=120)
            except queue.Empty:
                raise AssertionError(f"a rank did not report; got {results}") from None
            assert status == "ok", payload
            results[rank] = payload
        for p in procs:
            p.join(timeout=30)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    assert all(results.values()), results


def test_split_sizes_arithmetic():
    # 2 ranks x 3 local experts; this rank routes 1, 0, 2 rows to rank 0's experts and 4, 0, 1 to rank 1's
    offsets = [0, 1, 1, 3, 7, 7, 8]
    recv_counts = [2, 0, 0, 5, 1, 1]        # [source 0: experts 0..2, source 1: experts 0..2]
    assert moe.split_sizes(offsets, recv_counts, 2, 3) == ([3, 5], [2, 7])
