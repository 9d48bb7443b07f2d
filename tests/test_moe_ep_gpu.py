"""Expert-parallel MoE on 2 GPUs (one process per GPU, NCCL all-to-all for dispatch and
combine): every rank's output must equal the oracle's single-process result for its token
slice.  Skipped when fewer than 2 GPUs are visible."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import oracle
    from oracle import moe as omoe
    from pypto_b200.moe import MoELayer
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        tokens, hidden, inter, experts, topk = 256, 1024, 512, 16, 4
        m = oracle.inputs.moe_inputs(tokens=tokens, hidden=hidden, inter=inter, n_experts=experts, topk=topk, seed=9)
        y_exp, idx_exp, w_exp = omoe.moe_layer(m["x"], m["gate_w"], m["bias"], m["routed"], m["shared"], topk)
        L, tl = experts // world, tokens // world
        mine = {k: v[rank * L:(rank + 1) * L].cuda() for k, v in m["routed"].items()}
        layer = MoELayer(m["gate_w"].cuda(), m["bias"].cuda(), mine, {k: v.cuda() for k, v in m["shared"].items()},
                         topk, n_experts=experts, group=dist.group.WORLD)
        sl = slice(rank * tl, (rank + 1) * tl)
        y, _, _ = layer.forward(m["x"][sl].cuda(), routing=(idx_exp[sl].cuda(), w_exp[sl].cuda()))
        torch.cuda.synchronize()
        from pypto_b200 import ops
        status = ops.device_status()
        rel = ((y.cpu().float() - y_exp[sl].float()).norm() / y_exp[sl].float().norm()).item()
        y2, idx2, _ = layer.forward(m["x"][sl].cuda())        # own routing, a second pass over the exchange
        same = (idx2.cpu() == idx_exp[sl]).all(dim=1)
        rel2 = ((y2.cpu().float()[same] - y_exp[sl].float()[same]).norm() / y_exp[sl].float()[same].norm()).item()
        q.put((rank, rel, rel2, float(same.float().mean()), status[0]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_expert_parallel_layer_matches_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=300)
        assert p.exitcode == 0
    for _ in range(world):
        rank, rel, rel2, frac_same, status = q.get(timeout=5)
        assert status == 0
        assert rel < 2e-2 and rel2 < 2e-2 and frac_same > 0.97, (rank, rel, rel2, frac_same)
