"""Expert-parallel MoE on 2, 4 and 8 GPUs (one process per GPU): every rank's output must equal the oracle's
single-process result for its token slice.  Rows travel through the library's NCCL communicator, through peer memory
on the way back (the default on one node), or through peer memory both ways (PTO_EP_PEER = 0 / 1 / 2, set in every
rank); each case checks that the layer reports the path it was asked for.  Each world size is skipped when fewer GPUs
are visible."""

import os
import queue
import sys
import traceback

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# 7168 hidden channels: the gate/up GEMM of the benchmark layer (56 K blocks, four-stage pipeline)
SHAPE = dict(tokens=256, hidden=7168, inter=256, experts=16, topk=4)


def _worker(rank, world, uid, case_path, peer, q):
    try:
        sys.path.insert(0, ROOT)
        if peer is not None:
            os.environ["PTO_EP_PEER"] = str(peer)
        from pypto_b200 import ops
        from pypto_b200.comm import Communicator
        from pypto_b200.moe import MoELayer, PhaseTimer
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        torch.cuda.set_device(rank)
        tokens, experts, topk = SHAPE["tokens"], SHAPE["experts"], SHAPE["topk"]
        case = torch.load(case_path, weights_only=True)       # inputs and the oracle's layer output, made once by the parent
        m, y_exp, idx_exp, w_exp = case["inputs"], case["y"], case["idx"], case["w"]
        L, tl = experts // world, tokens // world
        mine = {k: v[rank * L:(rank + 1) * L].cuda() for k, v in m["routed"].items()}
        comm = Communicator(rank, world, uid, rank)          # collective: after everything that can fail alone
        try:
            layer = MoELayer(m["gate_w"].cuda(), m["bias"].cuda(), mine, {k: v.cuda() for k, v in m["shared"].items()},
                             topk, n_experts=experts, comm=comm)
            sl = slice(rank * tl, (rank + 1) * tl)
            y, _, _ = layer.forward(m["x"][sl].cuda(), routing=(idx_exp[sl].cuda(), w_exp[sl].cuda()))
            torch.cuda.synchronize()
            status = ops.device_status()
            side_status = layer.status()          # the layer's own error word (all of its kernels report there)
            rel = ((y.cpu().float() - y_exp[sl].float()).norm() / y_exp[sl].float().norm()).item()
            timer = PhaseTimer()
            y2, idx2, _ = layer.forward(m["x"][sl].cuda(), timer=timer)     # own routing, a second pass over the exchange
            phases = timer.result()
            same = (idx2.cpu() == idx_exp[sl]).all(dim=1)
            rel2 = ((y2.cpu().float()[same] - y_exp[sl].float()[same]).norm() / y_exp[sl].float()[same].norm()).item()
            q.put((rank, "ok", rel, rel2, float(same.float().mean()), status[0] or side_status[0], sorted(phases),
                   layer.peer_exchange_level))
        finally:
            comm.close()
    except BaseException:
        q.put((rank, "error", traceback.format_exc()))
        os._exit(1)         # leave at once: a peer may be blocked in a collective that will never complete


def run_ranks(target, world, args=(), timeout=420):
    """Start one child per rank, collect one message from each, and never leave a child behind: on a failure
    or a timeout every child still alive is terminated, then killed."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=target, args=(r, world) + tuple(args) + (q,)) for r in range(world)]
    results = []
    try:
        for p in procs:
            p.start()
        for _ in range(world):
            try:
                msg = q.get(timeout=timeout)
            except queue.Empty:
                raise AssertionError(f"a rank did not report within {timeout} s; got {results}") from None
            results.append(msg)
            if msg[1] != "ok":
                raise AssertionError(f"rank {msg[0]} failed:\n{msg[2]}")
        for p in procs:
            p.join(timeout=60)
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
                p.join(timeout=10)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return results


@pytest.fixture(scope="module")
def oracle_case(tmp_path_factory):
    """Inputs of the case and the oracle's single-process layer output, computed once for every world size."""
    import oracle
    from oracle import moe as omoe
    m = oracle.inputs.moe_inputs(tokens=SHAPE["tokens"], hidden=SHAPE["hidden"], inter=SHAPE["inter"],
                                 n_experts=SHAPE["experts"], topk=SHAPE["topk"], seed=9)
    y, idx, w = omoe.moe_layer(m["x"], m["gate_w"], m["bias"], m["routed"], m["shared"], SHAPE["topk"])
    path = str(tmp_path_factory.mktemp("ep_case") / "case.pt")
    torch.save(dict(inputs={k: v for k, v in m.items() if k != "topk"}, y=y, idx=idx, w=w), path)
    return path


@pytest.mark.parametrize("world,peer", [(2, None), (4, None), (8, None), (2, 0), (2, 2), (4, 2)])
def test_expert_parallel_layer_matches_oracle(world, peer, oracle_case):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    from pypto_b200 import comm
    results = run_ranks(_worker, world, args=(comm.unique_id(), oracle_case, peer))
    for rank, _ok, rel, rel2, frac_same, status, phases, level in results:
        assert status == 0
        assert level == (1 if peer is None else peer), (rank, level)      # one node: every rank maps every other
        assert rel < 2e-2 and rel2 < 2e-2 and frac_same > 0.97, (rank, rel, rel2, frac_same)
        assert {"plan", "pack", "exchange_out", "unpack", "experts", "exchange_back", "combine"} <= set(phases)
