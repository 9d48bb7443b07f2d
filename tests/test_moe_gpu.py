"""GPU parity for the MoE path: top-k (bit-exact indices), FP8 row quantisation (bit-exact),
dispatch plan (bit-exact against the reference-derived fixture), grouped FP8 expert GEMM and
the whole layer against the oracle."""

import pytest
import torch

import oracle
from oracle import ep as oep
from oracle import moe as omoe

pytestmark = pytest.mark.gpu


def _ops():
    from pypto_b200 import ops
    return ops


def test_topk_indices_bit_exact_on_unique_scores(golden):
    # unique values as in the reference's sort tests (tests/st/runtime/ops/test_sort.py:443-445)
    src = golden("sort_unique_2048")["src"].reshape(8, 256)
    scores = torch.sigmoid(src / 4)
    bias = torch.linspace(-0.1, 0.1, 256)
    exp_idx, exp_w = omoe.topk_from_scores(scores, bias, 8)
    idx, w = _ops().moe_topk(scores.cuda(), bias.cuda(), 8)
    assert torch.equal(idx.cpu(), exp_idx)
    assert torch.allclose(w.cpu(), exp_w, rtol=1e-6, atol=1e-7)


def test_topk_random_scores_and_ties():
    g = torch.Generator().manual_seed(0)
    scores = torch.rand(1000, 256, generator=g)
    bias = torch.rand(256, generator=g) * 0.2 - 0.1
    exp_idx, exp_w = omoe.topk_from_scores(scores, bias, 8)
    idx, w = _ops().moe_topk(scores.cuda(), bias.cuda(), 8)
    assert torch.equal(idx.cpu(), exp_idx) and torch.allclose(w.cpu(), exp_w, rtol=1e-6, atol=1e-7)
    tied = torch.tensor([[0.5, 0.9, 0.9, 0.1, 0.9], [0.2] * 5])
    exp_idx, _ = omoe.topk_from_scores(tied, torch.zeros(5), 3)
    idx, _ = _ops().moe_topk(tied.cuda(), None, 3)
    assert idx.cpu().tolist() == exp_idx.tolist() == [[1, 2, 4], [0, 1, 2]]


def test_fused_gate_topk_from_logits():
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(300, 64, generator=g)
    bias = torch.rand(64, generator=g) * 0.2 - 0.1
    scores = torch.sigmoid(logits)
    exp_idx, exp_w = omoe.topk_from_scores(scores, bias, 6)
    idx, w = _ops().moe_topk(logits.cuda(), bias.cuda(), 6, is_logits=True)
    sel = scores + bias
    mism = idx.cpu() != exp_idx
    # a differing index is only acceptable on a numerical near-tie of the selection score
    gap = (torch.gather(sel, 1, idx.cpu().long()) - torch.gather(sel, 1, exp_idx.long())).abs()
    assert (gap[mism] < 1e-6).all()
    assert torch.allclose(w.cpu()[~mism.any(1)], exp_w[~mism.any(1)], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_quantize_rows_bit_exact(dtype):
    g = torch.Generator().manual_seed(2)
    x = (torch.randn(77, 512, generator=g) * torch.rand(77, 1, generator=g) * 10).to(dtype)
    x[3, 128:256] = 0
    q_exp, s_exp = omoe.quantize_rows(x)
    q, s = _ops().quantize_rows(x.cuda())
    assert torch.equal(s.cpu(), s_exp)
    assert torch.equal(q.cpu().view(torch.uint8), q_exp.view(torch.uint8))


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_dispatch_plan_matches_reference_protocol(golden, n_ranks):
    """Replay the N-rank dispatch on one GPU: per source rank sort routes by global expert,
    hand each destination its (source-major) rows, regroup by local expert -- and compare with
    the goldens of the reference's _compute_golden_recv bit for bit."""
    ops = _ops()
    t = golden(f"ep_{n_ranks}")
    L, K, T = t["l"], t["topk"], t["t"]
    plans = []
    for s in range(n_ranks):
        eid = t["indices"][s].reshape(-1).to(torch.int32).cuda()
        counts, offsets, pos, route_at = ops.moe_dispatch_plan(eid, n_ranks * L)
        x_s, = ops.gather_rows([t["x"][s].cuda()], route_at, div=K)
        w_s, = ops.gather_rows([t["weights"][s].reshape(-1, 1).cuda()], route_at, div=1)
        plans.append((counts.cpu(), offsets.cpu(), route_at.cpu(), x_s.cpu(), w_s.cpu()))
    for d in range(n_ranks):
        rows_x, rows_w, rows_id, rows_e = [], [], [], []
        for s in range(n_ranks):
            counts, offsets, route_at, x_s, w_s = plans[s]
            lo, hi = int(offsets[d * L]), int(offsets[(d + 1) * L])
            rows_x.append(x_s[lo:hi]); rows_w.append(w_s[lo:hi]); rows_id.append(route_at[lo:hi])
            rows_e.append(torch.repeat_interleave(torch.arange(L, dtype=torch.int32), counts[d * L:(d + 1) * L].long()))
        x_r, w_r, id_r, e_r = (torch.cat(v) for v in (rows_x, rows_w, rows_id, rows_e))
        c2, off2, _pos2, route_at2 = ops.moe_dispatch_plan(e_r.cuda(), L)
        x_g, w_g, id_g = ops.gather_rows([x_r.cuda(), w_r.cuda(), id_r.reshape(-1, 1).cuda()], route_at2, div=1)
        assert torch.equal(c2.cpu(), t["count"][d])
        for e in range(L):
            n, o = int(c2[e]), int(off2[e])
            assert torch.equal(x_g[o:o + n].cpu().view(torch.int16), t["recv_x"][d, e, :n].view(torch.int16))
            assert torch.equal(w_g[o:o + n, 0].cpu(), t["recv_w"][d, e, :n])
            assert torch.equal(id_g[o:o + n, 0].cpu(), t["recv_idx"][d, e, :n])


def test_combine_matches_reference_golden(golden):
    """combine_step: every (t, k) row back at slot t*K+k, fp32 sum over k (golden
    _compute_golden_routed, test_l3_ep_dispatch_combine.py:617-629)."""
    t = golden("ep_2")
    K, T = t["topk"], t["t"]
    for r in range(2):
        rows = oep.standin_expert(t["x"][r].repeat_interleave(K, 0), t["weights"][r].reshape(-1))
        pos = torch.arange(T * K, dtype=torch.int32)
        _y, y32 = _ops().moe_combine(rows.cuda(), pos.cuda(), None, T, K, want_f32=True)
        assert torch.equal(y32.cpu(), t["routed"][r])


def _pack(stacked):
    from pypto_b200.moe import pack_expert_weights
    return pack_expert_weights({k: v.cuda() for k, v in stacked.items()})


@pytest.mark.parametrize("experts,hidden,inter,rows_per", [(3, 256, 128, [5, 0, 200]), (4, 512, 256, [128, 129, 1, 60]),
                                                           (2, 7168, 256, [130, 40])])
def test_grouped_fp8_gemms_match_oracle(experts, hidden, inter, rows_per):
    ops = _ops()
    m = oracle.inputs.moe_inputs(tokens=sum(rows_per), hidden=hidden, inter=inter, n_experts=experts, topk=1,
                                 shared=False, seed=experts)
    xq, xs = omoe.quantize_rows(m["x"])
    off = torch.tensor([0] + list(torch.tensor(rows_per).cumsum(0)), dtype=torch.int32)
    pk = _pack(m["routed"])
    act_dev = ops.moe_expert_gemm(True, pk["w_gu"], pk["s_gu"], xq.cuda(), xs.cuda(), off.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()
    route_w = torch.rand(sum(rows_per)) + 0.5
    for e in range(experts):
        lo, hi = int(off[e]), int(off[e + 1])
        if lo == hi:
            continue
        ex = omoe.expert_slice(m["routed"], e)
        g = omoe.fp8_gemm(xq[lo:hi], xs[lo:hi], ex["wg"], ex["sg"])
        u = omoe.fp8_gemm(xq[lo:hi], xs[lo:hi], ex["wu"], ex["su"])
        act = (g * torch.sigmoid(g) * u).bfloat16().float()
        got = act_dev[lo:hi].cpu().float()
        assert (got - act).abs().max().item() <= 1e-2 * act.abs().max().item() + 1e-7
    act_q, act_s = ops.quantize_rows(act_dev)
    # GEMM2 on the device's own (act_q, act_s): compare with the oracle GEMM on the same operands
    out = ops.moe_expert_gemm(False, pk["w_d"], pk["s_d"], act_q, act_s, off.cuda(), route_w.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()
    for e in range(experts):
        lo, hi = int(off[e]), int(off[e + 1])
        if lo == hi:
            continue
        ex = omoe.expert_slice(m["routed"], e)
        ref = omoe.fp8_gemm(act_q[lo:hi].cpu(), act_s[lo:hi].cpu(), ex["wd"], ex["sd"]) * route_w[lo:hi, None]
        got = out[lo:hi].cpu().float()
        assert (got - ref).abs().max().item() <= 1e-2 * ref.abs().max().item() + 1e-6


def test_expert_gemm_is_reproducible_under_stream_concurrency():
    """The grouped GEMM has no atomics: repeated launches on the same operands must give identical bits, also
    while a second stream runs the same kernel (the shared expert does in the layer).  Long K (7168, the
    four-stage pipeline), many units per CTA and ragged token counts: a pipeline stage recycled too early
    shows up here as a changed output."""
    ops = _ops()
    experts, hidden, inter = 24, 7168, 512
    g = torch.Generator(device="cuda").manual_seed(7)
    counts = torch.tensor([0, 481, 3, 128, 129, 257, 64, 0, 300, 17, 255, 1] * 2, dtype=torch.int32)
    off = torch.cat([torch.zeros(1, dtype=torch.int32), counts.cumsum(0).int()]).cuda()
    rows = int(counts.sum())
    w_gu = torch.randn(experts, 2 * inter, hidden, device="cuda", generator=g).to(torch.float8_e4m3fn)
    s_gu = torch.rand(experts, 2 * inter // 128, hidden // 128, device="cuda", generator=g) * 0.01 + 0.001
    w_d = torch.randn(experts, hidden, inter, device="cuda", generator=g).to(torch.float8_e4m3fn)
    s_d = torch.rand(experts, hidden // 128, inter // 128, device="cuda", generator=g) * 0.01 + 0.001
    x = torch.randn(rows, hidden, device="cuda", generator=g).bfloat16()
    xq, xs = ops.quantize_rows(x)
    side = torch.cuda.Stream()
    first_a = first_y = None
    for _ in range(12):
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ops.moe_expert_gemm(True, w_gu[:1], s_gu[:1], xq, xs, torch.tensor([0, rows], dtype=torch.int32, device="cuda"))
        a = ops.moe_expert_gemm(True, w_gu, s_gu, xq, xs, off)
        aq, asc = ops.quantize_rows(a)
        y = ops.moe_expert_gemm(False, w_d, s_d, aq, asc, off, None)
        torch.cuda.current_stream().wait_stream(side)
        if first_a is None:
            first_a, first_y = a.clone(), y.clone()
        else:
            assert torch.equal(a, first_a) and torch.equal(y, first_y)
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.isfinite(first_y.float()).all()


def _layer_vs_oracle(tokens, hidden, inter, experts, topk, seed):
    from pypto_b200.moe import MoELayer
    m = oracle.inputs.moe_inputs(tokens=tokens, hidden=hidden, inter=inter, n_experts=experts, topk=topk, seed=seed)
    y_exp, idx_exp, w_exp = omoe.moe_layer(m["x"], m["gate_w"], m["bias"], m["routed"], m["shared"], topk)
    layer = MoELayer(m["gate_w"].cuda(), m["bias"].cuda(), {k: v.cuda() for k, v in m["routed"].items()},
                     {k: v.cuda() for k, v in m["shared"].items()}, topk)
    # routing taken from the oracle so that the expert path is compared on identical routes
    y, _, _ = layer.forward(m["x"].cuda(), routing=(idx_exp.cuda(), w_exp.cuda()))
    torch.cuda.synchronize()
    _ops().check_device_status()
    y_own, idx, w = layer.forward(m["x"].cuda())
    return m, y.cpu().float(), y_exp.float(), idx.cpu(), idx_exp, y_own.cpu().float()


@pytest.mark.parametrize("tokens,hidden,inter,experts,topk", [(64, 512, 256, 8, 2), (300, 1024, 512, 32, 8)])
def test_moe_layer_matches_oracle(tokens, hidden, inter, experts, topk):
    m, y, y_exp, idx, idx_exp, y_own = _layer_vs_oracle(tokens, hidden, inter, experts, topk, seed=tokens)
    rel = ((y - y_exp).norm() / y_exp.norm()).item()
    assert rel < 2e-2, rel     # fp8 bar of the workload is 5e-2; identical quantisation points give far less
    same = (idx == idx_exp).all(dim=1)
    assert same.float().mean() > 0.98          # gate logits come from a different GEMM: near-ties may flip
    assert ((y_own[same] - y_exp[same]).norm() / y_exp[same].norm()).item() < 2e-2
    # looser mathematical target: dequantised weights, bf16 activations, fp32 math
    y_math = omoe.dequant_reference(m["x"], idx_exp.long(), omoe.gate_topk(m["x"], m["gate_w"], m["bias"], topk)[1],
                                    m["routed"], m["shared"])
    assert ((y - y_math).norm() / y_math.norm()).item() < 5e-2
