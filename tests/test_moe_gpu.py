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
    R = t["r"]
    for d in range(n_ranks):
        rows_x, rows_w, rows_id = [], [], []
        for s in range(n_ranks):
            counts, offsets, route_at, x_s, w_s = plans[s]
            lo, hi = int(offsets[d * L]), int(offsets[(d + 1) * L])
            rows_x.append(x_s[lo:hi]); rows_w.append(w_s[lo:hi]); rows_id.append(route_at[lo:hi])
        x_r, w_r, id_r = (torch.cat(v) for v in (rows_x, rows_w, rows_id))        # arrival order: source-major
        recv_counts = torch.stack([plans[s][0][d * L:(d + 1) * L] for s in range(n_ranks)]).contiguous().cuda()
        arrived = x_r.shape[0]
        # dense grouping (what the expert GEMM consumes)
        c2, off2, arrival_of, grouped_of = ops.moe_recv_plan(recv_counts, arrived)
        x_g, w_g, id_g = ops.gather_rows([x_r.cuda(), w_r.cuda(), id_r.reshape(-1, 1).cuda()], arrival_of[:arrived], div=1)
        assert torch.equal(c2.cpu(), t["count"][d])
        assert torch.equal(arrival_of[:arrived][grouped_of[:arrived].long()].cpu(), torch.arange(arrived, dtype=torch.int32))
        for e in range(L):
            n, o = int(c2[e]), int(off2[e])
            assert torch.equal(x_g[o:o + n].cpu().view(torch.int16), t["recv_x"][d, e, :n].view(torch.int16))
            assert torch.equal(w_g[o:o + n, 0].cpu(), t["recv_w"][d, e, :n])
            assert torch.equal(id_g[o:o + n, 0].cpu(), t["recv_idx"][d, e, :n])
        # the reference's padded [L, R] receive layout: unused slots stay zero, as in its zero-initialised outputs
        c3, off3, arrival_pad, _g3 = ops.moe_recv_plan(recv_counts, L * R, slot_stride=R)
        x_p, w_p, id_p = ops.gather_rows([x_r.cuda(), w_r.cuda(), id_r.reshape(-1, 1).cuda()], arrival_pad, div=1)
        assert torch.equal(c3.cpu(), t["count"][d]) and off3.cpu().tolist() == [e * R for e in range(L + 1)]
        assert torch.equal(x_p.cpu().view(torch.int16).reshape(L, R, -1), t["recv_x"][d].view(torch.int16))
        assert torch.equal(w_p.cpu().reshape(L, R), t["recv_w"][d])
        assert torch.equal(id_p.cpu().reshape(L, R), t["recv_idx"][d])
    torch.cuda.synchronize()
    ops.check_device_status()


def test_expert_id_outside_the_buckets_is_reported_not_dereferenced():
    """A route whose expert id is not a bucket: no address is formed from it; the route gets pos -1, the tail
    of route_at is -1, gathers through those entries give zero rows, the combine skips the route, and the
    error word carries code 3."""
    from pypto_b200 import _lib
    ops = _ops()
    torch.cuda.synchronize()
    ops.device_status()                                    # start from a clear word
    ids = torch.tensor([3, 1, 9999, 0, -7, 1], dtype=torch.int32, device="cuda")
    counts, offsets, pos, route_at = ops.moe_dispatch_plan(ids, 4)
    torch.cuda.synchronize()
    assert counts.cpu().tolist() == [1, 2, 0, 1] and offsets.cpu().tolist() == [0, 1, 3, 3, 4]
    assert pos.cpu().tolist() == [3, 1, -1, 0, -1, 2]
    assert route_at.cpu().tolist() == [3, 1, 5, 0, -1, -1]
    x = torch.arange(6 * 8, dtype=torch.float32, device="cuda").reshape(6, 8) + 1
    rows, = ops.gather_rows([x], route_at, div=1)
    assert torch.equal(rows[:4].cpu(), x.cpu()[[3, 1, 5, 0]]) and torch.count_nonzero(rows[4:]) == 0
    y, y32 = ops.moe_combine(x[:4].bfloat16().repeat(1, 1).contiguous(), pos, None, 3, 2, want_f32=True)
    xb = x[:4].bfloat16().float().cpu()
    assert torch.equal(y32.cpu(), torch.stack([xb[3] + xb[1], xb[0], xb[2]]))   # routes (1,0) and (2,0) contribute nothing
    code = ops.device_status()
    assert code[0] == 3 and code[1] == 60
    with pytest.raises(_lib.PtoError):
        ops.moe_dispatch_plan(ids, 4)
        torch.cuda.synchronize()
        ops.check_device_status()
    assert ops.device_status()[0] == 0                     # reading cleared it


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


def _pow2(shape, lo, hi, g):
    """Random powers of two 2^lo .. 2^hi."""
    return torch.pow(2.0, torch.randint(lo, hi + 1, shape, generator=g).float())


@pytest.mark.parametrize("hidden,inter,rows_per", [(7168, 256, [130, 1, 0, 260]), (2048, 512, [128, 77])])
def test_expert_gemm_exact_known_answer(hidden, inter, rows_per):
    """Known-answer test in the style of the reference's MX matmul test
    (tests/st/runtime/ops/test_matmul_mx.py:154-165, 283: integer-valued e4m3 operands, power-of-two scales,
    rtol = atol = 0).  Every partial sum is an exactly representable fp32 number whatever the summation order,
    so the grouped GEMM must equal the oracle bit for bit -- in the plain mode (the down projection; K = 2048
    runs the six-stage ring, K = 7168 the four-stage one) and in the SwiGLU mode, where positive gate operands
    put every gate value far above the point at which sigmoid(g) rounds to 1, so that silu(g) * u = g * u."""
    ops = _ops()
    g = torch.Generator().manual_seed(hidden + inter)
    experts, rows = len(rows_per), sum(rows_per)
    off = torch.tensor([0] + list(torch.tensor(rows_per).cumsum(0)), dtype=torch.int32)
    # plain mode: out = bf16(acc * route_w), signed operands
    x = torch.randint(-2, 3, (rows, hidden), generator=g).float()
    xs = _pow2((rows, hidden // 128), -1, 2, g)
    w = torch.randint(-2, 3, (experts, hidden, inter), generator=g).float()            # x @ W layout [K, N]
    ws = _pow2((experts, hidden // 128, inter // 128), -2, 1, g)
    route_w = _pow2((rows,), -2, 0, g)
    xq, wq = x.to(torch.float8_e4m3fn), w.to(torch.float8_e4m3fn)
    w_kmajor = wq.view(torch.uint8).transpose(1, 2).contiguous().view(torch.float8_e4m3fn).cuda()
    out = ops.moe_expert_gemm(False, w_kmajor, ws.transpose(1, 2).contiguous().cuda(), xq.cuda(), xs.cuda(), off.cuda(),
                              route_w.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()
    for e in range(experts):
        lo, hi = int(off[e]), int(off[e + 1])
        if lo == hi:
            continue
        ref = (omoe.fp8_gemm(xq[lo:hi], xs[lo:hi], wq[e], ws[e]) * route_w[lo:hi, None]).bfloat16()
        assert torch.equal(out[lo:hi].cpu().view(torch.int16), ref.view(torch.int16)), (e, (out[lo:hi].cpu().float() - ref.float()).abs().max())
    # SwiGLU mode: gate operands positive (so g >= K/2 >> 17 and sigmoid(g) == 1 in fp32), up weights signed
    xp = torch.randint(1, 3, (rows, hidden), generator=g).float()
    wg = torch.randint(1, 3, (experts, hidden, inter), generator=g).float()
    wu = torch.randint(-2, 3, (experts, hidden, inter), generator=g).float()
    sg, su = _pow2((experts, hidden // 128, inter // 128), -1, 0, g), _pow2((experts, hidden // 128, inter // 128), -2, 0, g)
    xs1 = _pow2((rows, hidden // 128), 0, 1, g)
    xpq = xp.to(torch.float8_e4m3fn)
    pk = _pack(dict(wg=wg.to(torch.float8_e4m3fn), sg=sg, wu=wu.to(torch.float8_e4m3fn), su=su,
                    wd=torch.zeros(experts, inter, 128).to(torch.float8_e4m3fn), sd=torch.ones(experts, inter // 128, 1)))
    act = ops.moe_expert_gemm(True, pk["w_gu"], pk["s_gu"], xpq.cuda(), xs1.cuda(), off.cuda())
    torch.cuda.synchronize()
    ops.check_device_status()
    for e in range(experts):
        lo, hi = int(off[e]), int(off[e + 1])
        if lo == hi:
            continue
        gate = omoe.fp8_gemm(xpq[lo:hi], xs1[lo:hi], wg[e].to(torch.float8_e4m3fn), sg[e])
        up = omoe.fp8_gemm(xpq[lo:hi], xs1[lo:hi], wu[e].to(torch.float8_e4m3fn), su[e])
        assert gate.min() > 20
        ref = (gate * torch.sigmoid(gate) * up).bfloat16()
        assert torch.equal(act[lo:hi].cpu().view(torch.int16), ref.view(torch.int16)), (e, (act[lo:hi].cpu().float() - ref.float()).abs().max())


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
    # ... and the bits that repeat are the right ones: three experts (481, 129 and 1 rows) against the oracle
    xq_h, xs_h, offs = xq.cpu(), xs.cpu(), off.cpu().tolist()
    aq_h, as_h = (v.cpu() for v in ops.quantize_rows(first_a))
    for e in (1, 4, 11):
        lo, hi = offs[e], offs[e + 1]
        w_e = w_gu[e].cpu().view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)      # [hidden, 2*inter]
        s_e = s_gu[e].cpu().t().contiguous()
        gu = omoe.fp8_gemm(xq_h[lo:hi], xs_h[lo:hi], w_e, s_e)
        gate, up = gu[:, :inter], gu[:, inter:]
        act = (gate * torch.sigmoid(gate) * up).bfloat16().float()
        got = first_a[lo:hi].cpu().float()
        assert (got - act).abs().max() <= 1e-2 * act.abs().max() + 1e-7, e
        wd_e = w_d[e].cpu().view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)      # [inter, hidden]
        ref = omoe.fp8_gemm(aq_h[lo:hi], as_h[lo:hi], wd_e, s_d[e].cpu().t().contiguous())
        got = first_y[lo:hi].cpu().float()
        assert (got - ref).abs().max() <= 1e-2 * ref.abs().max() + 1e-6, e


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
    assert layer.status()[0] == 0           # the layer's kernels report into its own error word
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


def test_moe_layer_object_regrows_times_its_phases_and_reports_bad_routes():
    """The runtime's layer object behind MoELayer.forward: a call with more tokens than it was sized for builds a
    larger one; a call with a timer returns the eight phase times; a route to an expert that does not exist is
    reported in the layer's error word (code 3, the route's index) and the layer stays usable."""
    from pypto_b200.moe import MoELayer, PhaseTimer
    tokens, hidden, inter, experts, topk = 96, 512, 256, 8, 2
    m = oracle.inputs.moe_inputs(tokens=tokens, hidden=hidden, inter=inter, n_experts=experts, topk=topk, shared=False,
                                 seed=21)
    y_exp, idx_exp, w_exp = omoe.moe_layer(m["x"], m["gate_w"], m["bias"], m["routed"], None, topk)
    layer = MoELayer(m["gate_w"].cuda(), m["bias"].cuda(), {k: v.cuda() for k, v in m["routed"].items()}, None, topk)
    x = m["x"].cuda()
    y_small, _, _ = layer.forward(x[:32], routing=(idx_exp[:32].cuda(), w_exp[:32].cuda()))
    first = layer._handle_tokens
    timer = PhaseTimer()
    y, _, _ = layer.forward(x, routing=(idx_exp.cuda(), w_exp.cuda()), timer=timer)
    assert first == 32 and layer._handle_tokens == tokens
    ph = timer.result()
    assert set(ph) == set(MoELayer.PHASES) and all(v >= 0 for v in ph.values()) and ph["experts"] > 0
    assert layer.status()[0] == 0
    for got, exp in ((y_small.cpu().float(), y_exp[:32].float()), (y.cpu().float(), y_exp.float())):
        assert ((got - exp).norm() / exp.norm()).item() < 2e-2
    bad = idx_exp.clone()
    bad[5, 1] = experts + 3
    layer.forward(x, routing=(bad.cuda(), w_exp.cuda()))
    code, site, _cta, detail = layer.status()
    assert code == 3 and site == 60 and detail == 5 * topk + 1
    y_again, _, _ = layer.forward(x, routing=(idx_exp.cuda(), w_exp.cuda()))
    assert layer.status()[0] == 0
    assert torch.equal(y_again.cpu(), y.cpu())
    layer.close()


def test_moe_layer_callable_of_the_op_table_matches_the_layer_object():
    """``moe_layer`` in the runtime's operator table (``pto_register_callable`` / ``pto_run``): tensors in the
    kernels' packed layout, top-k as the scalar.  Same kernels as ``MoELayer.forward``, so the outputs are equal;
    a second call with fewer tokens reuses the layer the first call built."""
    from pypto_b200.moe import MoELayer
    from pypto_b200.runtime import ChipWorker, DeviceTensor, RunConfig
    tokens, hidden, inter, experts, topk = 80, 512, 256, 8, 2
    m = oracle.inputs.moe_inputs(tokens=tokens, hidden=hidden, inter=inter, n_experts=experts, topk=topk, seed=33)
    layer = MoELayer(m["gate_w"].cuda(), m["bias"].cuda(), {k: v.cuda() for k, v in m["routed"].items()},
                     {k: v.cuda() for k, v in m["shared"].items()}, topk)
    x = m["x"].cuda()
    y_ref, _, _ = layer.forward(x)
    y_exp, _, _ = omoe.moe_layer(m["x"], m["gate_w"], m["bias"], m["routed"], m["shared"], topk)

    def dt(t):
        return DeviceTensor(t.data_ptr(), tuple(t.shape), t.dtype, buffer=t)

    worker = ChipWorker(RunConfig(platform="b200"))
    worker.init()
    try:
        weights = [layer.gate_packed, layer.bias] + [layer.routed[k] for k in ("w_gu", "s_gu", "w_d", "s_d")] + \
                  [layer.shared[k] for k in ("w_gu", "s_gu", "w_d", "s_d")]
        for n in (tokens, 48):
            y = torch.zeros(n, hidden, dtype=torch.bfloat16, device="cuda")
            torch.cuda.synchronize()
            worker.launch("moe_layer", [dt(x[:n].contiguous())] + [dt(w) for w in weights] + [dt(y)], [topk])
            worker.synchronize()
            assert worker.device_status()[0] == 0
            assert torch.equal(y.cpu(), y_ref[:n].cpu())
        rel = ((y_ref.cpu().float() - y_exp.float()).norm() / y_exp.float().norm()).item()
        assert rel < 3e-2, rel     # own routing: a near-tie in the gate may pick another expert for a token
        with pytest.raises(Exception):
            worker.launch("moe_layer", [dt(x)] + [dt(w) for w in weights[:-1]] + [dt(y)], [topk])
    finally:
        worker.close()
