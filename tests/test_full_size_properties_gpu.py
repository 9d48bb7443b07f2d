"""GPU: the benchmark workloads at their full sizes, checked through size-independent properties
(the CPU oracle cannot run these sizes in seconds) plus an oracle comparison on a sample."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_verify_attention_full_size_sample_and_value_linearity():
    """Speculative-verify attention at batch 256, q_len 4, 64/8 heads, ctx U[8192, 32768] (about
    24 GB of KV): (a) the first two sequences agree with the oracle; (b) doubling V doubles the
    output exactly (scaling by 2 is exact in bf16 and in every fp32 partial sum)."""
    import bench
    from pypto_b200 import ops
    if torch.cuda.mem_get_info()[0] < 60 << 30:
        pytest.skip("needs about 50 GB of free device memory")
    dev = torch.device("cuda", torch.cuda.current_device())
    g = bench.paged_inputs_device(dev, 7, **bench.VERIFY)
    kw = dict(num_heads=g["num_heads"], kv_heads=g["kv_heads"], head_dim=g["head_dim"], block_size=g["block_size"],
              scale=g["scale"], q_len=g["q_len"])
    out = ops.paged_attention(g["query"], g["key_cache"], g["value_cache"], g["block_table"], g["context_lens"], **kw)
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.isfinite(out.float()).all()
    sub = bench.host_subproblem(g, 2)
    from oracle import paged_attention as opa
    exp = opa.paged_attention(sub["query"], sub["key_cache"], sub["value_cache"], sub["block_table"],
                              sub["context_lens"], num_heads=g["num_heads"], head_dim=128, block_size=128,
                              scale=g["scale"], kv_heads=g["kv_heads"], q_len=g["q_len"]).bfloat16()
    got = out[: exp.shape[0]].cpu()
    assert torch.allclose(got.float(), exp.float(), rtol=2e-2, atol=4e-3)
    g["value_cache"].mul_(2)
    out2 = ops.paged_attention(g["query"], g["key_cache"], g["value_cache"], g["block_table"], g["context_lens"], **kw)
    torch.cuda.synchronize()
    assert torch.equal(out2.float(), out.float() * 2)


def test_moe_full_size_token_permutation_equivariance():
    """The 256 + 1 expert FP8 layer at 4096 tokens: quantisation and every dot product are per
    token, so with the routing held fixed, permuting the tokens permutes the output rows bit for
    bit (the gate logits themselves come from a stream-K GEMM whose fp32 atomics may flip a
    near-tie between runs, hence the fixed routing); the routing indices match the oracle's top-k
    on the device's own gate scores."""
    import bench
    from oracle import moe as omoe
    from pypto_b200 import ops
    from pypto_b200.moe import MoELayer
    if torch.cuda.mem_get_info()[0] < 40 << 30:
        pytest.skip("needs about 30 GB of free device memory")
    dev = torch.device("cuda", torch.cuda.current_device())
    m = bench.MOE
    gen = torch.Generator(device=dev).manual_seed(3)
    gate_w = (torch.randn(m["hidden"], m["n_experts"], device=dev, generator=gen) * 0.02).bfloat16()
    bias = torch.rand(m["n_experts"], device=dev, generator=gen) * 0.2 - 0.1
    layer = MoELayer.from_packed(ops.pack_weight(gate_w), bias,
                                 bench.synthetic_experts(dev, gen, m["n_experts"], m["hidden"], m["inter"]),
                                 bench.synthetic_experts(dev, gen, 1, m["hidden"], m["inter"]), m["topk"])
    x = torch.randn(m["tokens"], m["hidden"], device=dev, generator=gen).bfloat16()
    y, idx, w = layer.forward(x)
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.isfinite(y.float()).all() and y.float().abs().max() > 0
    perm = torch.randperm(m["tokens"], device=dev, generator=gen)
    y2, _, _ = layer.forward(x[perm].contiguous(), routing=(idx[perm].contiguous(), w[perm].contiguous()))
    torch.cuda.synchronize()
    assert torch.equal(y2.view(torch.int16), y[perm].view(torch.int16))
    scores = torch.sigmoid(ops.linear(x, layer.gate_packed)).cpu()
    exp_idx, _ = omoe.topk_from_scores(scores, bias.cpu(), m["topk"])
    assert (idx.cpu() == exp_idx).all(dim=1).float().mean() > 0.999   # sigmoid rounding may flip a near-tie

    # Oracle on a sample at the layer's own geometry (H = 7168 through the four-stage pipeline of the gate/up
    # GEMM, I = 2048 through the six-stage one of the down GEMM): 8 tokens spread over the batch, each through
    # its eight routed experts and the shared expert, with the device's routing.
    H, I = m["hidden"], m["inter"]
    sample = torch.arange(0, m["tokens"], m["tokens"] // 8)[:8] + 3
    xq, xs = omoe.quantize_rows(x[sample].cpu())
    idx_h, w_h = idx.cpu(), w.cpu()

    def oracle_expert(weights, e):
        """Expert e of a K-major device weight dict in the oracle's x @ W layout."""
        def t8(v):
            return v.cpu().view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)
        gu, s_gu = t8(weights["w_gu"][e]), weights["s_gu"][e].cpu().t().contiguous()
        return dict(wg=gu[:, :I], wu=gu[:, I:], sg=s_gu[:, :I // 128], su=s_gu[:, I // 128:],
                    wd=t8(weights["w_d"][e]), sd=weights["s_d"][e].cpu().t().contiguous())

    contrib = torch.zeros(len(sample), m["topk"], H)
    by_expert: dict = {}
    for i, t in enumerate(sample.tolist()):
        for k in range(m["topk"]):
            by_expert.setdefault(int(idx_h[t, k]), []).append((i, t, k))
    for e, uses in by_expert.items():
        ex = oracle_expert(layer.routed, e)
        rows = torch.tensor([i for i, _t, _k in uses])
        o = omoe.expert_ffn(xq[rows], xs[rows], ex)
        for j, (i, t, k) in enumerate(uses):
            contrib[i, k] = (o[j] * w_h[t, k]).bfloat16().float()
    y_exp = torch.zeros(len(sample), H)
    for k in range(m["topk"]):
        y_exp += contrib[:, k]
    y_exp += omoe.expert_ffn(xq, xs, oracle_expert(layer.shared, 0)).bfloat16().float()
    y_exp = y_exp.bfloat16().float()
    got = y[sample.to(dev)].cpu().float()
    rel = ((got - y_exp).norm() / y_exp.norm()).item()
    assert rel < 2e-2, rel
    per_row = (got - y_exp).norm(dim=1) / y_exp.norm(dim=1)
    assert per_row.max() < 5e-2, per_row


def test_matmul_mx_full_size_scale_shift_row_permutation_and_oracle_slab():
    """The MXFP8 matmul at the benchmark's 8192^3 (SM pairs, 256 x 224 tiles, scale blocks packed and fetched by TMA):
    (a) raising every scale code of `a` by one doubles the output exactly (a power of two, in every fp32 partial sum);
    (b) permuting the rows of `a` and of its scales permutes the output rows bit for bit (every row is accumulated
    in the same order whatever tile and whichever CTA of a pair it lands in);
    (c) 128 rows spread over the matrix agree with the reference's golden (dequantise per group, fp64 product,
    tests/st/runtime/ops/test_matmul_mx.py:119-131) to fp32 accumulation error."""
    import bench
    from oracle import matmul_mx as omx
    from pypto_b200 import ops
    m, n, k = bench.MX["m"], bench.MX["n"], bench.MX["k"]
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(11)
    a = (torch.randn(m, k, device=dev, generator=gen) * 2).to(torch.float8_e4m3fn)
    b_t = (torch.randn(n, k, device=dev, generator=gen) * 2).to(torch.float8_e4m3fn)
    sa = torch.randint(120, 134, (m, k // 32), device=dev, generator=gen).to(torch.uint8)
    sb = torch.randint(120, 134, (k // 32, n), device=dev, generator=gen).to(torch.uint8)
    out = ops.matmul_mx(a, sa, b_t, sb)
    torch.cuda.synchronize()
    ops.check_device_status()
    assert torch.isfinite(out).all()
    doubled = ops.matmul_mx(a, sa + 1, b_t, sb)
    assert torch.equal(doubled, out * 2)
    del doubled
    perm = torch.randperm(m, device=dev, generator=gen)
    permuted = ops.matmul_mx(a.view(torch.uint8)[perm].view(torch.float8_e4m3fn), sa[perm], b_t, sb)
    assert torch.equal(permuted, out[perm])
    del permuted
    rows = torch.arange(0, m, m // 128, device=dev)[:128] + 37           # rows of both CTAs of many pairs
    exp = omx.matmul_mx(a[rows].cpu(), sa[rows].cpu(),
                        b_t.cpu().view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn), sb.cpu())
    rel = ((out[rows].cpu() - exp).norm() / exp.norm()).item()
    assert rel < 1e-5, rel
