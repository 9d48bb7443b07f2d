"""Oracle for MoE routing and the FP8 expert FFN (test infrastructure, not product code).

PARITY UNPINNED.  The reference tree has no MoE model, no top-k operator, no
sigmoid gate and no FP8 format with 128x128 fp32 block scales.  Its nearest
pieces are a descending sort that carries original indices
(tests/st/runtime/ops/test_sort.py:626-632), the dequantise-then-matmul shape of
its MXFP8 golden (tests/st/runtime/ops/test_matmul_mx.py:119-131) and the
expert-parallel dispatch/combine test (tests/st/distributed/
test_l3_ep_dispatch_combine.py, restated in ``oracle.ep``).  This file is the
only definition of:

  gate      logits = fp32(x_bf16) @ fp32(Wgate_bf16); s = sigmoid(logits);
            experts chosen by the top-k of s + bias (ties: lower expert id),
            listed in descending order of s + bias; routing weight of a chosen
            expert = s / sum of the chosen s (the bias only steers selection).
  weights   e4m3 with one fp32 scale per 128x128 block, scale = amax / 448
            (1 where the block is all zero), W ~ fp32(q) * scale[k//128, n//128].
  tokens    e4m3 with one fp32 scale per (token, 128 input channels), same rule.
  GEMM      out[t, n] = sum over 128-wide k blocks of
            (sum_k fp32(xq) * fp32(wq)) * xs[t, kb] * ws[kb, n // 128], fp32.
  expert    gate/up GEMMs -> bf16(silu(g) * u) -> requantise per (token, 128)
            -> down GEMM (fp32).
  layer     y[t] = bf16( sum_k fp32(bf16(w[t,k] * expert_k(x[t]))) +
                         fp32(bf16(shared(x[t]))) ), k in routing order.

``dequant_reference`` gives the looser mathematical target (weights
dequantised, activations left in bf16, fp32 math) against which the fp8 path is
held to a norm-relative 5e-2.
"""

from __future__ import annotations

import torch

FP8_MAX = 448.0
BLK = 128


def _scale(amax):
    return torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))


def quantize_weight_blocks(w: torch.Tensor):
    """w [K, N] float -> (q e4m3 [K, N], scale fp32 [ceil(K/128), ceil(N/128)])."""
    k, n = w.shape
    kb, nb = -(-k // BLK), -(-n // BLK)
    wp = torch.zeros(kb * BLK, nb * BLK, dtype=torch.float32)
    wp[:k, :n] = w.float()
    blocks = wp.reshape(kb, BLK, nb, BLK)
    scale = _scale(blocks.abs().amax(dim=(1, 3)))
    q = (blocks / scale.reshape(kb, 1, nb, 1)).reshape(kb * BLK, nb * BLK)[:k, :n]
    return q.to(torch.float8_e4m3fn), scale


def quantize_rows(x: torch.Tensor):
    """x [T, K] (K % 128 == 0) -> (q e4m3 [T, K], scale fp32 [T, K/128])."""
    t, k = x.shape
    g = x.float().reshape(t, k // BLK, BLK)
    scale = _scale(g.abs().amax(dim=-1))
    q = (g / scale.unsqueeze(-1)).reshape(t, k)
    return q.to(torch.float8_e4m3fn), scale


def dequant_weight(q, scale):
    k, n = q.shape
    s = scale.repeat_interleave(BLK, 0)[:k].repeat_interleave(BLK, 1)[:, :n]
    return q.float() * s


def fp8_gemm(xq, xs, wq, ws):
    """Block-scaled GEMM: per 128-wide k block an exact-product fp32 partial sum,
    scaled by the token scale and the weight-block scale, added in k-block order."""
    t, k = xq.shape
    n = wq.shape[1]
    out = torch.zeros(t, n, dtype=torch.float32)
    col_scale_idx = torch.arange(n) // BLK
    xf, wf = xq.float(), wq.float()
    for kb in range(k // BLK):
        part = xf[:, kb * BLK : (kb + 1) * BLK] @ wf[kb * BLK : (kb + 1) * BLK]
        out += part * xs[:, kb : kb + 1] * ws[kb][col_scale_idx].unsqueeze(0)
    return out


def expert_ffn(xq, xs, ex):
    """ex = dict(wg, sg, wu, su, wd, sd) for one expert.  Returns fp32 [n, H]."""
    gate = fp8_gemm(xq, xs, ex["wg"], ex["sg"])
    up = fp8_gemm(xq, xs, ex["wu"], ex["su"])
    act = (gate * torch.sigmoid(gate) * up).bfloat16()
    aq, as_ = quantize_rows(act)
    return fp8_gemm(aq, as_, ex["wd"], ex["sd"])


def gate_scores(x_bf16, gate_w_bf16):
    """fp32 sigmoid scores [T, E]."""
    return torch.sigmoid(torch.matmul(x_bf16.float(), gate_w_bf16.float()))


def topk_from_scores(scores, bias, topk):
    """(indices int32 [T, k], weights fp32 [T, k]) from fp32 scores [T, E].
    Selection on scores + bias, descending, ties to the lower expert id
    (a stable descending sort keeps the lower index first)."""
    sel = scores + bias.reshape(1, -1)
    order = torch.sort(sel, dim=-1, descending=True, stable=True)[1][:, :topk]
    picked = torch.gather(scores, 1, order)
    weights = picked / picked.sum(dim=-1, keepdim=True)
    return order.to(torch.int32), weights


def gate_topk(x_bf16, gate_w_bf16, bias, topk):
    return topk_from_scores(gate_scores(x_bf16, gate_w_bf16), bias, topk)


def sort_desc_with_index(src):
    """Descending sort returning (values, original indices), the contract of the
    reference's sort32 + mrgsort + gather chain (test_sort.py:626-632)."""
    vals, order = torch.sort(src, dim=-1, descending=True, stable=True)
    return vals, order.to(torch.int32)


def expert_slice(stacked: dict, e: int) -> dict:
    return {k: v[e] for k, v in stacked.items()}


def moe_layer(x_bf16, gate_w, bias, routed: dict, shared: dict | None, topk: int):
    """Whole layer on one rank.  ``routed`` holds stacked tensors
    wg/wu [E, H, I] e4m3, sg/su [E, H/128, I/128], wd [E, I, H], sd [E, I/128, H/128];
    ``shared`` holds the same keys for one expert (no leading dim) or None.
    Returns (y bf16 [T, H], indices int32 [T, k], weights fp32 [T, k])."""
    t, h = x_bf16.shape
    idx, w = gate_topk(x_bf16, gate_w, bias, topk)
    xq, xs = quantize_rows(x_bf16)
    contrib = torch.zeros(t, topk, h, dtype=torch.float32)
    n_exp = routed["wg"].shape[0]
    for e in range(n_exp):
        tok, kk = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        o = expert_ffn(xq[tok], xs[tok], expert_slice(routed, e))
        contrib[tok, kk] = (o * w[tok, kk].unsqueeze(-1)).bfloat16().float()
    y = torch.zeros(t, h, dtype=torch.float32)
    for k in range(topk):  # fp32 sum in routing order, as combine_step does
        y += contrib[:, k]
    if shared is not None:
        y += expert_ffn(xq, xs, shared).bfloat16().float()
    return y.bfloat16(), idx, w


def dequant_reference(x_bf16, idx, w, routed, shared):
    """Looser mathematical target: dequantised weights, bf16 activations, fp32."""
    t, h = x_bf16.shape
    xf = x_bf16.float()
    y = torch.zeros(t, h, dtype=torch.float32)

    def ffn(xx, ex):
        g = xx @ dequant_weight(ex["wg"], ex["sg"])
        u = xx @ dequant_weight(ex["wu"], ex["su"])
        return (g * torch.sigmoid(g) * u) @ dequant_weight(ex["wd"], ex["sd"])

    for e in range(routed["wg"].shape[0]):
        tok, kk = torch.nonzero(idx == e, as_tuple=True)
        if tok.numel():
            y.index_put_((tok,), ffn(xf[tok], expert_slice(routed, e)) * w[tok, kk].unsqueeze(-1),
                         accumulate=True)
    if shared is not None:
        y += ffn(xf, shared)
    return y


def moe_flops(t, h, inter, n_exp, topk, shared=True):
    routed = t * topk * 6 * h * inter
    sh = t * 6 * h * inter if shared else 0
    return routed + sh + 2 * t * h * n_exp
