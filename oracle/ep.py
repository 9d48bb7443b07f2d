"""Oracle for expert-parallel dispatch and combine (test infrastructure, not product code).

Restates tests/st/distributed/test_l3_ep_dispatch_combine.py:
  _compute_golden_recv   :562-614  (dispatch: counts, slots, rows, weights, route ids)
  _compute_golden_routed :617-629  (combine with the stand-in expert bf16(fp32(x) * w))
Device-side protocol it mirrors: dispatch_step :104-299, combine_step :337-402.

Rule: destination rank = eid // L, local expert = eid % L; within the bucket
(dst, local expert) rows are ordered by source rank, then by (t, k)
lexicographically; the route id carried with a row is t * TOPK + k.
All outputs are integers or copied rows: compared bit-exactly.
"""

from __future__ import annotations

import torch


def dispatch(x, indices, weights, n_local, recv_max):
    """x [N, T, D] bf16, indices [N, T, K] int, weights [N, T, K] fp32.
    Returns recv_x [N, L, R, D], recv_w [N, L, R], recv_idx [N, L, R] int32,
    recv_src [N, L, R] int32 (source rank; not in the reference outputs, used by
    the combine), count [N, L] int32."""
    n, t, d = x.shape
    k = indices.shape[2]
    L, R = n_local, recv_max
    recv_x = torch.zeros(n, L, R, d, dtype=x.dtype)
    recv_w = torch.zeros(n, L, R, dtype=torch.float32)
    recv_idx = torch.zeros(n, L, R, dtype=torch.int32)
    recv_src = torch.zeros(n, L, R, dtype=torch.int32)
    count = torch.zeros(n, L, dtype=torch.int32)
    flat = indices.reshape(n, t * k).long()
    for dst in range(n):
        fill = [0] * L
        for src in range(n):
            routes = torch.nonzero(flat[src] // L == dst).flatten().tolist()
            for r in routes:  # ascending r = (t, k) lexicographic order
                e = int(flat[src, r]) % L
                slot = fill[e]
                fill[e] += 1
                assert slot < R, "receive bucket overflow"
                recv_x[dst, e, slot] = x[src, r // k]
                recv_w[dst, e, slot] = weights[src, r // k, r % k]
                recv_idx[dst, e, slot] = r
                recv_src[dst, e, slot] = src
        count[dst] = torch.tensor(fill, dtype=torch.int32)
    return recv_x, recv_w, recv_idx, recv_src, count


def standin_expert(recv_x, recv_w):
    """local_expert_step :309-327: y = bf16(fp32(x) * w)."""
    return (recv_x.float() * recv_w.unsqueeze(-1)).bfloat16()


def combine(recv_y, recv_idx, recv_src, count, n_tokens, topk):
    """combine_step :337-402: each expert-output row returns to slot t*K+k of its
    source rank; y[t] = sum_k fp32(row) in k order.  Returns fp32 [N, T, D]."""
    n, L, R, d = recv_y.shape
    routed = torch.zeros(n, n_tokens * topk, d, dtype=recv_y.dtype)
    for dst in range(n):
        for e in range(L):
            for s in range(int(count[dst, e])):
                routed[int(recv_src[dst, e, s]), int(recv_idx[dst, e, s])] = recv_y[dst, e, s]
    y = torch.zeros(n, n_tokens, d, dtype=torch.float32)
    rk = routed.reshape(n, n_tokens, topk, d)
    for k in range(topk):
        y += rk[:, :, k].float()
    return y
