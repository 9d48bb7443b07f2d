"""Mixture-of-experts layer: sigmoid gate + top-k routing, dispatch, grouped FP8 expert FFN,
combine; expert-parallel over ranks with NCCL all-to-all for dispatch and combine.

The data movement follows the reference's expert-parallel pattern (dispatch_step ->
local_expert_step -> combine_step, tests/st/distributed/test_l3_ep_dispatch_combine.py:104-402):
destination rank = expert id // L, rows inside a (rank, local expert) bucket ordered by source
rank then (t, k), route id t*TOPK + k, combine = fp32 sum over k of the returned bf16 rows.
The reference moves rows with one-sided puts into peer windows; here each exchange is one
``all_to_all_single`` (counts, then rows) over NVLink, exact row counts only.

Launch model: one process per GPU (``torch.distributed``); with ``group=None`` the layer runs
on one GPU with all experts local and no collective.
"""

from __future__ import annotations

import torch

from . import ops


def pack_expert_weights(stacked: dict) -> dict:
    """Expert weights in the ``x @ W`` layout (wg/wu [E, H, I], wd [E, I, H] e4m3 with scales
    [E, K/128, N/128]) -> the GEMM's K-major layout: w_gu [E, 2I, H] (gate rows, then up rows)
    with s_gu [E, 2I/128, H/128]; w_d [E, H, I] with s_d [E, H/128, I/128].  One-time."""
    def kt(w):   # [E, K, N] -> [E, N, K]
        return w.view(torch.uint8).transpose(1, 2).contiguous().view(ops.FP8)
    w_gu = torch.cat([kt(stacked["wg"]), kt(stacked["wu"])], dim=1).contiguous()
    s_gu = torch.cat([stacked["sg"].transpose(1, 2), stacked["su"].transpose(1, 2)], dim=1).contiguous()
    return dict(w_gu=w_gu, s_gu=s_gu, w_d=kt(stacked["wd"]), s_d=stacked["sd"].transpose(1, 2).contiguous())


def exchange_rows(buf: torch.Tensor, out_rows: int, out_split: list, in_split: list, group) -> torch.Tensor:
    """all-to-all-v of rows: this rank sends in_split[d] consecutive rows of ``buf`` to rank d
    and receives out_split[s] rows from rank s, in source-rank order.  Exact row counts, unlike
    the reference's all_to_all_v which always ships a full max_recv block
    (python/pypto/runtime/builtins/collectives/all_to_all_v/templates/kernel.cpp.in:118-127)."""
    import torch.distributed as dist
    out = torch.empty((out_rows,) + tuple(buf.shape[1:]), dtype=buf.dtype, device=buf.device)
    fp8 = getattr(torch, "float8_e4m3fn", None)
    flat_in = buf.view(torch.uint8) if buf.dtype == fp8 else buf
    flat_out = out.view(torch.uint8) if out.dtype == fp8 else out
    dist.all_to_all_single(flat_out, flat_in, out_split, in_split, group=group)
    return out


def exchange_counts(send_counts: torch.Tensor, group) -> torch.Tensor:
    """send_counts int32 [world, L] (rows for each destination's local experts) ->
    recv_counts [world, L] (rows arriving from each source for my local experts)."""
    import torch.distributed as dist
    recv = torch.empty_like(send_counts)
    dist.all_to_all_single(recv, send_counts.contiguous(), group=group)
    return recv


def arrival_expert_ids(recv_counts: torch.Tensor) -> torch.Tensor:
    """Local expert id of every arriving row: rows arrive source-major, and inside a source
    ordered by local expert (recv_counts[s][e] rows each)."""
    world, L = recv_counts.shape
    eid = torch.arange(L, device=recv_counts.device, dtype=torch.int32).repeat(world)
    return torch.repeat_interleave(eid, recv_counts.reshape(-1).long())


class MoELayer:
    def __init__(self, gate_w: torch.Tensor, bias: torch.Tensor, routed: dict, shared: dict | None, topk: int,
                 n_experts: int | None = None, group=None):
        """gate_w bf16 [H, E_global]; bias fp32 [E_global]; ``routed``: this rank's experts
        (stacked, ``x @ W`` layout, see pack_expert_weights); ``shared``: one expert (no leading
        dim) or None.  With a process group, global expert e lives on rank e // L."""
        import torch.distributed as dist
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.local_experts = routed["wg"].shape[0]
        self.n_experts = n_experts or self.local_experts * self.world
        assert self.n_experts == self.local_experts * self.world
        self.topk = topk
        self.gate_packed = ops.pack_weight(gate_w.contiguous())
        self.bias = bias.float().contiguous()
        self.routed = pack_expert_weights(routed)
        self.shared = pack_expert_weights({k: v.unsqueeze(0) for k, v in shared.items()}) if shared else None
        self.hidden = gate_w.shape[0]

    @classmethod
    def from_packed(cls, gate_packed: torch.Tensor, bias: torch.Tensor, routed: dict, shared: dict | None,
                    topk: int, n_experts: int | None = None, group=None) -> "MoELayer":
        """Build from weights already in the kernels' layout (gate packed [E, H] bf16; expert
        dicts with w_gu / s_gu / w_d / s_d as produced by pack_expert_weights)."""
        import torch.distributed as dist
        self = cls.__new__(cls)
        self.group = group
        self.world = dist.get_world_size(group) if group is not None else 1
        self.rank = dist.get_rank(group) if group is not None else 0
        self.local_experts = routed["w_gu"].shape[0]
        self.n_experts = n_experts or self.local_experts * self.world
        assert self.n_experts == self.local_experts * self.world
        self.topk, self.gate_packed, self.bias = topk, gate_packed, bias.float().contiguous()
        self.routed, self.shared, self.hidden = routed, shared, gate_packed.shape[1]
        return self

    def route(self, x: torch.Tensor):
        logits = ops.linear(x, self.gate_packed)
        return ops.moe_topk(logits, self.bias, self.topk, is_logits=True)

    def _experts(self, weights: dict, xq, xs, offsets, route_w):
        act = ops.moe_expert_gemm(True, weights["w_gu"], weights["s_gu"], xq, xs, offsets)
        act_q, act_s = ops.quantize_rows(act)
        return ops.moe_expert_gemm(False, weights["w_d"], weights["s_d"], act_q, act_s, offsets, route_w)

    def forward(self, x: torch.Tensor, routing=None):
        """x bf16 [T, H] (this rank's tokens) -> (y bf16 [T, H], idx int32 [T, k], w fp32 [T, k])."""
        t, _h = x.shape
        k = self.topk
        idx, w = routing if routing is not None else self.route(x)
        xq, xs = ops.quantize_rows(x)
        # The shared expert depends on nothing but the quantised tokens: run it on a side stream so
        # that it fills the GPU while the host waits for the row counts of the exchange.
        shared_out, side = None, None
        if self.shared is not None:
            main = torch.cuda.current_stream()
            side = self._side_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                off = torch.tensor([0, t], dtype=torch.int32, device=x.device)
                shared_out = self._experts(self.shared, xq, xs, off, None)
        counts, offsets, pos, route_at = ops.moe_dispatch_plan(idx.reshape(-1), self.n_experts)
        xq_s, xs_s = ops.gather_rows([xq, xs], route_at, div=k)
        (w_s,) = ops.gather_rows([w.reshape(-1, 1)], route_at, div=1)
        if self.world == 1:
            y_rows = self._experts(self.routed, xq_s, xs_s, offsets, w_s)
        else:
            L = self.local_experts
            send_counts = counts.view(self.world, L)
            recv_counts = exchange_counts(send_counts, self.group)
            splits = torch.stack([send_counts.sum(1), recv_counts.sum(1)]).tolist()   # the one host sync
            in_split, out_split = splits     # rows sent to each destination / received from each source
            r2 = sum(out_split)
            xq_r = exchange_rows(xq_s, r2, out_split, in_split, self.group)
            xs_r = exchange_rows(xs_s, r2, out_split, in_split, self.group)
            w_r = exchange_rows(w_s, r2, out_split, in_split, self.group)
            eid_r = arrival_expert_ids(recv_counts)
            _c2, offsets2, pos2, route_at2 = ops.moe_dispatch_plan(eid_r, L)
            xq_g, xs_g, w_g = ops.gather_rows([xq_r, xs_r, w_r], route_at2, div=1)
            y_g = self._experts(self.routed, xq_g, xs_g, offsets2, w_g)
            (y_r,) = ops.gather_rows([y_g], pos2, div=1)          # back to arrival order
            y_rows = exchange_rows(y_r, t * k, in_split, out_split, self.group)   # back to the senders' sorted order
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
            for tns in (xq, xs, shared_out):
                tns.record_stream(side)
        y = ops.moe_combine(y_rows, pos, shared_out, t, k)
        return y, idx, w

    _streams: dict = {}

    def _side_stream(self, dev):
        key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
        s = MoELayer._streams.get(key)
        if s is None:
            s = MoELayer._streams[key] = torch.cuda.Stream(device=dev)
        return s
