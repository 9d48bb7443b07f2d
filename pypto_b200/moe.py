"""Mixture-of-experts layer: sigmoid gate + top-k routing, dispatch, grouped FP8 expert FFN,
combine; expert-parallel over ranks with one payload exchange each way over NCCL.

The data movement follows the reference's expert-parallel pattern (dispatch_step ->
local_expert_step -> combine_step, tests/st/distributed/test_l3_ep_dispatch_combine.py:104-402):
destination rank = expert id // L, rows inside a (rank, local expert) bucket ordered by source
rank then (t, k), route id t*TOPK + k, combine = fp32 sum over k of the returned bf16 rows.
The reference moves rows with one-sided puts into peer windows; here a step is

    plan kernels -> counts all-to-all -> ONE all-to-all-v of packed payload rows ->
    receive-plan kernel -> unpack -> experts -> ONE all-to-all-v of result rows -> combine

with exact row counts only.  Everything that touches data is a kernel of the library or an NCCL
call issued through the C ABI (``pypto_b200.comm``); torch supplies buffers and streams.

Launch model: one process per GPU.  With ``comm=None`` the layer runs on one GPU with all experts
local and no collective.
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


def split_sizes(offsets, recv_counts, world: int, local_experts: int):
    """Host arithmetic of the exchange: ``offsets`` [world*L + 1] is the exclusive scan of this rank's
    per-global-expert route counts, ``recv_counts`` [world, L] what every source sends to this rank's experts.
    Returns (rows sent to each rank, rows received from each rank)."""
    L = local_experts
    send = [int(offsets[(d + 1) * L]) - int(offsets[d * L]) for d in range(world)]
    recv = [int(sum(int(v) for v in recv_counts[s * L:(s + 1) * L])) for s in range(world)]
    return send, recv


class Dispatched:
    """What one ``EpExchanger.dispatch`` leaves behind: the grouped payload and the plans that bring the
    results back."""
    __slots__ = ("routes", "pos", "route_at", "send_rows", "recv_rows", "rows", "capacity", "counts", "offsets",
                 "arrival_of", "grouped_of", "parts", "phases")


class EpExchanger:
    """Dispatch and return of routed rows for one rank.

    ``dispatch`` sorts this rank's routes by global expert, ships every route's payload (any number of row
    arrays, packed side by side into one row) to the rank that owns the expert, and groups what arrives by
    local expert in the reference's slot order.  ``give_back`` returns one result row per route to the
    senders in their sorted order, ready for ``ops.moe_combine`` with ``Dispatched.pos``."""

    def __init__(self, comm, local_experts: int):
        self.comm = comm
        self.world = comm.world if comm is not None else 1
        self.local_experts = local_experts
        self._pinned = None

    def _host_ints(self, n: int) -> torch.Tensor:
        if self._pinned is None or self._pinned.numel() < n:
            self._pinned = torch.empty(max(n, 1024), dtype=torch.int32).pin_memory()
        return self._pinned

    def dispatch(self, expert_ids: torch.Tensor, sources: list, slot_stride: int = 0, timer=None) -> Dispatched:
        """expert_ids int32 [routes] (global ids).  ``sources``: list of (tensor [n_src, ...], div) -- route r
        ships row r // div of the tensor (div = TOPK for per-token arrays, 1 for per-route arrays); a tensor
        may be a strided column view ``t[:, :c]`` of a contiguous 2-D tensor."""
        dev = expert_ids.device
        W, L = self.world, self.local_experts
        routes = expert_ids.numel()
        d = Dispatched()
        d.routes = routes
        counts, offsets, d.pos, d.route_at = ops.moe_dispatch_plan(expert_ids, W * L)
        if timer:
            timer("plan")
        geom, payload_bytes = [], 0
        for t, div in sources:
            rb = t.shape[1] * t.element_size() if t.dim() > 1 else t.element_size()
            stride = t.stride(0) * t.element_size()
            geom.append((t, div, rb, stride, payload_bytes))
            payload_bytes += (rb + 15) // 16 * 16
        if W == 1 and slot_stride == 0:
            # all experts are local and the grouped layout is dense: the sorted rows are the grouped rows
            d.rows = d.capacity = routes
            d.send_rows = d.recv_rows = [routes]
            d.counts, d.offsets, d.arrival_of, d.grouped_of = counts, offsets, None, None
            d.parts = []
            for t, div, rb, stride, _o in geom:
                out = torch.empty((routes,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev)
                ops.move_rows([(t.data_ptr(), stride, out.data_ptr(), rb, rb)], d.route_at, div, routes, t.shape[0])
                d.parts.append(out)
            if timer:
                timer("pack")
            return d
        send_counts = counts.view(W, L)
        if W == 1:
            recv_counts = send_counts
        else:
            recv_counts = torch.empty_like(send_counts)
            self.comm.all_to_all(send_counts, recv_counts)
        host = self._host_ints(2 * W * L + 1)
        host[:W * L + 1].copy_(offsets, non_blocking=True)
        host[W * L + 1:2 * W * L + 1].copy_(recv_counts.reshape(-1), non_blocking=True)
        ready = torch.cuda.Event()
        ready.record()
        # packing does not depend on the host: it runs while the host waits for the counts
        send_buf = torch.empty(max(routes, 1), payload_bytes, dtype=torch.uint8, device=dev)
        by_div: dict = {}
        for g in geom:
            by_div.setdefault(g[1], []).append(g)
        for div, group in by_div.items():       # arrays that share a divisor move in one launch (three at most)
            for i in range(0, len(group), 3):
                chunk = group[i:i + 3]
                ops.move_rows([(t.data_ptr(), stride, send_buf.data_ptr() + off, payload_bytes, rb)
                               for t, _d, rb, stride, off in chunk], d.route_at, div, routes,
                              min(t.shape[0] for t, *_ in chunk))
        if timer:
            timer("pack")
        ready.synchronize()                                  # the one host wait of a step
        h = host[:2 * W * L + 1].tolist()
        d.send_rows, d.recv_rows = split_sizes(h[:W * L + 1], h[W * L + 1:], W, L)
        arrived = sum(d.recv_rows)
        if W == 1:
            recv_buf = send_buf
        else:
            recv_buf = torch.empty(max(arrived, 1), payload_bytes, dtype=torch.uint8, device=dev)
            self.comm.all_to_all_v(send_buf, d.send_rows, recv_buf, d.recv_rows)
        if timer:
            timer("exchange_out")
        d.capacity = L * slot_stride if slot_stride else arrived
        d.rows = arrived
        d.counts, d.offsets, d.arrival_of, d.grouped_of = ops.moe_recv_plan(recv_counts, max(d.capacity, arrived),
                                                                             slot_stride)
        d.parts = [torch.empty((d.capacity,) + tuple(t.shape[1:]), dtype=t.dtype, device=dev) for t, *_ in geom]
        for i in range(0, len(geom), 3):
            ops.move_rows([(recv_buf.data_ptr() + off, payload_bytes, out.data_ptr(), rb, rb)
                           for (_t, _d, rb, _s, off), out in zip(geom[i:i + 3], d.parts[i:i + 3])],
                          d.arrival_of, 1, d.capacity, arrived)
        if timer:
            timer("unpack")
        return d

    def give_back(self, d: Dispatched, y_grouped: torch.Tensor, timer=None, in_arrival_order: bool = False) -> torch.Tensor:
        """y_grouped [capacity, H] (one result row per grouped row, or already one per arrival row with
        ``in_arrival_order``) -> [routes, H] in this rank's sorted route order (row ``Dispatched.pos[t*K + k]``
        belongs to route (t, k))."""
        if d.grouped_of is None:
            return y_grouped
        shape = tuple(y_grouped.shape[1:])
        if in_arrival_order and d.rows:
            y_arrival = y_grouped
        elif d.rows:
            (y_arrival,) = ops.gather_rows([y_grouped], d.grouped_of, div=1, rows=d.rows)
        else:
            y_arrival = torch.zeros((1,) + shape, dtype=y_grouped.dtype, device=y_grouped.device)
        if self.world == 1:
            return y_arrival
        back = torch.empty((max(d.routes, 1),) + shape, dtype=y_grouped.dtype, device=y_grouped.device)
        self.comm.all_to_all_v(y_arrival, d.recv_rows, back, d.send_rows)
        if timer:
            timer("exchange_back")
        return back


class PhaseTimer:
    """CUDA-event stopwatch over the phases of a step (``MoELayer.forward(..., timer=PhaseTimer())``)."""

    def __init__(self):
        self.marks = []
        self("start")

    def __call__(self, name: str) -> None:
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.marks.append((name, e))

    def result(self) -> dict:
        torch.cuda.synchronize()
        out: dict = {}
        for (_n0, e0), (n1, e1) in zip(self.marks, self.marks[1:]):
            out[n1] = out.get(n1, 0.0) + e0.elapsed_time(e1)
        return out


class MoELayer:
    def __init__(self, gate_w: torch.Tensor, bias: torch.Tensor, routed: dict, shared: dict | None, topk: int,
                 n_experts: int | None = None, comm=None):
        """gate_w bf16 [H, E_global]; bias fp32 [E_global]; ``routed``: this rank's experts
        (stacked, ``x @ W`` layout, see pack_expert_weights); ``shared``: one expert (no leading
        dim) or None.  With a communicator, global expert e lives on rank e // L."""
        self._setup(comm, routed["wg"].shape[0], n_experts, topk)
        self.gate_packed = ops.pack_weight(gate_w.contiguous())
        self.bias = bias.float().contiguous()
        self.routed = pack_expert_weights(routed)
        self.shared = pack_expert_weights({k: v.unsqueeze(0) for k, v in shared.items()}) if shared else None
        self.hidden = gate_w.shape[0]

    def _setup(self, comm, local_experts, n_experts, topk):
        self.comm = comm
        self.world = comm.world if comm is not None else 1
        self.rank = comm.rank if comm is not None else 0
        self.local_experts = local_experts
        self.n_experts = n_experts or self.local_experts * self.world
        if self.n_experts != self.local_experts * self.world:
            raise ValueError("experts must be split evenly over the ranks")
        self.topk = topk
        self.exchanger = EpExchanger(comm, local_experts)

    @classmethod
    def from_packed(cls, gate_packed: torch.Tensor, bias: torch.Tensor, routed: dict, shared: dict | None,
                    topk: int, n_experts: int | None = None, comm=None) -> "MoELayer":
        """Build from weights already in the kernels' layout (gate packed [E, H] bf16; expert
        dicts with w_gu / s_gu / w_d / s_d as produced by pack_expert_weights)."""
        self = cls.__new__(cls)
        self._setup(comm, routed["w_gu"].shape[0], n_experts, topk)
        self.gate_packed, self.bias = gate_packed, bias.float().contiguous()
        self.routed, self.shared, self.hidden = routed, shared, gate_packed.shape[1]
        return self

    def route(self, x: torch.Tensor):
        logits = ops.linear(x, self.gate_packed)
        return ops.moe_topk(logits, self.bias, self.topk, is_logits=True)

    def _experts(self, weights: dict, xq, xs, offsets, route_w, out_rows=None):
        act = ops.moe_expert_gemm(True, weights["w_gu"], weights["s_gu"], xq, xs, offsets)
        act_q, act_s = ops.quantize_rows(act)
        return ops.moe_expert_gemm(False, weights["w_d"], weights["s_d"], act_q, act_s, offsets, route_w, out_rows)

    def forward(self, x: torch.Tensor, routing=None, timer=None):
        """x bf16 [T, H] (this rank's tokens) -> (y bf16 [T, H], idx int32 [T, k], w fp32 [T, k])."""
        t, _h = x.shape
        k = self.topk
        idx, w = routing if routing is not None else self.route(x)
        xq, xs = ops.quantize_rows(x)
        if timer:
            timer("route_quantize")
        # The shared expert depends on nothing but the quantised tokens: run it on a side stream so
        # that it fills the GPU while the host waits for the row counts of the exchange.
        shared_out, side = None, None
        if self.shared is not None:
            main = torch.cuda.current_stream()
            side = self._side_stream(x.device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                shared_out = self._experts(self.shared, xq, xs, self._whole(t, x.device), None)
        d = self.exchanger.dispatch(idx.reshape(-1), [(xq, k), (xs, k), (w.reshape(-1, 1), 1)], timer=timer)
        xq_g, xs_g, w_g = d.parts
        # with ranks to return to, the down projection writes its rows straight in arrival order (no regrouping pass)
        in_arrival_order = d.grouped_of is not None
        if d.capacity > 0:
            y_g = self._experts(self.routed, xq_g, xs_g, d.offsets, w_g.reshape(-1),
                                d.arrival_of if in_arrival_order else None)
        else:
            y_g = torch.empty(0, self.hidden, dtype=torch.bfloat16, device=x.device)
        if timer:
            timer("experts")
        y_rows = self.exchanger.give_back(d, y_g, timer=timer, in_arrival_order=in_arrival_order)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
            for tns in (xq, xs, shared_out):
                tns.record_stream(side)
        y = ops.moe_combine(y_rows, d.pos, shared_out, t, k)
        if timer:
            timer("combine")
        return y, idx, w

    _streams: dict = {}
    _whole_cache: dict = {}

    def _whole(self, t: int, dev) -> torch.Tensor:
        """offsets [0, t] of a one-expert group that spans all tokens (the shared expert)."""
        key = (dev.index, t)
        o = MoELayer._whole_cache.get(key)
        if o is None:
            o = MoELayer._whole_cache[key] = torch.tensor([0, t], dtype=torch.int32, device=dev)
        return o

    def _side_stream(self, dev):
        key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
        s = MoELayer._streams.get(key)
        if s is None:
            s = MoELayer._streams[key] = torch.cuda.Stream(device=dev)
        return s
