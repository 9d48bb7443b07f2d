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
call issued through the C ABI; ``MoELayer.forward`` is ONE call into the runtime's layer object
(``pto_moe_layer_forward``), which issues the whole step.  ``EpExchanger`` is the same exchange as a
building block with any payload, for programs that dispatch other data (the reference's own
expert-parallel test program does).  torch supplies buffers and streams.

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

    def ingest(self, phases: dict) -> None:
        """Phase times measured inside the runtime's own forward call (``pto_moe_layer_forward``)."""
        self.given = dict(phases)

    def result(self) -> dict:
        if getattr(self, "given", None) is not None:
            return dict(self.given)
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
        self._handle, self._handle_tokens = None, 0

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

    PHASES = ("route_quantize", "plan", "pack", "exchange_out", "unpack", "experts", "exchange_back", "combine")

    def _native(self, tokens: int, dev):
        """The runtime's layer object (``pto_moe_layer``), created on first use and again if a call brings more
        tokens than it was sized for.  With a communicator, creation is collective like the forward call."""
        import ctypes as C

        from . import _lib
        h = getattr(self, "_handle", None)
        if h is not None and self._handle_tokens >= tokens:
            return h
        lib = _lib.load()
        if h is not None:
            _lib.check(lib.pto_moe_layer_destroy(h))
            self._handle = None
        d = _lib.MoeLayerDesc()
        d.hidden, d.inter = self.hidden, self.routed["w_d"].shape[2]
        d.n_experts, d.topk, d.max_tokens = self.n_experts, self.topk, tokens
        d.gate_packed, d.bias = self.gate_packed.data_ptr(), self.bias.data_ptr()
        for k in ("w_gu", "s_gu", "w_d", "s_d"):
            setattr(d, k, self.routed[k].data_ptr())
            setattr(d, "sh_" + k, self.shared[k].data_ptr() if self.shared is not None else None)
        d.comm = self.comm._h if self.comm is not None else None
        out = C.c_void_p()
        with torch.cuda.device(dev):
            _lib.check(lib.pto_moe_layer_create(C.byref(d), C.byref(out)))
        self._handle, self._handle_tokens = out, tokens
        return out

    def close(self) -> None:
        h = getattr(self, "_handle", None)
        if h is not None:
            from . import _lib
            self._handle = None
            _lib.check(_lib.load().pto_moe_layer_destroy(h))

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def peer_exchange(self) -> bool:
        """True when the experts' results return through peer memory (the library's own kernel and flags) instead of
        an all-to-all: every rank could map every other rank's buffers when the layer was created."""
        return self.peer_exchange_level > 0

    @property
    def peer_exchange_level(self) -> int:
        """0: both exchanges are collectives; 1: results return through peer memory; 2: rows go out that way too
        (``PTO_EP_PEER=2`` on every rank)."""
        from . import _lib
        h = getattr(self, "_handle", None)
        return int(_lib.load().pto_moe_layer_peer_exchange(h)) if h is not None else 0

    def status(self) -> tuple:
        """The layer's device error word (code, site, CTA, detail); reading clears it."""
        import ctypes as C

        from . import _lib
        h = getattr(self, "_handle", None)
        if h is None:
            return (0, 0, 0, 0)
        words = (C.c_int32 * 4)()
        dev = self.gate_packed.device
        with torch.cuda.device(dev):
            _lib.check(_lib.load().pto_moe_layer_status(h, words, torch.cuda.current_stream(dev).cuda_stream))
        return tuple(words)

    def forward(self, x: torch.Tensor, routing=None, timer=None):
        """x bf16 [T, H] (this rank's tokens) -> (y bf16 [T, H], idx int32 [T, k], w fp32 [T, k]).  One call into
        the runtime (``pto_moe_layer_forward``) issues every kernel and both exchanges of the step."""
        import ctypes as C

        from . import _lib
        if not x.is_cuda or x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != self.hidden or not x.is_contiguous():
            raise ValueError("MoELayer.forward: x must be a contiguous CUDA bf16 [tokens, hidden] tensor")
        t, dev = x.shape[0], x.device
        h = self._native(t, dev)
        y = torch.empty_like(x)
        if routing is not None:
            idx, w = routing
            if idx.dtype != torch.int32 or w.dtype != torch.float32 or tuple(idx.shape) != (t, self.topk) \
                    or tuple(w.shape) != (t, self.topk) or not idx.is_contiguous() or not w.is_contiguous():
                raise ValueError("MoELayer.forward: routing must be (int32 [T, k], fp32 [T, k]) contiguous tensors")
            args = (idx.data_ptr(), w.data_ptr(), y.data_ptr(), None, None)
        else:
            idx = torch.empty(t, self.topk, dtype=torch.int32, device=dev)
            w = torch.empty(t, self.topk, dtype=torch.float32, device=dev)
            args = (None, None, y.data_ptr(), idx.data_ptr(), w.data_ptr())
        phases = (C.c_float * 8)() if timer is not None else None
        with torch.cuda.device(dev):
            _lib.check(_lib.load().pto_moe_layer_forward(h, x.data_ptr(), t, *args, phases,
                                                         torch.cuda.current_stream(dev).cuda_stream))
        if timer is not None:
            timer.ingest(dict(zip(self.PHASES, list(phases))))
        return y, idx, w

