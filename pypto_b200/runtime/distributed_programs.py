"""Rank-side bodies of level-3 (multi-GPU) programs: what one GPU does for its shard of a HOST-level
orchestration.  A HOST orchestrator of the reference loops ``for r in pl.range(pld.world_size())`` and
dispatches a chip-level function with the r-th slice of every rank-stacked tensor
(tests/st/distributed/test_l3_ep_dispatch_combine.py:455-512); here every rank is one process that runs the
fused equivalent of that chip-level function, with cross-rank movement through ``pypto_b200.comm``.

A program whose HOST entry is not in the table has no multi-GPU kernel here and ``lookup`` raises.
"""

from __future__ import annotations

import torch


class DistributedFusedOp:
    def matches(self, entry) -> bool:
        raise NotImplementedError

    def validate(self, world: int, host: dict) -> None:
        """Shape / dtype checks on the rank-stacked host tensors, before anything is launched."""

    def run_rank(self, state: dict, rank: int, world: int, comm, t: dict) -> None:
        """``t`` maps parameter names to this rank's CUDA tensors (the leading rank dimension removed);
        outputs are written in place.  ``state`` persists across dispatches of one worker."""
        raise NotImplementedError


class EpDispatchCombineOp(DistributedFusedOp):
    """``host_orch(indices, x_norms, w_padded, idx_padded, recv_x_outs, recv_w_outs, recv_idx_outs,
    recv_count_outs, recv_ys, routed_ys)`` of the reference's expert-parallel program
    (test_l3_ep_dispatch_combine.py:455-512): per rank dispatch_step -> local_expert_step -> combine_step
    (:104-402).  Rank-stacked shapes: indices [N, T, TOPK] int32; x_norms [N, T, D] bf16; w_padded
    [N, T*TOPK, W_PAD] fp32 (weight in column 0); idx_padded [N, T*TOPK, IDX_PAD] int32 (route id in column
    0); recv_x_outs / recv_ys [N, L*R, D] bf16; recv_w_outs fp32 / recv_idx_outs int32 [N, L, R];
    recv_count_outs [N, L, 1] int32; routed_ys [N, T, D] fp32.  Unused receive slots are left zero."""

    names = ("indices", "x_norms", "w_padded", "idx_padded", "recv_x_outs", "recv_w_outs", "recv_idx_outs",
             "recv_count_outs", "recv_ys", "routed_ys")

    def matches(self, entry) -> bool:
        return tuple(p.name for p in entry.params) == self.names

    def validate(self, world, host):
        ind, x, w, idx = (host[n] for n in self.names[:4])
        if ind.dim() != 3 or x.dim() != 3 or ind.shape[0] != world or x.shape[0] != world:
            raise ValueError(f"indices / x_norms must be rank-stacked with a leading dimension of {world}")
        n, t, k = ind.shape
        d = x.shape[2]
        if ind.dtype != torch.int32 or x.dtype != torch.bfloat16 or w.dtype != torch.float32 or idx.dtype != torch.int32:
            raise TypeError("indices int32, x_norms bf16, w_padded fp32, idx_padded int32 expected")
        if x.shape[1] != t or w.shape[:2] != (n, t * k) or idx.shape[:2] != (n, t * k):
            raise ValueError("x_norms / w_padded / idx_padded do not match indices [N, T, TOPK]")
        rw = host["recv_w_outs"]
        if rw.dim() != 3 or rw.shape[0] != n:
            raise ValueError("recv_w_outs must be [N, L, R]")
        L, R = rw.shape[1:]
        want = {"recv_x_outs": (n, L * R, d), "recv_idx_outs": (n, L, R), "recv_count_outs": (n, L, 1),
                "recv_ys": (n, L * R, d), "routed_ys": (n, t, d)}
        for name, shape in want.items():
            if tuple(host[name].shape) != shape:
                raise ValueError(f"{name} has shape {tuple(host[name].shape)}, expected {shape}")
        if d % 8:
            raise ValueError("the row width D must be a multiple of 8")
        if int(ind.min()) < 0 or int(ind.max()) >= n * L:
            raise ValueError(f"expert ids must lie in [0, {n * L})")

    def run_rank(self, state, rank, world, comm, t):
        from .. import ops
        from ..moe import EpExchanger
        ind, x = t["indices"], t["x_norms"]
        tokens, topk = ind.shape
        L, R = t["recv_w_outs"].shape
        ex = state.get("exchanger")
        if ex is None or ex.local_experts != L:
            ex = state["exchanger"] = EpExchanger(comm, L)
        d = ex.dispatch(ind.reshape(-1), [(x, topk), (t["w_padded"][:, :1], 1), (t["idx_padded"][:, :1], 1)],
                        slot_stride=R)
        recv_x, recv_w, recv_idx = d.parts
        t["recv_x_outs"].copy_(recv_x)
        t["recv_w_outs"].view(-1).copy_(recv_w.view(-1))
        t["recv_idx_outs"].view(-1).copy_(recv_idx.view(-1))
        t["recv_count_outs"].view(-1).copy_(d.counts)
        ops.scale_rows(recv_x, recv_w.view(-1), 1, d.counts, R, out=t["recv_ys"])       # local_expert_step
        rows = ex.give_back(d, t["recv_ys"])
        _y, y32 = ops.moe_combine(rows, d.pos, None, tokens, topk, want_f32=True)      # combine_step
        t["routed_ys"].copy_(y32)


REGISTRY: list[DistributedFusedOp] = [EpDispatchCombineOp()]


def lookup(entry) -> DistributedFusedOp:
    for op in REGISTRY:
        if op.matches(entry):
            return op
    sig = ", ".join(p.name for p in entry.params)
    raise NotImplementedError(f"no multi-GPU kernel registered for host entry '{entry.name}({sig})'; "
                              "this backend runs fused operators only and has no CPU fallback")
