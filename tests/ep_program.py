"""The reference's level-3 expert-parallel program, signatures only (bodies are DSL text that this backend
never executes): tests/st/distributed/test_l3_ep_dispatch_combine.py:86-512 at the sizes of the committed
fixtures.  Shared by the CPU and GPU tests of the distributed launch surface."""

import torch

import pypto_b200.language as pl
import pypto_b200.language.distributed as pld

W_PAD = IDX_PAD = 8


def build(n_ranks, T, TOPK, D, L, R):
    N_RANKS, N_ROUTES = n_ranks, T * TOPK

    @pl.program
    class EpDispatchCombine:
        @pl.function(type=pl.FunctionType.Orchestration)
        def chip_orch(self,
                      indices: pl.Tensor[[T, TOPK], pl.INT32],
                      x_norm: pl.Tensor[[T, D], pl.BF16],
                      w_padded: pl.Tensor[[N_ROUTES, W_PAD], pl.FP32],
                      idx_padded: pl.Tensor[[N_ROUTES, IDX_PAD], pl.INT32],
                      recv_x_out: pl.Out[pl.Tensor[[L * R, D], pl.BF16]],
                      recv_w_out: pl.Out[pl.Tensor[[L, R], pl.FP32]],
                      recv_idx_out: pl.Out[pl.Tensor[[L, R], pl.INT32]],
                      recv_count_out: pl.Out[pl.Tensor[[L, 1], pl.INT32]],
                      recv_y: pl.Out[pl.Tensor[[L * R, D], pl.BF16]],
                      routed_y: pl.Out[pl.Tensor[[T, D], pl.FP32]],
                      pub_counts: pld.DistributedTensor[[N_RANKS * N_RANKS, L], pl.INT32],
                      my_rank: pl.Scalar[pl.INT32]) -> pl.Tensor[[T, D], pl.FP32]:
            ...

        @pl.function(level=pl.Level.HOST, role=pl.Role.Orchestrator)
        def host_orch(self,
                      indices: pl.Tensor[[N_RANKS, T, TOPK], pl.INT32],
                      x_norms: pl.Tensor[[N_RANKS, T, D], pl.BF16],
                      w_padded: pl.Tensor[[N_RANKS, N_ROUTES, W_PAD], pl.FP32],
                      idx_padded: pl.Tensor[[N_RANKS, N_ROUTES, IDX_PAD], pl.INT32],
                      recv_x_outs: pl.Out[pl.Tensor[[N_RANKS, L * R, D], pl.BF16]],
                      recv_w_outs: pl.Out[pl.Tensor[[N_RANKS, L, R], pl.FP32]],
                      recv_idx_outs: pl.Out[pl.Tensor[[N_RANKS, L, R], pl.INT32]],
                      recv_count_outs: pl.Out[pl.Tensor[[N_RANKS, L, 1], pl.INT32]],
                      recv_ys: pl.Out[pl.Tensor[[N_RANKS, L * R, D], pl.BF16]],
                      routed_ys: pl.Out[pl.Tensor[[N_RANKS, T, D], pl.FP32]]) -> pl.Tensor[[N_RANKS, T, D], pl.FP32]:
            ...

    return EpDispatchCombine


def host_tensors(x, weights, indices, L, R):
    """The ten rank-stacked host tensors of host_orch from x [N, T, D], weights [N, T, K], indices [N, T, K]:
    weights and route ids padded to 8 columns as the reference packs them (:541-560), outputs zeroed."""
    n, t, d = x.shape
    k = indices.shape[2]
    w_padded = torch.zeros(n, t * k, W_PAD)
    w_padded[:, :, 0] = weights.reshape(n, t * k)
    idx_padded = torch.zeros(n, t * k, IDX_PAD, dtype=torch.int32)
    idx_padded[:, :, 0] = torch.arange(t * k, dtype=torch.int32)
    return [indices.to(torch.int32).contiguous(), x.contiguous(), w_padded, idx_padded,
            torch.zeros(n, L * R, d, dtype=torch.bfloat16), torch.zeros(n, L, R), torch.zeros(n, L, R, dtype=torch.int32),
            torch.zeros(n, L, 1, dtype=torch.int32), torch.zeros(n, L * R, d, dtype=torch.bfloat16), torch.zeros(n, t, d)]
