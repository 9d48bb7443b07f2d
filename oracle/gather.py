"""Oracle for the block-table row gather (test infrastructure, not product code).

Restates tests/st/runtime/ops/test_paged_gather.py:65-74 (semantics stated at
:14-17 and in src/ir/op/tensor_ops/paged_gather.cpp:63-169):
    phys   = block_table[idx // block_size] * block_size + idx % block_size
    out[i] = src[phys, col_off : col_off + size]
Integer arithmetic only: results are compared bit-exactly.
"""

from __future__ import annotations

import torch


def paged_gather(src, indices, block_table, block_size, size, col_off=0):
    idx = indices.long()
    phys = block_table.long()[idx // block_size] * block_size + idx % block_size
    return src[phys, col_off : col_off + size].clone()
