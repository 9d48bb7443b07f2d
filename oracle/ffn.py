"""Oracle for the FFNs of examples/models/01_ffn.py (test infrastructure, not product code).

Restates
  examples/models/01_ffn.py:174-176  fp32: (gate * sigmoid(gate) * up) @ W_down
  examples/models/01_ffn.py:51-62, 80-86  the GELU (x * sigmoid(1.702 x)) and ReLU variants
  tests/st/runtime/framework_and_models/test_qwen3_decode_scope3_mixed.py:282-285
      bf16 variant: operands bf16, fp32 accumulate, activation rounded to bf16
      before the down projection.
"""

from __future__ import annotations

import torch


def ffn_swiglu(x, w_gate, w_up, w_down):
    """fp32 SwiGLU FFN, the expression of 01_ffn.py:174-176."""
    gate = x @ w_gate
    up = x @ w_up
    return (gate * torch.sigmoid(gate) * up) @ w_down


def ffn_swiglu_bf16(x_bf16, w_gate, w_up, w_down):
    """bf16-operand FFN with the reference's rounding points
    (test_qwen3_decode_scope3_mixed.py:282-285): fp32 accumulate, activation
    rounded to bf16, fp32 result returned (the caller adds the residual)."""
    xf = x_bf16.float()
    gate = torch.matmul(xf, w_gate.float())
    up = torch.matmul(xf, w_up.float())
    act = (gate * torch.sigmoid(gate) * up).bfloat16()
    return torch.matmul(act.float(), w_down.float())


def ffn_gelu(x, w_gate, w_down, alpha=1.702):
    """fp32 FFN with the reference's GELU, x * sigmoid(1.702 x) (examples/models/01_ffn.py:51-62, 92-108)."""
    gate = x @ w_gate
    return (gate * torch.sigmoid(alpha * gate)) @ w_down


def ffn_relu(x, w_gate, w_down):
    """fp32 FFN with ReLU (examples/models/01_ffn.py:80-86, 134-150)."""
    return torch.relu(x @ w_gate) @ w_down


def ffn_flops(m, k, inter):
    return 3 * 2 * m * k * inter
