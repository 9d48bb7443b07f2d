"""Decoder-layer composition on the device: the order of scopes and every rounding point of
the reference's decode layer (examples/models/qwen3_jit/qwen3_decode.py:50-112; golden
tests/st/runtime/framework_and_models/test_qwen3_decode_scope3_mixed.py:256-287), with the
paged-attention kernel in the place the reference example leaves open (:95-99).

    RMSNorm (bf16) -> QKV projection (fp32) -> RoPE + KV-cache append (bf16) -> paged
    attention (bf16) -> o-proj + residual (fp32) -> RMSNorm (bf16) -> SwiGLU MLP (bf16
    activation) -> down-proj + residual (fp32) -> bf16

Weights are packed once at construction ([K, N] -> [N, K] bf16, Q/K/V and gate/up
concatenated so each pair is one GEMM).  torch supplies buffers and the stream only.
"""

from __future__ import annotations

import torch

from . import ops


class SwiGLUFFN:
    """``ffn_swiglu(x, Wg, Wu, Wd)`` of examples/models/01_ffn.py:112-131 with weights packed
    once.  fp32 inputs are cast to bf16 operands (fp32 accumulation), which the 2e-2 bar of the
    workload definition allows."""

    launches_per_call = 2   # kernels of one call with fp32 input and at most 128 rows: cast + clear, fused FFN

    def __init__(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor):
        self.hidden, self.inter = w_gate.shape
        self.n_out = w_down.shape[1]
        self.w_gate_up = ops.pack_weight(torch.cat([w_gate, w_up], dim=1).contiguous())
        self.w_down = ops.pack_weight(w_down.contiguous())

    def __call__(self, x: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
        if x.dtype == torch.bfloat16:
            return ops.ffn_swiglu(x, self.w_gate_up, self.w_down, out=out, accumulate=accumulate)
        if out is None:
            out = torch.empty(x.shape[0], self.n_out, dtype=torch.float32, device=x.device)
        if accumulate or (out.numel() * 4) % 16 or out.data_ptr() % 16:
            return ops.ffn_swiglu(ops.cast(x.contiguous(), torch.bfloat16), self.w_gate_up, self.w_down, out=out,
                                  accumulate=accumulate)
        # the cast of x also clears the output, so the FFN accumulates into zeros without a launch of its own.  (The
        # operator also takes fp32 x directly and then casts inside its one launch -- ops.ffn_swiglu -- which is
        # 3-4 us quicker for a lone call; in a stream of calls the separate cast overlaps the tail of the kernel
        # before it and a step is 1.4 us shorter this way.)
        xb = ops.cast(x.contiguous(), torch.bfloat16, zero=out)
        return ops.ffn_swiglu(xb, self.w_gate_up, self.w_down, out=out, accumulate=True)

    def weight_bytes(self) -> int:
        return (self.w_gate_up.numel() + self.w_down.numel()) * 2


class DecoderLayer:
    # kernels of one step: RMSNorm, QKV GEMM, RoPE + append, attention, merge, O GEMM, RMSNorm, gate/up GEMM,
    # SwiGLU, down GEMM, cast
    launches_per_step = 11

    def __init__(self, t: dict, *, num_heads: int, kv_heads: int, head_dim: int, block_size: int, eps: float,
                 scale: float):
        """``t`` holds device tensors wq/wk/wv/wo/w_gate/w_up/w_down in the reference's
        ``x @ W`` layout ([in, out], bf16), input_rms_weight/post_rms_weight fp32 [1, H],
        rope_cos/rope_sin fp32 [S, D]."""
        self.num_heads, self.kv_heads, self.head_dim = num_heads, kv_heads, head_dim
        self.block_size, self.eps, self.scale = block_size, eps, scale
        self.w_qkv = ops.pack_weight(torch.cat([t["wq"], t["wk"], t["wv"]], dim=1).contiguous())
        self.w_o = ops.pack_weight(t["wo"].contiguous())
        self.ffn = SwiGLUFFN(t["w_gate"], t["w_up"], t["w_down"])
        self.gamma_in = t["input_rms_weight"].reshape(-1).contiguous()
        self.gamma_post = t["post_rms_weight"].reshape(-1).contiguous()
        self.cos, self.sin = t["rope_cos"].contiguous(), t["rope_sin"].contiguous()

    def weight_bytes(self) -> int:
        return (self.w_qkv.numel() + self.w_o.numel()) * 2 + self.ffn.weight_bytes()

    def step(self, hidden: torch.Tensor, seq_lens: torch.Tensor, block_table: torch.Tensor,
             k_cache: torch.Tensor, v_cache: torch.Tensor) -> torch.Tensor:
        """One decode step for ``hidden`` bf16 [batch, H]; the caches are updated in place at
        position seq_len - 1 of every sequence.  Returns bf16 [batch, H]."""
        batch = hidden.shape[0]
        # the input norm also leaves fp32(hidden) as the residual and clears the QKV accumulator
        resid = torch.empty(hidden.shape, dtype=torch.float32, device=hidden.device)
        qkv = torch.empty(batch, self.w_qkv.shape[0], dtype=torch.float32, device=hidden.device)
        normed = ops.rms_norm(hidden, self.gamma_in, self.eps, torch.bfloat16, copy_fp32=resid, zero=qkv)
        ops.linear(normed, self.w_qkv, out=qkv, accumulate=True)
        q_rot = ops.rope_kv_append(qkv, seq_lens, self.cos, self.sin, block_table, k_cache, v_cache,
                                   num_heads=self.num_heads, kv_heads=self.kv_heads, head_dim=self.head_dim,
                                   block_size=self.block_size)
        attn = ops.paged_attention(q_rot, k_cache, v_cache, block_table, seq_lens, num_heads=self.num_heads,
                                   kv_heads=self.kv_heads, head_dim=self.head_dim, block_size=self.block_size,
                                   scale=self.scale, out_dtype=torch.bfloat16)
        ops.linear(attn.view(batch, self.num_heads * self.head_dim), self.w_o, out=resid, accumulate=True)
        post = ops.rms_norm(resid, self.gamma_post, self.eps, torch.bfloat16)
        self.ffn(post, out=resid, accumulate=True)   # resid now holds down + resid1
        return ops.cast(resid, torch.bfloat16)
