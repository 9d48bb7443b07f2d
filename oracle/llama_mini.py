"""Oracle for the reference's minimal LLaMA forward pass (test infrastructure, not product code).

Restates ``compute_expected`` of tests/st/examples/03_llm_models/test_llama_7b_mini_1h.py:118-199 (the golden of
examples/models/08_llama_mini.py:384-483): one decoder layer with one head -- RMSNorm without gamma (divisor = the
hidden size, eps 1e-6), q/k/v projections, rotate-half RoPE with [S, D/2] tables, causal softmax attention scaled by
D^-0.5 with the mask ADDED to the scores, dense projection + residual, RMSNorm, SwiGLU MLP + residual, final RMSNorm,
LM head.  Everything in fp32.  Pinned by tests/golden/llama_mini.pt, which the reference's own function produced.
"""

from __future__ import annotations

import torch


def make_inputs(seq_len=16, head_dim=64, vocab=64, seed=0):
    """Inputs with the distributions of the reference's ``define_tensors`` (:69-113): N(0,1) hidden states, weights
    U(-0.02, 0.02), mask 0 / -1e9 above the diagonal, RoPE tables theta_i = 10000^(-2i/D)."""
    g = torch.Generator().manual_seed(seed)

    def w(rows, cols):
        return torch.rand(rows, cols, generator=g) * 0.04 - 0.02
    half = head_dim // 2
    pos = torch.arange(seq_len).float().unsqueeze(1)
    theta = 1.0 / (10000.0 ** (2 * torch.arange(half).float() / head_dim))
    ang = pos * theta.unsqueeze(0)
    t = dict(hidden=torch.randn(seq_len, head_dim, generator=g),
             causal_mask=torch.zeros(seq_len, seq_len).masked_fill(
                 torch.triu(torch.ones(seq_len, seq_len), diagonal=1).bool(), -1e9),
             cos_emb=torch.cos(ang), sin_emb=torch.sin(ang))
    for name in ("wq", "wk", "wv", "w_dense", "w_gate", "w_up", "w_down"):
        t[name] = w(head_dim, head_dim)
    t["w_lm"] = w(head_dim, vocab)
    return t


def forward(t: dict) -> torch.Tensor:
    """logits [S, V] (test_llama_7b_mini_1h.py:118-199)."""
    hidden = t["hidden"]
    d = hidden.shape[1]
    half = d // 2
    eps = 1e-6
    scale = d ** -0.5

    def rms_norm(h):
        return h / torch.sqrt((h ** 2).sum(dim=-1, keepdim=True) / d + eps)

    def rope(x):
        lo, hi = x[:, :half], x[:, half:]
        return torch.cat([lo * t["cos_emb"] - hi * t["sin_emb"], hi * t["cos_emb"] + lo * t["sin_emb"]], dim=-1)

    normed = rms_norm(hidden)
    q, k, v = rope(normed @ t["wq"]), rope(normed @ t["wk"]), normed @ t["wv"]
    probs = torch.softmax(q @ k.T * scale + t["causal_mask"], dim=-1)
    attn_res = hidden + (probs @ v) @ t["w_dense"]
    n2 = rms_norm(attn_res)
    gate, up = n2 @ t["w_gate"], n2 @ t["w_up"]
    h1 = attn_res + (gate * torch.sigmoid(gate) * up) @ t["w_down"]
    return rms_norm(h1) @ t["w_lm"]
