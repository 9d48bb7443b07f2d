"""Pin the oracle: bit-for-bit against fixtures produced by the reference's own
golden functions (tests/golden/make_golden.py), and against those functions
directly whenever the reference tree is present."""

import pytest
import torch

import oracle
from oracle import ep, ffn, gather, layer, llama_mini, matmul_mx, moe
from oracle import paged_attention as pa

PA_CASES = ["pa04_aligned", "pa04_unaligned", "pa04_ragged", "pa04_h64_b64", "pa04_tiny"]


def _run_pa(t):
    cfg = t["config"]
    scale = float(t["scale"][0]) if "scale" in t else pa.unpack_scale(cfg)
    return pa.paged_attention(t["query"], t["key_cache"], t["value_cache"], t["block_table"],
                              t["context_lens"], num_heads=int(cfg[1]), head_dim=int(cfg[3]),
                              block_size=int(cfg[4]), scale=scale, kv_heads=1)


@pytest.mark.parametrize("name", PA_CASES + ["pa09_empty_seq"])
def test_paged_attention_matches_reference_golden(golden, name):
    t = golden(name)
    got = _run_pa(t)
    assert torch.equal(got, t["out"].reshape(got.shape)), (got - t["out"]).abs().max()


def test_golden_entry_point_matches(golden):
    t = golden("pa04_unaligned")
    mine = dict(t)
    mine["out"] = torch.zeros_like(t["out"])
    pa.golden(mine)
    assert torch.equal(mine["out"], t["out"])


def test_empty_sequence_rows_are_zero(golden):
    t = golden("pa09_empty_seq")
    out = _run_pa(t).reshape(3, 16, 128)
    assert torch.count_nonzero(out[0]) == 0 and torch.count_nonzero(out[1]) > 0


def test_paged_gather_fixture(golden):
    t = golden("paged_gather")
    got = gather.paged_gather(t["src"], t["indices"], t["block_table"], t["block_size"], t["size"])
    assert torch.equal(got, t["out"])
    # src[r, c] = r, so every gathered row is the constant phys index (test_paged_gather.py:22-27)
    bs = t["block_size"]
    phys = t["block_table"].long()[t["indices"].long() // bs] * bs + t["indices"].long() % bs
    assert torch.equal(got[:, 0].long(), phys)


@pytest.mark.parametrize("n_ranks", [2, 4])
def test_ep_dispatch_combine_fixture(golden, n_ranks):
    t = golden(f"ep_{n_ranks}")
    rx, rw, ri, rs, cnt = ep.dispatch(t["x"], t["indices"], t["weights"], t["l"], t["r"])
    assert torch.equal(cnt, t["count"])
    assert torch.equal(ri, t["recv_idx"])
    assert torch.equal(rx.view(torch.int16), t["recv_x"].view(torch.int16))
    assert torch.equal(rw, t["recv_w"])
    y = ep.combine(ep.standin_expert(rx, rw), ri, rs, cnt, t["t"], t["topk"])
    assert torch.equal(y, t["routed"])


def test_scope3_fixture(golden):
    t = golden("scope3")
    resid1 = torch.matmul(t["attn_out"].float(), t["wo"].float()) + t["hidden_states"].float()
    post = layer.rms_norm(resid1, t["post_rms_weight"], 1e-6, torch.bfloat16)
    down = ffn.ffn_swiglu_bf16(post, t["w_gate"], t["w_up"], t["w_down"])
    got = (down + resid1).bfloat16()
    assert torch.equal(got.view(torch.int16), t["out"].view(torch.int16))


def test_sort_with_index_on_reference_unique_values(golden):
    src = golden("sort_unique_2048")["src"].reshape(1, -1)
    vals, idx = moe.sort_desc_with_index(src)
    assert torch.equal(vals, torch.sort(src, descending=True)[0])
    assert torch.equal(src[0, idx[0].long()], vals[0])
    assert idx.unique().numel() == 2048


def test_ffn_fp32_expression():
    x, wg, wu, wd = oracle.inputs.ffn_inputs(64, 64, 64, seed=0, w_std=1.0)
    torch.manual_seed(0)  # 01_ffn.py:155-160 draws x, Wg, Wu, Wd in this order
    g = x @ wg
    assert torch.equal(ffn.ffn_swiglu(x, wg, wu, wd), (g * torch.sigmoid(g) * (x @ wu)) @ wd)


def test_rms_norm_forms_agree():
    torch.manual_seed(0)  # test_rms_norm.py:25-37 shapes
    x, gamma = torch.randn(32, 64), torch.randn(1, 64)
    a = layer.rms_norm(x, gamma, 1e-5)
    b = layer.rms_norm_sqrt_div(x, gamma, 1e-5)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-5)


def test_rope_tables_and_rotation():
    cos, sin = layer.rope_tables(16, 64, 10000.0)
    assert cos.shape == (16, 64) and torch.equal(cos[:, :32], cos[:, 32:])
    x = torch.randn(16, 64)
    y = layer.rope_rotate(x, cos, sin)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), rtol=1e-5)  # a rotation
    assert torch.equal(y[0], x[0])  # position 0 rotates by angle 0


def test_fp8_block_quant_roundtrip_and_gemm():
    g = torch.Generator().manual_seed(3)
    w = torch.randn(256, 384, generator=g) * 0.02
    q, s = moe.quantize_weight_blocks(w)
    assert s.shape == (2, 3) and q.dtype == torch.float8_e4m3fn
    assert (moe.dequant_weight(q, s) - w).abs().max() <= w.abs().max() * 2**-4
    x = torch.randn(8, 256, generator=g).bfloat16()
    xq, xs = moe.quantize_rows(x)
    ref = (xq.float() * xs.repeat_interleave(128, 1)) @ moe.dequant_weight(q, s)
    assert torch.allclose(moe.fp8_gemm(xq, xs, q, s), ref, rtol=1e-4, atol=1e-5)


def test_topk_tie_break_and_normalisation():
    scores = torch.tensor([[0.5, 0.9, 0.9, 0.1], [0.2, 0.2, 0.2, 0.2]])
    idx, w = moe.topk_from_scores(scores, torch.zeros(4), 2)
    assert idx.tolist() == [[1, 2], [0, 1]]
    assert torch.allclose(w.sum(-1), torch.ones(2))
    idx, w = moe.topk_from_scores(scores, torch.tensor([1.0, 0, 0, 0]), 1)
    assert idx[0, 0] == 0 and w[0, 0] == 1.0  # bias steers selection, not the weight


def test_gqa_and_draft_mask_extension_consistency():
    """kv_heads>1 equals running each KV head alone; q_len>1 equals q_len single-token
    calls with the context shortened per draft position."""
    d = oracle.inputs.paged_attention_inputs(batch=3, num_heads=8, kv_heads=2, ctx_lo=5,
                                             ctx_hi=300, q_len=3, seed=5)
    kw = dict(num_heads=8, head_dim=128, block_size=128, scale=d["scale"])
    full = pa.paged_attention(d["query"], d["key_cache"], d["value_cache"], d["block_table"],
                              d["context_lens"], kv_heads=2, q_len=3, **kw).reshape(3, 3, 8, 128)
    q = d["query"].reshape(3, 3, 8, 128)
    for j in range(3):
        one = pa.paged_attention(q[:, j].reshape(-1, 128), d["key_cache"], d["value_cache"],
                                 d["block_table"], d["context_lens"] - 3 + j + 1, kv_heads=2,
                                 q_len=1, **kw).reshape(3, 8, 128)
        assert torch.allclose(one, full[:, j], rtol=1e-5, atol=1e-6)  # bmm tiling differs


def test_against_reference_tree_when_present():
    import ref_extract

    if not ref_extract.available():
        pytest.skip("reference tree not mounted")
    ns = ref_extract.extract("examples/models/04_paged_attention.py", ["golden", "build_tensors"])
    torch.manual_seed(1234)
    q, kc, vc, bt, cl, out, cfg = ns["build_tensors"](4, 16, 128, 128, 8, 1000, 0.125)
    t = dict(query=q, key_cache=kc, value_cache=vc, block_table=bt, context_lens=cl, out=out,
             config=cfg)
    ns["golden"](t)
    assert torch.equal(_run_pa(t), t["out"])


def test_rope_tables_and_rotation_fixture(golden):
    """cos/sin tables and the rotate-half of the reference's llama test
    (test_llama_7b_mini_1h.py:83-95, 146-159), bit for bit."""
    t = golden("rope")
    cos, sin = layer.rope_tables(t["cos_emb"].shape[0], t["head_dim"], t["theta"])
    half = t["head_dim"] // 2
    assert torch.equal(cos[:, :half], t["cos_emb"]) and torch.equal(cos[:, half:], t["cos_emb"])
    assert torch.equal(sin[:, :half], t["sin_emb"]) and torch.equal(sin[:, half:], t["sin_emb"])
    assert torch.equal(layer.rope_rotate(t["x"], cos, sin), t["rotated"])


def test_matmul_mx_fixture(golden):
    """The MXFP8 golden and the two physical scale layouts (test_matmul_mx.py:38-131), bit for bit."""
    t = golden("matmul_mx")
    a, b = t["a"].view(torch.float8_e4m3fn), t["b"].view(torch.float8_e4m3fn)
    out = matmul_mx.matmul_mx(a, t["a_scale_codes"], b, t["b_scale_codes"])
    assert torch.equal(out, t["out"])
    assert torch.equal(matmul_mx.matmul_mx(a, t["a_scale_codes"], b, t["b_scale_codes"], acc=out), t["out_acc"])
    assert torch.equal(matmul_mx.pack_a_scale(t["a_scale_codes"]), t["a_scale_packed"])
    assert torch.equal(matmul_mx.pack_b_scale(t["b_scale_codes"]), t["b_scale_packed"])
    assert torch.equal(matmul_mx.unpack_a_scale(t["a_scale_packed"]), t["a_scale_codes"])
    assert torch.equal(matmul_mx.unpack_b_scale(t["b_scale_packed"]), t["b_scale_codes"])


def test_quantize_mx_round_trips_within_e4m3_precision():
    g = torch.Generator().manual_seed(5)
    x = torch.randn(64, 256, generator=g) * 3
    q, codes = matmul_mx.quantize_mx(x, dim=1)
    deq = q.float() * matmul_mx.decode_scale(codes).float().repeat_interleave(32, dim=1)
    assert codes.shape == (64, 8) and (deq - x).abs().max() <= x.abs().max() * 2 ** -3


def test_llama_mini_fixture(golden):
    """The minimal LLaMA forward pass against the output of the reference's own ``compute_expected``
    (test_llama_7b_mini_1h.py:118-199) on tensors made by its own initialisers."""
    t = golden("llama_mini")
    got = llama_mini.forward(t)
    assert got.shape == t["output"].shape
    assert torch.allclose(got, t["output"], rtol=1e-6, atol=1e-7)
    own = llama_mini.make_inputs(seed=3)
    assert llama_mini.forward(own).shape == (16, 64)
    assert torch.equal(own["cos_emb"], t["cos_emb"]) and torch.equal(own["causal_mask"], t["causal_mask"])
