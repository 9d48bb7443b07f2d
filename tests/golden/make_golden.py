"""Generate the committed golden fixtures from the reference's own golden functions.

Run from the repository root with the reference tree present:
    python tests/golden/make_golden.py
Each fixture is a ``torch.save`` dict of the inputs handed to an (AST-extracted,
unmodified) reference function and the outputs it produced.  The CPU tests check
the oracle against these files bit-for-bit, so the pin holds on machines that do
not have the reference tree.
"""

from __future__ import annotations

import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import ref_extract  # noqa: E402

PA04 = "examples/models/04_paged_attention.py"
PA09 = "examples/models/09_paged_attention_spmd.py"
GATHER = "tests/st/runtime/ops/test_paged_gather.py"
EP = "tests/st/distributed/test_l3_ep_dispatch_combine.py"
SCOPE3 = "tests/st/runtime/framework_and_models/test_qwen3_decode_scope3_mixed.py"
SORT = "tests/st/runtime/ops/test_sort.py"
LLAMA = "tests/st/examples/03_llm_models/test_llama_7b_mini_1h.py"
MX = "tests/st/runtime/ops/test_matmul_mx.py"

EP_SMALL = dict(T=16, TOPK=3, D=32, L=4, R=40, N_ROUTES=48)


def pa04_case(batch, heads, head_dim, block, max_blocks, ctx, scale, seed, ctx_list=None):
    ns = ref_extract.extract(PA04, ["golden", "build_tensors"])
    torch.manual_seed(seed)
    q, kc, vc, bt, cl, out, cfg = ns["build_tensors"](batch, heads, head_dim, block, max_blocks,
                                                      ctx, scale)
    if ctx_list is not None:
        cl = torch.tensor(ctx_list, dtype=torch.int32)
    t = dict(query=q, key_cache=kc, value_cache=vc, block_table=bt, context_lens=cl, out=out,
             config=cfg)
    ns["golden"](t)
    return t


def rope_case():
    """RoPE tables and rotate-half from the reference's llama test (helpers nested in
    define_tensors / compute_expected, test_llama_7b_mini_1h.py:83-95, 146-159)."""
    tab = ref_extract.extract(LLAMA, ["make_cos_emb", "make_sin_emb"], overrides={"head_dim": 64}, nested=True)
    cos, sin = tab["make_cos_emb"](), tab["make_sin_emb"]()
    rot = ref_extract.extract(LLAMA, ["apply_rope"], overrides={"cos_emb": cos, "sin_emb": sin}, nested=True)
    x = torch.randn(16, 64, generator=torch.Generator().manual_seed(11))
    return dict(cos_emb=cos, sin_emb=sin, x=x, rotated=rot["apply_rope"](x), head_dim=64, theta=10000.0)


def llama_mini_case():
    """The reference's minimal LLaMA case (test_llama_7b_mini_1h.py:69-199): its own tensor initialisers (nested in
    define_tensors) and its own ``compute_expected``, run unmodified; S = 16, D = 64, V = 64."""
    init = ref_extract.extract(LLAMA, ["make_small_weight", "make_causal_mask", "make_cos_emb", "make_sin_emb"],
                               overrides={"head_dim": 64}, nested=True)
    torch.manual_seed(29)
    t = dict(hidden=torch.randn(16, 64), causal_mask=init["make_causal_mask"](), cos_emb=init["make_cos_emb"](),
             sin_emb=init["make_sin_emb"]())
    for name in ("wq", "wk", "wv", "w_dense", "w_gate", "w_up", "w_down", "w_lm"):
        t[name] = init["make_small_weight"]()
    t["output"] = torch.zeros(16, 64)
    ns = ref_extract.extract(LLAMA, ["compute_expected"], nested=True)
    ns["compute_expected"](None, t)
    return t


def matmul_mx_case():
    """The reference's MXFP8 x MXFP8 case (test_matmul_mx.py:146-168): integer-valued e4m3 data in
    [-2, 2], E8M0 scale codes 126..129, scales in the packed MX_A_ZZ / MX_B_NN layouts it hands to the
    kernel, and the golden of :119-131 (dequantise per 32-wide K group, fp64 matmul, fp32 result)."""
    names = ["_pack_a_scale", "_unpack_a_scale", "_pack_b_scale", "_unpack_b_scale", "_matmul_mx_golden",
             "M", "K", "N", "MX_GROUP_SIZE", "SCALE_BLOCK_SIZE", "SCALE_C0_SIZE"]
    ns = ref_extract.extract(MX, names)
    m, k, n = ns["M"], ns["K"], ns["N"]
    g = torch.Generator().manual_seed(23)                       # _make_case_inputs(lhs_fp4=False), :156-168
    a = torch.randint(-2, 3, (m, k), generator=g).to(torch.float8_e4m3fn)
    b = torch.randint(-2, 3, (k, n), generator=g).to(torch.float8_e4m3fn)
    a_codes = torch.randint(126, 130, (m, k // 32), generator=g).to(torch.uint8)
    b_codes = torch.randint(126, 130, (k // 32, n), generator=g).to(torch.uint8)
    a_packed, b_packed = ns["_pack_a_scale"](a_codes), ns["_pack_b_scale"](b_codes)
    assert torch.equal(ns["_unpack_a_scale"](a_packed), a_codes) and torch.equal(ns["_unpack_b_scale"](b_packed), b_codes)
    out = ns["_matmul_mx_golden"](a.to(torch.float64), a_codes, b.to(torch.float64), b_codes)
    return dict(a=a.view(torch.uint8), b=b.view(torch.uint8), a_scale_codes=a_codes, b_scale_codes=b_codes,
                a_scale_packed=a_packed, b_scale_packed=b_packed, out=out, out_acc=2 * out, m=m, k=k, n=n)


def main():
    fx = {}
    # reference-shaped attention cases, shrunk pools; the aligned/unaligned/ragged
    # lengths mirror test_paged_attention.py:843-887 and
    # test_dynamic_paged_attention.py:220-229 at small scale
    fx["pa04_aligned"] = pa04_case(2, 16, 128, 128, 4, 256, 1.0, 42)
    fx["pa04_unaligned"] = pa04_case(2, 16, 128, 128, 4, 300, 0.0884, 43)
    fx["pa04_ragged"] = pa04_case(4, 16, 128, 128, 4, 0, 1.0, 44, ctx_list=[1, 127, 129, 512])
    fx["pa04_h64_b64"] = pa04_case(2, 64, 128, 64, 6, 200, 0.5, 45)
    fx["pa04_tiny"] = pa04_case(2, 16, 16, 16, 16, 64, 1.0, 46)  # test_batch_paged_attention.py:1090

    ns = ref_extract.extract(PA09, ["golden"])
    t = pa04_case(3, 16, 128, 128, 4, 0, 1.0, 47, ctx_list=[0, 200, 384])
    t["config"] = torch.tensor([3, 16, 1, 128, 128, 4, 4], dtype=torch.int64)
    t["scale"] = torch.tensor([0.25], dtype=torch.float32)
    t["out"] = torch.zeros_like(t["out"])
    ns["golden"](t)
    fx["pa09_empty_seq"] = t

    ns = ref_extract.extract(GATHER, ["_paged_gather_golden", "_make_src", "_make_block_table",
                                      "_make_indices", "_BLOCK_SIZE", "_PHYS_BLOCKS",
                                      "_POOL_ROWS", "_HIDDEN", "_NUM_IDX"])
    src, bt, idx = ns["_make_src"](), ns["_make_block_table"](), ns["_make_indices"]()
    fx["paged_gather"] = dict(src=src, block_table=bt, indices=idx, block_size=ns["_BLOCK_SIZE"],
                              size=ns["_HIDDEN"],
                              out=ns["_paged_gather_golden"](src, idx, bt, ns["_BLOCK_SIZE"],
                                                             ns["_HIDDEN"]))

    ns = ref_extract.extract(EP, ["_compute_golden_recv", "_compute_golden_routed",
                                  "_generate_routing_indices", "T", "TOPK", "D", "L", "R",
                                  "N_ROUTES"], overrides=EP_SMALL)
    for n_ranks in (2, 4):
        T, K, D = EP_SMALL["T"], EP_SMALL["TOPK"], EP_SMALL["D"]
        x = torch.tensor([[[r * 100 + t * 10 + d for d in range(D)] for t in range(T)]
                          for r in range(n_ranks)], dtype=torch.bfloat16)
        w = torch.tensor([[[(r + 1) * 0.01 + t * 0.1 + k * 0.001 for k in range(K)]
                           for t in range(T)] for r in range(n_ranks)], dtype=torch.float32)
        ind = ns["_generate_routing_indices"](seed=20260510, n_ranks=n_ranks)
        rx, rw, ri, cnt = ns["_compute_golden_recv"](x, ind, w)
        fx[f"ep_{n_ranks}"] = dict(x=x, weights=w, indices=ind, recv_x=rx, recv_w=rw, recv_idx=ri,
                                   count=cnt, routed=ns["_compute_golden_routed"](x, w),
                                   **{k.lower(): v for k, v in EP_SMALL.items()})

    ns = ref_extract.extract(SCOPE3, ["golden"])
    g = torch.Generator().manual_seed(7)
    b, h, inter = 4, 256, 512
    t = dict(attn_out=(torch.randn(b, h, generator=g) / h**0.5).bfloat16(),
             hidden_states=torch.randn(b, h, generator=g).bfloat16(),
             wo=(torch.randn(h, h, generator=g) / h**0.5).bfloat16(),
             post_rms_weight=torch.rand(1, h, generator=g) + 0.5,
             w_gate=(torch.randn(h, inter, generator=g) / h**0.5).bfloat16(),
             w_up=(torch.randn(h, inter, generator=g) / h**0.5).bfloat16(),
             w_down=(torch.randn(inter, h, generator=g) / inter**0.5).bfloat16(),
             out=torch.zeros(b, h, dtype=torch.bfloat16))
    ns["golden"](t)
    fx["scope3"] = t

    ns = ref_extract.extract(SORT, ["_make_unique_fp32_values"])
    fx["sort_unique_2048"] = dict(src=ns["_make_unique_fp32_values"](2048))

    fx["rope"] = rope_case()
    fx["matmul_mx"] = matmul_mx_case()
    fx["llama_mini"] = llama_mini_case()

    for name, data in fx.items():
        torch.save(data, os.path.join(HERE, name + ".pt"))
        print(name, os.path.getsize(os.path.join(HERE, name + ".pt")))


if __name__ == "__main__":
    if not ref_extract.available():
        sys.exit("reference tree not found; set PYPTO_REFERENCE_ROOT")
    main()
