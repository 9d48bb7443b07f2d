"""GPU: reference-style programs for the remaining fused entries -- the SPMD paged-attention
signature, the @pl.jit ffn_swiglu and rms_norm functions -- run through run() / the JIT call
and are checked against the oracle."""

import pytest
import torch

import oracle
import pypto_b200.language as pl
from oracle import ffn as offn
from oracle import layer as olayer
from oracle import paged_attention as opa
from pypto_b200.runtime import RunConfig, run, validate_golden

pytestmark = pytest.mark.gpu


def test_jit_ffn_swiglu_reference_signature():
    @pl.jit
    def ffn_swiglu(hidden_states: pl.Tensor, gate_proj_weight: pl.Tensor, up_proj_weight: pl.Tensor,
                   down_proj_weight: pl.Tensor, output: pl.Out[pl.Tensor]):
        ...
    x, wg, wu, wd = oracle.inputs.ffn_inputs(64, 64, 64, seed=0, w_std=1.0)      # 01_ffn.py:155-160
    out = torch.zeros(64, 64)
    ffn_swiglu(x, wg, wu, wd, out, config=RunConfig())
    exp = offn.ffn_swiglu(x, wg, wu, wd)
    assert (out - exp).abs().max() <= 2e-2 * exp.abs().max()
    x, wg, wu, wd = oracle.inputs.ffn_inputs(128, 1024, 4096, seed=0)             # the benchmark shape
    out = torch.zeros(128, 1024)
    ffn_swiglu(x, wg, wu, wd, out)
    exp = offn.ffn_swiglu(x, wg, wu, wd)
    assert (out - exp).abs().max() <= 2e-2 * exp.abs().max()
    assert len(ffn_swiglu._cache) == 2


def test_jit_rms_norm_reference_signature():
    @pl.jit
    def rms_norm(x: pl.Tensor, gamma: pl.Tensor, output: pl.Out[pl.Tensor]):
        ...
    torch.manual_seed(0)                                                           # test_rms_norm.py:25-37
    x, gamma = torch.randn(32, 64), torch.randn(1, 64)
    out = torch.zeros_like(x)
    rms_norm(x, gamma, out)
    validate_golden({"output": out}, {"output": olayer.rms_norm_sqrt_div(x, gamma, 1e-5)}, rtol=1e-5, atol=1e-5)


def test_spmd_paged_attention_signature(golden):
    t = golden("pa09_empty_seq")
    cfg = t["config"]
    batch, heads, hd, bs, nblk = int(cfg[0]), int(cfg[1]), int(cfg[3]), int(cfg[4]), int(cfg[5])

    @pl.program
    class SpmdPagedAttention:
        @pl.function(type=pl.FunctionType.Orchestration)
        def paged_attention_spmd(self, query: pl.Tensor[[batch * heads, hd], pl.BF16], key_cache: pl.Tensor[pl.BF16],
                                 value_cache: pl.Tensor[pl.BF16], block_table: pl.Tensor[[batch * nblk], pl.INT32],
                                 context_lens: pl.Tensor[[batch], pl.INT32], scale: pl.Tensor[[1], pl.FP32],
                                 out: pl.Out[pl.Tensor[[batch * heads, hd], pl.FP32]],
                                 config: pl.Tensor[[7], pl.INT64]):
            ...
    out = torch.zeros_like(t["out"])
    run(SpmdPagedAttention, t["query"], t["key_cache"], t["value_cache"], t["block_table"], t["context_lens"],
        t["scale"], out, cfg)
    validate_golden({"out": out}, {"out": t["out"]}, rtol=2e-2, atol=4e-3)
    # fewer active blocks than the contexts need: blocks past them are not read (09_...:604-607)
    cfg2 = cfg.clone()
    cfg2[6] = 1
    out2 = torch.zeros_like(out)
    run(SpmdPagedAttention, t["query"], t["key_cache"], t["value_cache"], t["block_table"], t["context_lens"],
        t["scale"], out2, cfg2)
    exp = opa.paged_attention(t["query"], t["key_cache"], t["value_cache"], t["block_table"],
                              torch.clamp(t["context_lens"], max=bs), num_heads=heads, head_dim=hd, block_size=bs,
                              scale=float(t["scale"][0]))
    validate_golden({"out": out2}, {"out": exp.reshape(out2.shape)}, rtol=2e-2, atol=4e-3)


def test_programs_recognised_by_what_they_compute_run_on_the_fused_kernels():
    """A gated MLP and a scaled norm under names, parameter orders and algebraic spellings of their own
    (tests/dsl_programs/renamed_idioms.py): the idiom recogniser binds the fused operators' roles to their parameters."""
    from tests.dsl_programs import renamed_idioms as progs
    x, wg, wu, wd = oracle.inputs.ffn_inputs(128, 1024, 4096, seed=3)
    y = torch.zeros(128, 1024)
    progs.gated_mlp(wd, wu, x, wg, y)                     # (w_out, w_lin, tokens, w_act, y)
    exp = offn.ffn_swiglu(x, wg, wu, wd)
    assert (y - exp).abs().max() <= 2e-2 * exp.abs().max()
    swapped = torch.zeros(128, 1024)
    progs.gated_mlp(wd, wg, x, wu, swapped)               # gate and up exchanged: another function of the inputs
    assert (swapped - offn.ffn_swiglu(x, wu, wg, wd)).abs().max() <= 2e-2 * exp.abs().max()
    assert (swapped - exp).abs().max() > 0.1 * exp.abs().max()
    torch.manual_seed(1)
    rows, weight = torch.randn(32, 64), torch.randn(1, 64)
    normed = torch.zeros_like(rows)
    progs.scaled_norm(weight, rows, normed)
    validate_golden({"normed": normed}, {"normed": olayer.rms_norm_sqrt_div(rows, weight, progs.EPS)}, rtol=1e-5, atol=1e-5)
    with pytest.raises(ValueError, match="not 1 / 128"):
        progs.scaled_norm(torch.randn(1, 128), torch.randn(32, 128), torch.zeros(32, 128))   # the program divides by 64


def test_matrix_product_programs_run_on_the_tensor_core_gemm():
    """`dst = lhs @ rhs` and `dst = offset + lhs @ rhs` under names of their own (the shapes of the reference's
    05_matmul.py and 01_fused_linear.py examples, fp32 tensors): recognised by their bodies, run by the `linear`
    callable with bf16 operands and fp32 accumulation, held to 2e-2 of the output scale."""
    from tests.dsl_programs import renamed_idioms as progs
    torch.manual_seed(0)
    a, b, off = torch.randn(64, 64), torch.randn(64, 64), torch.randn(64, 64)
    dst = torch.zeros(64, 64)
    progs.product(a, b, dst)
    exp = a @ b
    assert (dst - exp).abs().max() <= 2e-2 * exp.abs().max()
    dst2 = torch.full((64, 64), 9.0)
    progs.affine(off, a, b, dst2)
    assert (dst2 - (exp + off)).abs().max() <= 2e-2 * (exp + off).abs().max()
    a, b = torch.randn(300, 520), torch.randn(520, 384)                # ragged tiles, more than 256 rows
    dst = torch.zeros(300, 384)
    progs.product(a, b, dst)
    exp = a.bfloat16().float() @ b.bfloat16().float()
    assert (dst - exp).abs().max() <= 2e-3 * exp.abs().max()


def test_gelu_and_relu_ffns_by_name_and_by_body():
    """`ffn_gelu` / `ffn_relu` with the reference's signature (examples/models/01_ffn.py:92-108, 134-150; 64 x 64 fp32,
    N(0,1) weights as in :155-160) and a SiLU MLP under names of its own: the one-projection FFN (GEMM, activation,
    GEMM) against the fp32 expressions, bf16 operands held to 2e-2 of the output scale."""
    from tests.dsl_programs import renamed_idioms as progs

    @pl.jit
    def ffn_gelu(hidden_states: pl.Tensor, gate_proj_weight: pl.Tensor, down_proj_weight: pl.Tensor,
                 output: pl.Out[pl.Tensor]):
        ...

    @pl.jit
    def ffn_relu(hidden_states: pl.Tensor, gate_proj_weight: pl.Tensor, down_proj_weight: pl.Tensor,
                 output: pl.Out[pl.Tensor]):
        ...
    torch.manual_seed(0)
    x, wg, wd = torch.randn(64, 64), torch.randn(64, 64), torch.randn(64, 64)
    for fn, exp in ((ffn_gelu, offn.ffn_gelu(x, wg, wd)), (ffn_relu, offn.ffn_relu(x, wg, wd))):
        out = torch.zeros(64, 64)
        fn(x, wg, wd, out)
        assert (out - exp).abs().max() <= 2e-2 * exp.abs().max(), fn.name
    x, wa, wb = torch.randn(200, 512) , torch.randn(512, 1024) * 0.05, torch.randn(1024, 256) * 0.05
    y = torch.zeros(200, 256)
    progs.swish_mlp(wb, x, wa, y)
    exp = offn.ffn_gelu(x, wa, wb, alpha=1.0)
    assert (y - exp).abs().max() <= 2e-2 * exp.abs().max()
