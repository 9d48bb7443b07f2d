"""Programs of the reference that reach a registered callable of the C++ runtime through ``compiled(...)``: the
decode layer (``qwen3_decode``), its third scope against the reference-generated fixture, the MX matmul
program with the reference's physical scale layouts, and the error word surfacing as an exception."""

import math
import struct

import pytest
import torch

import pypto_b200.language as pl
from oracle import layer as olayer

pytestmark = pytest.mark.gpu


def _qwen3_decode_program():
    @pl.jit
    def qwen3_decode(hidden_states: pl.Tensor, input_rms_weight: pl.Tensor, wq: pl.Tensor, wk: pl.Tensor,
                     wv: pl.Tensor, seq_lens: pl.Tensor, rope_cos: pl.Tensor, rope_sin: pl.Tensor,
                     k_cache: pl.Tensor, v_cache: pl.Tensor, wo: pl.Tensor, post_rms_weight: pl.Tensor,
                     w_gate: pl.Tensor, w_up: pl.Tensor, w_down: pl.Tensor, out: pl.Out[pl.Tensor]):
        ...                      # signature of examples/models/qwen3_jit/qwen3_decode.py:49-66
    return qwen3_decode


def test_qwen3_decode_layer_matches_oracle():
    b, hidden, heads, kvh, hd, inter, max_seq = 4, 512, 4, 2, 128, 1024, 256
    g = torch.Generator().manual_seed(21)

    def w(*shape, std=0.05):
        return (torch.randn(*shape, generator=g) * std).bfloat16()

    cos, sin = olayer.rope_tables(max_seq, hd, 10000.0)
    t = dict(hidden=torch.randn(b, hidden, generator=g).bfloat16(),
             input_rms_weight=torch.rand(1, hidden, generator=g) + 0.5, post_rms_weight=torch.rand(1, hidden, generator=g) + 0.5,
             wq=w(hidden, heads * hd), wk=w(hidden, kvh * hd), wv=w(hidden, kvh * hd), wo=w(heads * hd, hidden),
             w_gate=w(hidden, inter), w_up=w(hidden, inter), w_down=w(inter, hidden),
             seq_lens=torch.tensor([1, 100, 129, 256], dtype=torch.int32), rope_cos=cos, rope_sin=sin,
             k_cache=torch.randn(b * kvh * max_seq, hd, generator=g).bfloat16(),
             v_cache=torch.randn(b * kvh * max_seq, hd, generator=g).bfloat16())
    # the contiguous cache row (b * kvh + ki) * max_seq + pos is the paged layout with one block of max_seq tokens
    ref = {k: v.clone() for k, v in t.items()}
    ref["block_table"] = torch.arange(b, dtype=torch.int32).reshape(b, 1)
    exp = olayer.decoder_layer(ref, num_heads=heads, kv_heads=kvh, head_dim=hd, block_size=max_seq, eps=1e-6,
                               scale=1.0 / math.sqrt(hd))
    out = torch.zeros(b, hidden, dtype=torch.bfloat16)
    prog = _qwen3_decode_program()
    prog(t["hidden"], t["input_rms_weight"], t["wq"], t["wk"], t["wv"], t["seq_lens"], t["rope_cos"], t["rope_sin"],
         t["k_cache"], t["v_cache"], t["wo"], t["post_rms_weight"], t["w_gate"], t["w_up"], t["w_down"], out)
    rel = ((out.float() - exp.float()).norm() / exp.float().norm()).item()
    assert rel < 1e-2, rel
    # the caches were updated in place at pos = seq_len - 1 and read back
    for name in ("k_cache", "v_cache"):
        changed = (t[name].view(torch.int16) != ref[name].view(torch.int16)).any(dim=1)
        assert int(changed.sum()) == 0, name            # same rows, same rounded values as the oracle's append
    rows = [(bi * kvh + ki) * max_seq + int(t["seq_lens"][bi]) - 1 for bi in range(b) for ki in range(kvh)]
    assert torch.equal(t["k_cache"][rows].view(torch.int16), ref["k_cache"][rows].view(torch.int16))


def test_scope3_program_matches_reference_fixture(golden):
    t = golden("scope3")
    b, h = t["hidden_states"].shape
    inter = t["w_gate"].shape[1]

    @pl.program
    class Qwen3Scope3:
        @pl.function(type=pl.FunctionType.Orchestration)
        def scope3(self, attn_out: pl.Tensor[[b, h], pl.BF16], hidden_states: pl.Tensor[[b, h], pl.BF16],
                   wo: pl.Tensor[[h, h], pl.BF16], post_rms_weight: pl.Tensor[[1, h], pl.FP32],
                   w_gate: pl.Tensor[[h, inter], pl.BF16], w_up: pl.Tensor[[h, inter], pl.BF16],
                   w_down: pl.Tensor[[inter, h], pl.BF16],
                   out: pl.Out[pl.Tensor[[b, h], pl.BF16]]) -> pl.Tensor[[b, h], pl.BF16]:
            ...

    from pypto_b200.runtime import RunConfig, run
    out = torch.zeros(b, h, dtype=torch.bfloat16)
    run(Qwen3Scope3, t["attn_out"], t["hidden_states"], t["wo"], t["post_rms_weight"], t["w_gate"], t["w_up"],
        t["w_down"], out, config=RunConfig(platform="b200"))
    exp = t["out"].float()
    assert ((out.float() - exp).norm() / exp.norm()).item() < 1e-2
    assert torch.allclose(out.float(), exp, rtol=2e-2, atol=2e-2 * exp.abs().max().item())


def test_matmul_mx_program_with_reference_scale_layouts(golden):
    t = golden("matmul_mx")
    M, K, N = t["m"], t["k"], t["n"]

    @pl.program
    class MatmulMx:
        @pl.function(type=pl.FunctionType.Orchestration)
        def orchestrator(self, a: pl.Tensor[[M, K], pl.FP8E4M3FN],
                         a_scale: pl.Tensor[[M, K // 32], pl.FP8E8M0, pl.MX_A_ZZ],
                         b: pl.Tensor[[K, N], pl.FP8E4M3FN],
                         b_scale: pl.Tensor[[K // 32, N], pl.FP8E8M0, pl.MX_B_NN],
                         out: pl.Out[pl.Tensor[[M, N], pl.FP32]],
                         out_acc: pl.Out[pl.Tensor[[M, N], pl.FP32]]):
            ...

    from pypto_b200 import ir
    compiled = ir.compile(MatmulMx, platform="b200")
    e8 = torch.float8_e8m0fnu
    out, out_acc = compiled(t["a"].view(torch.float8_e4m3fn), t["a_scale_packed"].view(e8),
                            t["b"].view(torch.float8_e4m3fn), t["b_scale_packed"].view(e8))     # return style
    assert torch.equal(out, t["out"]) and torch.equal(out_acc, t["out_acc"])      # rtol = atol = 0


def test_block_id_outside_the_pool_raises_through_the_launch_surface():
    """The device error word reaches the caller of ``compiled(...)``: a block id outside the pool is replaced by
    block 0 inside the kernel (no out-of-bounds read) and the call raises instead of returning a wrong output."""
    import oracle
    from pypto_b200 import PtoError, ir
    from pypto_b200.runtime import fused_programs
    d = oracle.inputs.paged_attention_inputs(batch=2, num_heads=8, kv_heads=2, ctx_lo=200, ctx_hi=300, seed=5)
    prog = fused_programs.paged_attention_program(d["batch"], d["num_heads"], d["head_dim"], d["block_size"],
                                                  d["max_blocks"], kv_heads=d["kv_heads"], out_dtype=torch.float32)
    compiled = ir.compile(prog, platform="b200")
    out = torch.zeros(d["query"].shape, dtype=torch.float32)
    cfg = fused_programs.pack_config(d)
    args = [d["query"], d["key_cache"], d["value_cache"], d["block_table"].flatten().clone(), d["context_lens"], out, cfg]
    compiled(*args)                                        # a clean call passes
    args[3][0] = d["pool_blocks"] + 7
    with pytest.raises(PtoError, match="block id"):
        compiled(*args)
    compiled(*[a if i != 3 else d["block_table"].flatten() for i, a in enumerate(args)])      # and the word was cleared


def test_llama_mini_program_matches_reference_fixture(golden):
    """``llama_mini_orch`` (examples/models/08_llama_mini.py:385-408) through ``run``: logits against the output of the
    reference's own golden, and a second size against the oracle."""
    from oracle import llama_mini as olm
    from pypto_b200.runtime import RunConfig, run

    def program(S, D, V):
        H = D // 2

        @pl.program
        class LlamaMiniProgram:
            @pl.function(type=pl.FunctionType.Orchestration)
            def llama_mini_orch(self, hidden: pl.Tensor[[S, D], pl.FP32], causal_mask: pl.Tensor[[S, S], pl.FP32],
                                cos_emb: pl.Tensor[[S, H], pl.FP32], sin_emb: pl.Tensor[[S, H], pl.FP32],
                                wq: pl.Tensor[[D, D], pl.FP32], wk: pl.Tensor[[D, D], pl.FP32],
                                wv: pl.Tensor[[D, D], pl.FP32], w_dense: pl.Tensor[[D, D], pl.FP32],
                                w_gate: pl.Tensor[[D, D], pl.FP32], w_up: pl.Tensor[[D, D], pl.FP32],
                                w_down: pl.Tensor[[D, D], pl.FP32], w_lm: pl.Tensor[[D, V], pl.FP32],
                                logits: pl.Out[pl.Tensor[[S, V], pl.FP32]]) -> pl.Tensor[[S, V], pl.FP32]:
                ...
        return LlamaMiniProgram

    names = ("hidden", "causal_mask", "cos_emb", "sin_emb", "wq", "wk", "wv", "w_dense", "w_gate", "w_up", "w_down", "w_lm")
    t = golden("llama_mini")
    out = torch.zeros(16, 64)
    run(program(16, 64, 64), *[t[n] for n in names], out, config=RunConfig(platform="b200"))
    assert torch.allclose(out, t["output"], rtol=1e-4, atol=1e-5), (out - t["output"]).abs().max()
    big = olm.make_inputs(seq_len=48, head_dim=128, vocab=320, seed=5)
    out2 = torch.zeros(48, 320)
    run(program(48, 128, 320), *[big[n] for n in names], out2, config=RunConfig(platform="b200"))
    exp2 = olm.forward(big)
    assert torch.allclose(out2, exp2, rtol=1e-4, atol=1e-5), (out2 - exp2).abs().max()


def test_traced_callable_reports_its_device_time():
    """Trace level 2 (``RunConfig(enable_pmu=1)``): the runtime brackets every callable with CUDA events and NVTX ranges;
    the result is unchanged and ``last_run_ms`` returns a plausible device time."""
    from pypto_b200 import _lib
    from pypto_b200.runtime import ChipWorker, DeviceTensor, RunConfig
    lib = _lib.load()
    before = lib.pto_get_trace()
    x = torch.randn(64, 4096, device="cuda").bfloat16()
    gamma = torch.rand(4096, device="cuda") + 0.5
    out = torch.zeros_like(x)
    try:
        with ChipWorker(RunConfig(platform="b200", enable_pmu=1)) as wk:
            assert lib.pto_get_trace() == 2
            dt = [DeviceTensor(t.data_ptr(), tuple(t.shape), t.dtype, buffer=t) for t in (x, gamma, out)]
            torch.cuda.synchronize()
            wk.launch("rms_norm", dt, [struct.unpack("I", struct.pack("f", 1e-5))[0]])
            ms = wk.last_run_ms()
            assert 0.0 < ms < 50.0
        exp = (x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-5) * gamma).bfloat16()
        assert torch.allclose(out.float(), exp.float(), rtol=2e-2, atol=2e-2)
    finally:
        lib.pto_set_trace(before)
