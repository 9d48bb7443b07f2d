"""GPU: the launch surface end to end -- run() with host tensors, ChipWorker memory calls,
resident DeviceTensors, the register-once benchmark loop."""

import pytest
import torch

import oracle
from oracle import paged_attention as opa
from pypto_b200.runtime import ChipWorker, RunConfig, benchmark, fused_programs, run, validate_golden

pytestmark = pytest.mark.gpu


def _case(**kw):
    d = oracle.inputs.paged_attention_inputs(**kw)
    exp = opa.paged_attention(d["query"], d["key_cache"], d["value_cache"], d["block_table"], d["context_lens"],
                              num_heads=d["num_heads"], head_dim=d["head_dim"], block_size=d["block_size"],
                              scale=d["scale"], kv_heads=d["kv_heads"], q_len=d["q_len"])
    prog = fused_programs.paged_attention_program(d["batch"], d["num_heads"], d["head_dim"], d["block_size"],
                                                  d["max_blocks"], kv_heads=d["kv_heads"], q_len=d["q_len"])
    return d, exp, prog


def test_run_with_host_tensors_matches_oracle():
    d, exp, prog = _case(batch=3, num_heads=32, kv_heads=8, ctx_lo=50, ctx_hi=900, seed=2)
    out = torch.zeros(d["query"].shape, dtype=torch.float32)
    compiled = run(prog, d["query"], d["key_cache"], d["value_cache"], d["block_table"].flatten(),
                   d["context_lens"], out, fused_programs.pack_config(d), config=RunConfig(platform="b200"))
    validate_golden({"out": out}, {"out": exp}, rtol=2e-2, atol=4e-3)
    # return style: output allocated and returned (compiled_program.py:559-655)
    out2 = compiled(d["query"], d["key_cache"], d["value_cache"], d["block_table"].flatten(),
                    d["context_lens"], fused_programs.pack_config(d))
    assert torch.equal(out, out2)


def test_reference_shaped_single_kv_head_fp32_out(golden):
    t = golden("pa04_unaligned")
    cfg = t["config"]
    prog = fused_programs.paged_attention_program(int(cfg[0]), int(cfg[1]), int(cfg[3]), int(cfg[4]), int(cfg[5]))
    out = torch.zeros_like(t["out"])
    run(prog, t["query"], t["key_cache"], t["value_cache"], t["block_table"], t["context_lens"], out, cfg)
    validate_golden({"out": out}, {"out": t["out"]}, rtol=2e-2, atol=4e-3)


def test_chip_worker_memory_and_resident_tensors():
    d, exp, prog = _case(batch=2, num_heads=16, kv_heads=2, ctx_lo=10, ctx_hi=400, seed=8)
    from pypto_b200 import ir
    compiled = ir.compile(prog, platform="b200")
    with ChipWorker(RunConfig(platform="b200")) as w:
        p = w.malloc(1024)
        host = torch.arange(256, dtype=torch.int32)
        w.copy_to(p, host, 1024)
        back = torch.zeros(256, dtype=torch.int32)
        w.copy_from(back, p, 1024)
        assert torch.equal(host, back)
        w.free(p)
        with pytest.raises(ValueError, match="double free"):
            w.free(p)
        kc = w.alloc_tensor(d["key_cache"].shape, torch.bfloat16, init=d["key_cache"])
        vc = w.alloc_tensor(d["value_cache"].shape, torch.bfloat16, init=d["value_cache"])
        with pytest.raises(ValueError):
            w.alloc_tensor((4,), torch.float32, init=torch.zeros(5))
        out = torch.zeros(d["query"].shape, dtype=torch.float32)
        handle = w.register(compiled)
        handle(d["query"], kc, vc, d["block_table"].flatten(), d["context_lens"], out, fused_programs.pack_config(d))
        validate_golden({"out": out}, {"out": exp}, rtol=2e-2, atol=4e-3)
        assert w.device_status()[0] == 0
        w.free_tensor(kc)
        with pytest.raises(ValueError, match="not a live allocation"):
            handle(d["query"], kc, vc, d["block_table"].flatten(), d["context_lens"], out, fused_programs.pack_config(d))
    assert handle.closed and not w.initialized
    w.close()  # idempotent
    with pytest.raises(RuntimeError):
        w.malloc(16)


def test_benchmark_register_once_loop():
    d, _exp, prog = _case(batch=4, num_heads=32, kv_heads=8, ctx_lo=500, ctx_hi=2000, seed=5)
    from pypto_b200 import ir
    compiled = ir.compile(prog, platform="b200")
    with ChipWorker(RunConfig(platform="b200")) as w:
        dev = [w.alloc_tensor(t.shape, t.dtype, init=t) for t in
               (d["query"], d["key_cache"], d["value_cache"], d["block_table"].flatten(), d["context_lens"])]
        out = w.alloc_tensor(d["query"].shape, torch.float32)
        stats = benchmark(compiled, (*dev, out, fused_programs.pack_config(d)), rounds=5, warmup=2, worker=w)
    assert stats.rounds == 5 and 0 < stats.min_us < 1e5
