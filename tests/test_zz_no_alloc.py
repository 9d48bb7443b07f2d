"""The allocation-free paged-attention entry point (``pto_paged_attention_static``).

Engines that pre-commit all device memory, plugins inside a foreign allocator and
latency-critical loops cannot call cudaMalloc when they launch; this entry point keeps its
scratch in a fixed array inside the library.  The test drives it through the C ABI with raw
pointers and checks it against the oracle and against ``pto_paged_attention`` on two consecutive
calls with different inputs (the shared array keeps the first call's contents, so the second
call shows whether stale partial rows or a stale plan leak through).  Collected last so that a
failure here cannot hide the other tests in a stop-at-first-failure run.
"""

import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 4e-3   # the bar used by the other paged-attention GPU tests


def _call_both(d):
    from pypto_b200 import _lib, ops
    lib = _lib.load()
    g = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    ref = ops.paged_attention(g["query"], g["key_cache"], g["value_cache"], g["block_table"], g["context_lens"],
                              num_heads=d["num_heads"], kv_heads=d["kv_heads"], block_size=d["block_size"],
                              scale=d["scale"], q_len=d["q_len"], out_dtype=torch.float32)
    out = torch.full_like(ref, float("nan"))
    status = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    free_before = torch.cuda.mem_get_info()[0]
    _lib.check(lib.pto_paged_attention_static(
        g["query"].data_ptr(), g["key_cache"].data_ptr(), g["value_cache"].data_ptr(),
        g["block_table"].data_ptr(), g["context_lens"].data_ptr(), out.data_ptr(), _lib.PTO_FP32, d["batch"],
        d["num_heads"], d["kv_heads"], d["head_dim"], d["block_size"], d["max_blocks"], d["pool_blocks"],
        d["q_len"], d["scale"], status.data_ptr(), stream))
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free_before, "the call must not take device memory"
    assert status.tolist() == [0, 0, 0, 0]
    return out.cpu(), ref.cpu()


def test_static_scratch_entry_matches_allocating_entry_twice_in_a_row():
    first = oracle.inputs.paged_attention_inputs(batch=24, num_heads=32, kv_heads=8, ctx_lo=1, ctx_hi=3000, seed=31)
    second = oracle.inputs.paged_attention_inputs(batch=7, num_heads=16, kv_heads=2, ctx_lo=200, ctx_hi=5000,
                                                  q_len=2, seed=32)
    from oracle import paged_attention as opa
    for d in (first, second):
        got, ref = _call_both(d)
        assert torch.isfinite(got).all()
        exp = opa.paged_attention(d["query"], d["key_cache"], d["value_cache"], d["block_table"], d["context_lens"],
                                  num_heads=d["num_heads"], head_dim=d["head_dim"], block_size=d["block_size"],
                                  scale=d["scale"], kv_heads=d["kv_heads"], q_len=d.get("q_len", 1)).float()
        assert torch.allclose(got, exp.reshape(got.shape), rtol=RTOL, atol=ATOL), (got - exp.reshape(got.shape)).abs().max()
        assert torch.equal(got, ref)   # same kernels, same order of operations as the allocating entry


def test_static_scratch_rejects_geometry_beyond_its_capacity():
    from pypto_b200 import _lib
    lib = _lib.load()
    need = lib.pto_paged_attention_scratch_bytes(4096, 64, 8, 4)
    assert need > 32 << 20
    dummy = torch.zeros(64, dtype=torch.int32, device="cuda")
    rc = lib.pto_paged_attention_static(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(),
                                        dummy.data_ptr(), dummy.data_ptr(), _lib.PTO_BF16, 4096, 64, 8, 128, 128,
                                        8, 1024, 4, 1.0, None, None)
    assert rc == 1
    assert b"32" in lib.pto_last_error() or b"33554432" in lib.pto_last_error()
