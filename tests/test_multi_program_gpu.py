"""Two compiled programs on one worker sharing a resident paged KV cache: a prefill-side program
writes K/V rows into the cache, the decode program (the fused paged attention) reads it, then a
decode step appends one token per sequence and attention runs again.  The pattern of the
reference's examples/runtime/multi_program_kv_cache.py:101-140 (one worker, a DeviceTensor that
survives dispatches from different compiled programs), with real paged-attention arithmetic in
place of its add kernels.  The cache writer is an external kernel attached to its program."""

from pathlib import Path

import pytest
import torch

import oracle
import pypto_b200.language as pl
from oracle import paged_attention as opa
from pypto_b200 import ir
from pypto_b200.runtime import ChipWorker, RunConfig
from pypto_b200.runtime.fused_programs import pack_config, paged_attention_program

pytestmark = pytest.mark.gpu

_SRC = Path(__file__).parent / "extern_kernels" / "aiv" / "paged_kv_write.cu"
HEADS, D, BS = 16, 128, 128


def _writer_program(max_blocks):
    @pl.program
    class WriteKV:
        @pl.function(type=pl.FunctionType.AIV, external_source=_SRC, threads_per_block=64)
        def KV_WRITE(self, rows: pl.Tensor, pool: pl.InOut[pl.Tensor], block_table: pl.Tensor, start: pl.Tensor,
                     count: pl.Tensor, offset: pl.Tensor, block_size: pl.Scalar[pl.INDEX],
                     max_blocks: pl.Scalar[pl.INDEX], head_dim: pl.Scalar[pl.INDEX]) -> pl.Tensor: ...

        @pl.function(type=pl.FunctionType.Orchestration)
        def write_kv(self, k_rows: pl.Tensor, v_rows: pl.Tensor, key_cache: pl.InOut[pl.Tensor],
                     value_cache: pl.InOut[pl.Tensor], block_table: pl.Tensor, start: pl.Tensor, count: pl.Tensor,
                     offset: pl.Tensor):
            with pl.spmd(core_num=3):
                key_cache = self.KV_WRITE(k_rows, key_cache, block_table, start, count, offset, BS, max_blocks, D)
                value_cache = self.KV_WRITE(v_rows, value_cache, block_table, start, count, offset, BS, max_blocks, D)
            return key_cache
    return WriteKV


def _logical_rows(pool, bt, b, lo, hi):
    t = torch.arange(lo, hi)
    return pool[bt[b, t // BS].long() * BS + t % BS]


def test_prefill_and_decode_programs_share_a_resident_kv_cache():
    ctx = [512, 300, 1000, 129]
    d = oracle.inputs.paged_attention_inputs(num_heads=HEADS, kv_heads=1, head_dim=D, block_size=BS,
                                             context_lens=ctx, seed=3)
    bt, batch, max_blocks = d["block_table"], d["batch"], d["max_blocks"]
    writer = ir.compile(_writer_program(max_blocks), platform="b200")
    attention = ir.compile(paged_attention_program(batch, HEADS, D, BS, max_blocks, kv_heads=1), platform="b200")
    cfg_t = pack_config(d)

    def attend(w, kc, vc, lens):
        out = torch.zeros(batch * HEADS, D)
        w.run(attention, d["query"], kc, vc, bt.flatten(), lens, out, cfg_t)
        want = opa.paged_attention(d["query"], d["key_cache"], d["value_cache"], bt, lens, num_heads=HEADS,
                                   head_dim=D, block_size=BS, scale=d["scale"], kv_heads=1)
        assert (out - want).abs().max() <= 2e-2 * want.abs().max()

    def write(w, kc, vc, start, count):
        offset = torch.cumsum(count, 0, dtype=torch.int32) - count
        k_rows = torch.cat([_logical_rows(d["key_cache"], bt, b, int(start[b]), int(start[b] + count[b])) for b in range(batch)])
        v_rows = torch.cat([_logical_rows(d["value_cache"], bt, b, int(start[b]), int(start[b] + count[b])) for b in range(batch)])
        w.run(writer, k_rows, v_rows, kc, vc, bt.flatten(), start, count, offset)

    lens = torch.tensor(ctx, dtype=torch.int32)
    with ChipWorker(RunConfig(platform="b200")) as w:
        kc = w.alloc_tensor(d["key_cache"].shape, torch.bfloat16, init=torch.zeros_like(d["key_cache"]))
        vc = w.alloc_tensor(d["value_cache"].shape, torch.bfloat16, init=torch.zeros_like(d["value_cache"]))
        # prefill: everything but the last token of every sequence
        write(w, kc, vc, torch.zeros(batch, dtype=torch.int32), lens - 1)
        attend(w, kc, vc, lens - 1)
        # decode step: append the last token, attend over the full context
        write(w, kc, vc, lens - 1, torch.ones(batch, dtype=torch.int32))
        attend(w, kc, vc, lens)
        # the resident cache now holds exactly the logical rows, and nothing else was touched
        got = w.read_tensor(kc)
        for b in range(batch):
            assert torch.equal(_logical_rows(got, bt, b, 0, ctx[b]), _logical_rows(d["key_cache"], bt, b, 0, ctx[b]))
        used = torch.zeros(got.shape[0], dtype=torch.bool)
        for b in range(batch):
            t = torch.arange(ctx[b])
            used[bt[b, t // BS].long() * BS + t % BS] = True
        assert not got[~used].any()
