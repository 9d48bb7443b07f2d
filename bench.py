"""Benchmarks of the fused-operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload decode|verify|ffn|layer|moe] [--kernel-only]

Default workload ``decode`` is the one the headline metric is quoted on: paged-attention
decode, batch 64 sequences per GPU, 32 query heads / 8 KV heads, head_dim 128, KV blocks of
128 tokens, q_len 1, context lengths uniform in [1024, 8192], block tables a random
permutation of a pool sized to need + 10 %, bf16 in / bf16 out, fp32 accumulation.  One step =
one pass of the hot path over one batch of synthetic input.  With N > 1 (torchrun, one rank
per GPU) every rank decodes its own sequences -- the path shards by batch with no collective.

Other workloads (same JSON schema, one line each):
  verify  speculative-verify attention: batch 256 in total split by batch over the ranks,
          q_len 4 causal, 64/8 heads, ctx U[8192, 32768]            (strong scaling)
  ffn     SwiGLU FFN x[128,1024] fp32, W N(0, 0.02^2), plus an M sweep  (replicas)
  layer   Llama-style decoder layer, decode step, batch 32, 4096-token paged caches (replicas)
  moe     DeepSeek-V3-shaped MoE layer, 4096 tokens, 256+1 experts FP8, top-8; expert-parallel
          over the ranks with NCCL all-to-all                        (strong scaling)

Prints ONE JSON line (rank 0).  ``value`` is device throughput with inputs resident in HBM
(CUDA events, max over ranks); ``e2e`` is the same metric through the public call with HOST
tensors, copies inside the timed region.  ``--impl reference`` times the CPU golden
restatement (``oracle/``) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

DECODE = dict(batch=64, num_heads=32, kv_heads=8, head_dim=128, block_size=128, ctx_lo=1024, ctx_hi=8192, q_len=1)
VERIFY = dict(batch=256, num_heads=64, kv_heads=8, head_dim=128, block_size=128, ctx_lo=8192, ctx_hi=32768, q_len=4)
LAYER = dict(batch=32, hidden=4096, num_heads=32, kv_heads=8, head_dim=128, inter=14336, ctx=4096)
FFN = dict(m=128, k=1024, inter=4096)
MOE = dict(tokens=4096, hidden=7168, inter=2048, n_experts=256, topk=8)

# dram bytes (read + write) of one launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (None where no capture exists yet)
NCU_TRAFFIC = {"decode": 1406460304,   # pa_decode_kernel<1>, profiles/pa_decode_kernel_decode_batch64_ctx1k-8k.md
               "verify": None,         # scaled from a batch-16 capture, see VERIFY_TRAFFIC_PER_KV_BYTE
               "ffn": 17104384 + 10026752,   # the two gemm_bf16_kernel launches of a step (gate/up + SwiGLU 17.1 MB, down 10.0 MB)
               "layer": 243135232,     # gate/up gemm_bf16_kernel launch (235.4 MB read + 7.7 MB written), profiles/gemm_bf16_*.md
               "moe": 499609856 * 16}  # gate/up moe_gemm_fp8_kernel: 489.7 MB read + 9.9 MB written on the 16-expert capture, x16 for 256 experts


# pa_decode_kernel<2> on `--workload verify --small` (batch 16): 1.2221 GB read + 12.4 MB written for 1.2157 GB of
# K/V that the step must read; traffic grows in proportion to the K/V bytes, so a full launch is scaled by them.
VERIFY_TRAFFIC_PER_KV_BYTE = (1222118000 + 12380416) / 1215746048


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return dict(hbm=float(d["hbm_gbs"]), bf16=float(d["bf16_tflops"]),
                    bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    source="measured (MEASURED_PEAKS.json)")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback (earlier measurement on this pool)")


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read only)."""

    _NAMES = {0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x10: "sync_boost",
              0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int, period: float = 0.002):
        self.index, self.period = index, period
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop, self._thread, self.active = threading.Event(), None, False

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def sample_now(self):
        """One sample from the calling thread (the timed region of a short run can be shorter than the
        sampling period; the caller takes this sample while the queued steps are still executing)."""
        if self._thread is None:
            return
        try:
            nv = self.nv
            self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
            mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
            self.reasons.update(n for b, n in self._NAMES.items() if mask & b)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            if self.active:
                self.sample_now()
            time.sleep(self.period)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


class Dist:
    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        self.dev = None

    def init(self):
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
        return self

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(device_ids=[self.local])
        torch.cuda.synchronize()

    def reduce(self, values, op):
        t = torch.tensor(values, dtype=torch.float64, device=self.dev)
        if self.world > 1:
            import torch.distributed as dist
            dist.all_reduce(t, op=getattr(dist.ReduceOp, op))
        return t.tolist()

    def close(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


def timed(step, d: Dist, steps: int, warmup: int):
    """W warm-up steps, barrier + synchronize, K steps between CUDA events on the current
    stream, synchronize.  Returns (ms of the K steps on this rank, clock record)."""
    sampler = ClockSampler(d.local).start()
    for _ in range(max(warmup, 3)):
        step()
    d.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.active = True
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    sampler.sample_now()           # the steps above are queued and still running
    torch.cuda.synchronize()
    sampler.active = False
    d.barrier()
    return e0.elapsed_time(e1), sampler.stop()


def graphed(step):
    """Capture one step into a CUDA graph (launch-bound chains of small kernels)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            step()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    return g.replay


def wall(fn, n):
    fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n):
        fn()
    torch.cuda.synchronize()
    return (time.perf_counter() - t0) / n


def emit(args, d: Dist, *, metric, unit, value, sec_per_step, scaling, dtype, config, launches, clocks, roofline,
         cpu_baseline, e2e, extra=None):
    line = {"metric": metric, "value": value, "unit": unit, "n_gpus": d.world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": config,
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu_baseline,
            "e2e": e2e}
    line.update(extra or {})
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------
# paged attention: decode (headline) and verify
# --------------------------------------------------------------------------------------

def paged_inputs_device(dev, seed, batch, num_heads, kv_heads, head_dim, block_size, ctx_lo, ctx_hi, q_len):
    """Same shapes and distributions as oracle.inputs.paged_attention_inputs, drawn on the
    device (the verify pool is tens of GB: drawing it on the host would take minutes)."""
    g = torch.Generator().manual_seed(seed)
    ctx = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=g, dtype=torch.int32)
    n_blk = (ctx.long() + block_size - 1) // block_size
    pool_blocks = max(1, math.ceil(int(n_blk.sum()) * 1.10))
    max_blocks = int(n_blk.max())
    perm = torch.randperm(pool_blocks, generator=g).to(torch.int32)
    bt = torch.zeros(batch, max_blocks, dtype=torch.int32)
    o = 0
    for b in range(batch):
        nb = int(n_blk[b])
        bt[b, :nb] = perm[o:o + nb]
        o += nb
    gd = torch.Generator(device=dev).manual_seed(seed)
    rows = pool_blocks * kv_heads * block_size
    kc = torch.empty(rows, head_dim, dtype=torch.bfloat16, device=dev)
    vc = torch.empty(rows, head_dim, dtype=torch.bfloat16, device=dev)
    chunk = 1 << 22
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        kc[r0:r1] = torch.randn(r1 - r0, head_dim, device=dev, generator=gd).bfloat16()
        vc[r0:r1] = torch.randn(r1 - r0, head_dim, device=dev, generator=gd).bfloat16()
    q = torch.randn(batch * q_len * num_heads, head_dim, device=dev, generator=gd).bfloat16()
    return dict(query=q, key_cache=kc, value_cache=vc, block_table=bt.to(dev), context_lens=ctx.to(dev),
                scale=1.0 / math.sqrt(head_dim), batch=batch, num_heads=num_heads, kv_heads=kv_heads,
                head_dim=head_dim, block_size=block_size, q_len=q_len, pool_blocks=pool_blocks, max_blocks=max_blocks)


def attn_bytes(d):
    kv = int(d["context_lens"].long().sum().item()) * d["kv_heads"] * d["head_dim"] * 2 * 2
    extra = d["query"].numel() * 2 * 2 + d["block_table"].numel() * 4 + d["context_lens"].numel() * 4
    return kv, kv + extra


def host_subproblem(d, n_seq):
    """First n_seq sequences with their KV blocks compacted into a small host pool."""
    bt = d["block_table"][:n_seq].cpu()
    ctx = d["context_lens"][:n_seq].cpu()
    bs, kvh, hd = d["block_size"], d["kv_heads"], d["head_dim"]
    n_blk = (ctx.long() + bs - 1) // bs
    used = torch.cat([bt[b, :int(n_blk[b])] for b in range(n_seq)]).long()
    remap = torch.zeros(d["pool_blocks"], dtype=torch.int32)
    remap[used] = torch.arange(used.numel(), dtype=torch.int32)
    sel = used.to(d["key_cache"].device)
    kc = d["key_cache"].view(-1, kvh * bs, hd)[sel].reshape(-1, hd).cpu()
    vc = d["value_cache"].view(-1, kvh * bs, hd)[sel].reshape(-1, hd).cpu()
    rows = n_seq * d["q_len"] * d["num_heads"]
    sub = dict(d)
    sub.update(query=d["query"][:rows].cpu(), key_cache=kc, value_cache=vc, block_table=remap[bt.long()],
               context_lens=ctx, batch=n_seq, pool_blocks=int(used.numel()))
    return sub


def cpu_attention(sub, repeats=1):
    from oracle import paged_attention as opa

    def once():
        return opa.paged_attention(sub["query"], sub["key_cache"], sub["value_cache"], sub["block_table"],
                                   sub["context_lens"], num_heads=sub["num_heads"], head_dim=sub["head_dim"],
                                   block_size=sub["block_size"], scale=sub["scale"], kv_heads=sub["kv_heads"],
                                   q_len=sub["q_len"])
    once()
    t0 = time.perf_counter()
    for _ in range(repeats):
        once()
    dt = (time.perf_counter() - t0) / repeats
    return dt, opa.kv_bytes(sub["context_lens"], sub["kv_heads"], sub["head_dim"])


def run_attention(args, d: Dist, which: str):
    from pypto_b200 import ir, ops
    from pypto_b200.runtime import ChipWorker, RunConfig, fused_programs
    pk = peaks()
    if which == "decode":
        from oracle import inputs
        host = inputs.paged_attention_inputs(seed=d.rank, **DECODE)     # every rank decodes its own sequences
        g = {k: (v.to(d.dev) if isinstance(v, torch.Tensor) else v) for k, v in host.items()}
        scaling, metric = "weak", "paged_attn_decode_GBps"
        desc = "paged_attention_decode batch64/GPU hq32 hkv8 d128 block128 ctx U[1024,8192] q_len1"
    else:
        w = dict(VERIFY)
        assert w["batch"] % d.world == 0
        w["batch"] //= d.world                                           # strong scaling: split by batch
        g = paged_inputs_device(d.dev, 100 + d.rank, **w)
        host = None
        scaling, metric = "strong", "paged_attn_verify_GBps"
        desc = (f"speculative_verify batch{VERIFY['batch']} total ({w['batch']}/GPU) q_len4 causal hq64 hkv8 d128 "
                "block128 ctx U[8192,32768]")
    out = torch.empty(g["query"].shape, dtype=torch.bfloat16, device=d.dev)
    kw = dict(num_heads=g["num_heads"], kv_heads=g["kv_heads"], head_dim=g["head_dim"], block_size=g["block_size"],
              scale=g["scale"], q_len=g["q_len"])

    def step():
        ops.paged_attention(g["query"], g["key_cache"], g["value_cache"], g["block_table"], g["context_lens"],
                            out=out, **kw)

    ms, clocks = timed(step, d, args.steps, args.warmup)
    ops.check_device_status()
    kv_b, alg_b = attn_bytes(g)
    ms_max, = d.reduce([ms], "MAX")
    tot_b, tot_seq = d.reduce([float(alg_b), float(g["batch"])], "SUM")
    sec = ms_max / 1e3 / args.steps
    value = tot_b / sec / 1e9

    e2e = cpu = None
    if not args.kernel_only:
        small = {k: g[k].cpu().pin_memory() for k in ("query", "block_table", "context_lens")}
        host_out = torch.empty(g["query"].shape, dtype=torch.bfloat16).pin_memory()
        small_b = sum(t.numel() * t.element_size() for t in small.values())
        if which == "decode":
            # the launch surface with HOST tensors: every input (KV pools included) copied per call
            prog = fused_programs.paged_attention_program(g["batch"], g["num_heads"], g["head_dim"], g["block_size"],
                                                          g["max_blocks"], kv_heads=g["kv_heads"], q_len=g["q_len"],
                                                          out_dtype=torch.bfloat16)
            compiled = ir.compile(prog, platform="b200")
            cfg_t = fused_programs.pack_config(g)
            pinned = {k: host[k].pin_memory() for k in ("key_cache", "value_cache")}
            a = (small["query"], pinned["key_cache"], pinned["value_cache"], small["block_table"].flatten(),
                 small["context_lens"], host_out, cfg_t)
            run_cfg = RunConfig(platform="b200", device_id=d.local)
            all_sec, = d.reduce([wall(lambda: compiled(*a, config=run_cfg), 3)], "MAX")
            # resident variant: pools live on the worker as DeviceTensors, registered handle
            with ChipWorker(run_cfg) as wk:
                kc = wk.alloc_tensor(tuple(host["key_cache"].shape), torch.bfloat16, init=host["key_cache"])
                vc = wk.alloc_tensor(tuple(host["value_cache"].shape), torch.bfloat16, init=host["value_cache"])
                handle = wk.register(compiled)
                b = (small["query"], kc, vc, small["block_table"].flatten(), small["context_lens"], host_out, cfg_t)
                res_sec = wall(lambda: handle(*b), 50)
            res_sec, = d.reduce([res_sec], "MAX")
            e2e = {"value": tot_b / all_sec / 1e9, "unit": "GB/s",
                   "h2d_bytes_per_step": small_b + cfg_t.numel() * 8 + 2 * host["key_cache"].numel() * 2,
                   "d2h_bytes_per_step": host_out.numel() * 2,
                   "note": "CompiledProgram call with every tensor on the host, KV pools included (PCIe-bound)",
                   "resident_kv_cache_value": tot_b / res_sec / 1e9}
        else:
            def call():
                q = small["query"].to(d.dev, non_blocking=True)
                bt = small["block_table"].to(d.dev, non_blocking=True)
                cl = small["context_lens"].to(d.dev, non_blocking=True)
                o = ops.paged_attention(q, g["key_cache"], g["value_cache"], bt, cl, **kw)
                host_out.copy_(o, non_blocking=True)
                torch.cuda.synchronize()
            res_sec, = d.reduce([wall(call, 10)], "MAX")
            e2e = {"value": tot_b / res_sec / 1e9, "unit": "GB/s", "h2d_bytes_per_step": small_b,
                   "d2h_bytes_per_step": host_out.numel() * 2,
                   "note": "pypto_b200.ops.paged_attention with the KV pools resident (tens of GB); query, tables, "
                           "lengths from pinned host memory and the output back every step"}
        if d.rank == 0:
            n_seq = g["batch"] if which == "decode" else 2
            sub = host if which == "decode" else host_subproblem(g, n_seq)
            cdt, cb = cpu_attention(sub, repeats=3 if which == "decode" else 1)
            cpu = {"value": cb / cdt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": f"{n_seq} of {g['batch']} sequences of rank 0, torch CPU oracle",
                   "host_cpus": os.cpu_count()}
    if d.rank == 0:
        achieved = alg_b / (ms / 1e3 / args.steps) / 1e9
        emit(args, d, metric=metric, unit="GB/s", value=value, sec_per_step=sec, scaling=scaling, dtype="bf16",
             config={"workload": desc, "l2": "inputs larger than L2", "kv_bytes_per_step_per_gpu": kv_b},
             launches=2 * args.steps, clocks=clocks,
             roofline={"bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                       "frac": achieved / pk["hbm"],
                       "traffic": NCU_TRAFFIC[which] if which == "decode" else int(VERIFY_TRAFFIC_PER_KV_BYTE * kv_b),
                       "peak_source": pk["source"],
                       "note": "algorithmic bytes of one step / CUDA-event time of the step (pa_decode_kernel + "
                               "pa_merge_kernel), rank 0"},
             cpu_baseline=cpu, e2e=e2e, extra={"tokens_per_s": tot_seq * g["q_len"] / sec})


# --------------------------------------------------------------------------------------
# SwiGLU FFN
# --------------------------------------------------------------------------------------

def run_ffn(args, d: Dist):
    from oracle import ffn as offn
    from oracle import inputs
    from pypto_b200 import ops
    from pypto_b200.layers import SwiGLUFFN
    pk = peaks()
    m, k, inter = FFN["m"], FFN["k"], FFN["inter"]
    x, wg, wu, wd = inputs.ffn_inputs(m, k, inter, seed=0)
    copies = 8    # 8 x 25 MB of packed weights > L2: rotating them keeps the step HBM-bound
    ffns = [SwiGLUFFN(wg.to(d.dev), wu.to(d.dev), wd.to(d.dev)) for _ in range(copies)]
    xd = x.to(d.dev)
    out = torch.empty(m, k, dtype=torch.float32, device=d.dev)
    replays = [graphed(lambda f=f: f(xd, out=out)) for f in ffns]
    i = [0]

    def step():
        replays[i[0] % copies]()
        i[0] += 1

    ms, clocks = timed(step, d, args.steps, args.warmup)
    ops.check_device_status()
    ms_max, = d.reduce([ms], "MAX")
    sec = ms_max / 1e3 / args.steps
    flops = offn.ffn_flops(m, k, inter)
    alg_b = 3 * k * inter * 2 + m * k * 4 * 2        # packed bf16 weights + fp32 x and y
    sweep = []
    e2e = cpu = None
    if not args.kernel_only:
        if d.rank == 0:
            for ms_ in (128, 512, 2048, 8192):
                xs = torch.randn(ms_, k, device=d.dev).bfloat16()
                o = torch.empty(ms_, k, dtype=torch.float32, device=d.dev)
                j = [0]

                def st():
                    ffns[j[0] % copies](xs, out=o)
                    j[0] += 1
                for _ in range(3):
                    st()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                for _ in range(20):
                    st()
                e1.record()
                torch.cuda.synchronize()
                t = e0.elapsed_time(e1) / 20 / 1e3
                tf = offn.ffn_flops(ms_, k, inter) / t / 1e12
                sweep.append({"M": ms_, "K": k, "I": inter, "us": t * 1e6, "tflops": tf, "frac_bf16_peak": tf / pk["bf16"]})
            # the decoder layer's FFN shape (hidden 4096, intermediate 14336) at prefill size
            gk, gi, gm = LAYER["hidden"], LAYER["inter"], 8192
            gen = torch.Generator(device=d.dev).manual_seed(1)
            big = SwiGLUFFN(*[(torch.randn(a, b, device=d.dev, generator=gen) * 0.02).bfloat16()
                              for a, b in ((gk, gi), (gk, gi), (gi, gk))])
            xs = torch.randn(gm, gk, device=d.dev, generator=gen).bfloat16()
            o = torch.empty(gm, gk, dtype=torch.float32, device=d.dev)
            for _ in range(3):
                big(xs, out=o)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                big(xs, out=o)
            e1.record()
            torch.cuda.synchronize()
            t = e0.elapsed_time(e1) / 10 / 1e3
            tf = offn.ffn_flops(gm, gk, gi) / t / 1e12
            sweep.append({"M": gm, "K": gk, "I": gi, "us": t * 1e6, "tflops": tf, "frac_bf16_peak": tf / pk["bf16"]})
            del big, xs, o
        xh, yh = x.pin_memory(), torch.empty(m, k).pin_memory()

        def call():
            y = ffns[0](xh.to(d.dev, non_blocking=True))
            yh.copy_(y, non_blocking=True)
            torch.cuda.synchronize()
        e2e_sec, = d.reduce([wall(call, 50)], "MAX")
        e2e = {"value": d.world * flops / e2e_sec / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": m * k * 4,
               "d2h_bytes_per_step": m * k * 4,
               "note": "x from pinned host memory, y back to the host; packed weights resident; eager launches"}
        if d.rank == 0:
            offn.ffn_swiglu(x, wg, wu, wd)
            t0 = time.perf_counter()
            for _ in range(20):
                offn.ffn_swiglu(x, wg, wu, wd)
            cdt = (time.perf_counter() - t0) / 20
            cpu = {"value": flops / cdt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": "the full fp32 workload, mean of 20 passes, torch CPU oracle"}
    if d.rank == 0:
        t_rank = ms / 1e3 / args.steps
        emit(args, d, metric="ffn_swiglu_TFLOPs", unit="TFLOP/s", value=d.world * flops / sec / 1e12,
             sec_per_step=sec, scaling="weak", dtype="bf16",
             config={"workload": "swiglu_ffn x[128,1024] fp32 N(0,1), W N(0,0.02^2), bf16 operands fp32 accumulate",
                     "l2": "8 packed weight copies (201 MB) rotated between steps", "parallelism": "replicas only",
                     "launch": "CUDA graph of cast + gate/up GEMM + SwiGLU + down GEMM"},
             launches=5 * args.steps, clocks=clocks,
             roofline={"bound": "hbm", "achieved": alg_b / t_rank / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                       "frac": alg_b / t_rank / 1e9 / pk["hbm"], "traffic": NCU_TRAFFIC["ffn"],
                       "peak_source": pk["source"],
                       "note": "M = 128 is below the ridge (AI 124 FLOP/B): weight-bandwidth bound; the M sweep "
                               "shows the tensor-bound side against the measured bf16 burst peak"},
             cpu_baseline=cpu, e2e=e2e, extra={"sweep": sweep, "tflops_at_M128": flops / t_rank / 1e12})


# --------------------------------------------------------------------------------------
# decoder layer
# --------------------------------------------------------------------------------------

def run_layer(args, d: Dist):
    from oracle import inputs
    from oracle import layer as olayer
    from pypto_b200 import ops
    from pypto_b200.layers import DecoderLayer
    pk = peaks()
    t, geom = inputs.decoder_layer_inputs(**LAYER)
    dev_t = {k: v.to(d.dev) for k, v in t.items()}
    layer = DecoderLayer(dev_t, **geom)
    a = (dev_t["hidden"], dev_t["seq_lens"], dev_t["block_table"], dev_t["k_cache"], dev_t["v_cache"])
    keep = []
    replay = graphed(lambda: keep.append(layer.step(*a)))
    ms, clocks = timed(replay, d, args.steps, args.warmup)
    ops.check_device_status()
    ms_max, = d.reduce([ms], "MAX")
    sec = ms_max / 1e3 / args.steps
    alg_b = layer.weight_bytes() + LAYER["batch"] * LAYER["ctx"] * geom["kv_heads"] * geom["head_dim"] * 2 * 2
    e2e = cpu = None
    if not args.kernel_only:
        hh = t["hidden"].pin_memory()
        oh = torch.empty_like(t["hidden"]).pin_memory()

        def call():
            y = layer.step(hh.to(d.dev, non_blocking=True), *a[1:])
            oh.copy_(y, non_blocking=True)
            torch.cuda.synchronize()
        e2e_sec, = d.reduce([wall(call, 30)], "MAX")
        e2e = {"value": d.world * alg_b / e2e_sec / 1e9, "unit": "GB/s", "h2d_bytes_per_step": hh.numel() * 2,
               "d2h_bytes_per_step": oh.numel() * 2,
               "note": "hidden states from pinned host memory, output back; weights and KV cache resident; "
                       "eager launches"}
        if d.rank == 0:
            ref = {k: (v.clone() if isinstance(v, torch.Tensor) else v) for k, v in t.items()}
            t0 = time.perf_counter()
            olayer.decoder_layer(ref, **geom)
            cdt = time.perf_counter() - t0
            cpu = {"value": alg_b / cdt / 1e9, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                   "sample": "the full layer once, torch CPU oracle"}
    if d.rank == 0:
        t_rank = ms / 1e3 / args.steps
        emit(args, d, metric="decoder_layer_GBps", unit="GB/s", value=d.world * alg_b / sec / 1e9, sec_per_step=sec,
             scaling="weak", dtype="bf16",
             config={"workload": "llama_decoder_layer decode batch32 hidden4096 hq32 hkv8 d128 ffn14336 ctx4096 "
                                 "block128", "l2": "weights + KV (973 MB) larger than L2",
                     "parallelism": "replicas only", "launch": "one CUDA graph of the layer's kernels"},
             launches=14 * args.steps, clocks=clocks,
             roofline={"bound": "hbm", "achieved": alg_b / t_rank / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                       "frac": alg_b / t_rank / 1e9 / pk["hbm"], "traffic": NCU_TRAFFIC["layer"],
                       "peak_source": pk["source"], "note": "packed bf16 weights + visible KV rows, whole layer"},
             cpu_baseline=cpu, e2e=e2e, extra={"tokens_per_s": d.world * LAYER["batch"] / sec})


# --------------------------------------------------------------------------------------
# MoE
# --------------------------------------------------------------------------------------

def synthetic_experts(dev, gen, e, hidden, inter, w_std=0.02):
    """Random expert weights N(0, w_std^2) quantised to e4m3 with one fp32 scale per 128x128
    block, produced on the device directly in the GEMM's K-major layout."""
    def qw(n, k):
        out = torch.empty(e, n, k, dtype=torch.float8_e4m3fn, device=dev)
        sc = torch.empty(e, n // 128, k // 128, device=dev)
        for i in range(e):
            w = torch.randn(n, k, device=dev, generator=gen) * w_std
            b = w.view(n // 128, 128, k // 128, 128)
            s = b.abs().amax(dim=(1, 3)) / 448.0
            out[i] = (b / s[:, None, :, None]).view(n, k).to(torch.float8_e4m3fn)
            sc[i] = s
        return out, sc
    w_gu, s_gu = qw(2 * inter, hidden)
    w_d, s_d = qw(hidden, inter)
    return dict(w_gu=w_gu, s_gu=s_gu, w_d=w_d, s_d=s_d)


def run_moe(args, d: Dist):
    from oracle import moe as omoe
    from pypto_b200 import ops
    from pypto_b200.comm import Communicator
    from pypto_b200.moe import MoELayer
    pk = peaks()
    T, H, I, E, K = MOE["tokens"], MOE["hidden"], MOE["inter"], MOE["n_experts"], MOE["topk"]
    L, tl = E // d.world, T // d.world
    gen = torch.Generator(device=d.dev).manual_seed(d.rank)
    gshared = torch.Generator(device=d.dev).manual_seed(12345)       # replicated pieces: same on all ranks
    gate_w = (torch.randn(H, E, device=d.dev, generator=gshared) * 0.02).bfloat16()
    bias = torch.rand(E, device=d.dev, generator=gshared) * 0.2 - 0.1
    comm = Communicator.from_torch_distributed(device=d.local) if d.world > 1 else None
    layer = MoELayer.from_packed(ops.pack_weight(gate_w), bias, synthetic_experts(d.dev, gen, L, H, I),
                                 synthetic_experts(d.dev, gshared, 1, H, I), K, n_experts=E, comm=comm)
    x = torch.randn(tl, H, device=d.dev, generator=gen).bfloat16()

    ms, clocks = timed(lambda: layer.forward(x), d, args.steps, args.warmup)
    ops.check_device_status()
    ms_max, = d.reduce([ms], "MAX")
    sec = ms_max / 1e3 / args.steps
    flops = omoe.moe_flops(T, H, I, E, K)
    w_bytes = sum(v.numel() * v.element_size() for v in layer.routed.values()) + \
        sum(v.numel() * v.element_size() for v in layer.shared.values())
    e2e = cpu = None
    if not args.kernel_only:
        xh = x.cpu().pin_memory()
        yh = torch.empty_like(xh).pin_memory()

        def call():
            y, _, _ = layer.forward(xh.to(d.dev, non_blocking=True))
            yh.copy_(y, non_blocking=True)
            torch.cuda.synchronize()
        e2e_sec, = d.reduce([wall(call, 5)], "MAX")
        e2e = {"value": flops / e2e_sec / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": xh.numel() * 2,
               "d2h_bytes_per_step": yh.numel() * 2,
               "note": "tokens from pinned host memory, layer output back; expert weights resident"}
        if d.rank == 0:
            # CPU arm on a bounded sample: 2 routed experts x 128 tokens each through the oracle's FP8 FFN
            from oracle import inputs
            mo = inputs.moe_inputs(tokens=256, hidden=H, inter=I, n_experts=2, topk=1, shared=False, seed=0)
            xq, xs = omoe.quantize_rows(mo["x"])
            t0 = time.perf_counter()
            for e in range(2):
                omoe.expert_ffn(xq[e * 128:(e + 1) * 128], xs[e * 128:(e + 1) * 128],
                                omoe.expert_slice(mo["routed"], e))
            cdt = time.perf_counter() - t0
            cpu = {"value": 2 * 128 * 6 * H * I / cdt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                   "kind": "port",
                   "sample": "2 of 257 experts x 128 tokens each, torch CPU oracle (FP8 block-scaled FFN)"}
    if d.rank == 0:
        t_rank = ms / 1e3 / args.steps
        emit(args, d, metric="moe_layer_TFLOPs", unit="TFLOP/s", value=flops / sec / 1e12, sec_per_step=sec,
             scaling="strong", dtype="fp8_e4m3",
             config={"workload": f"deepseek_v3_moe tokens{T} hidden7168 experts{E}+1 inter2048 top8 fp8 block128; "
                                 f"{L} routed experts and {tl} tokens per GPU",
                     "l2": f"expert weights per GPU {w_bytes / 1e9:.2f} GB, larger than L2",
                     "parallelism": f"ep{d.world}" if d.world > 1 else "single GPU, all experts local"},
             launches=16 * args.steps, clocks=clocks,
             roofline={"bound": "hbm", "achieved": w_bytes / t_rank / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                       "frac": w_bytes / t_rank / 1e9 / pk["hbm"], "traffic": NCU_TRAFFIC["moe"],
                       "peak_source": pk["source"],
                       "note": "weight-bandwidth bound at ~128 tokens per expert: expert weight bytes of this GPU / "
                               "time of the whole layer step"},
             cpu_baseline=cpu, e2e=e2e, extra={"tokens_per_s": T / sec})


# --------------------------------------------------------------------------------------
# CPU arm
# --------------------------------------------------------------------------------------

def run_reference(args):
    """The oracle (a port of the reference's torch golden) on the host cores, all threads."""
    d = Dist()
    if d.rank != 0:
        return
    if args.workload != "decode":
        print(json.dumps({"impl": "reference", "unavailable":
                          f"the CPU arm is implemented for the headline workload (decode); '{args.workload}' reports "
                          "its cpu_baseline inside the main line"}), flush=True)
        return
    from oracle import inputs
    host = inputs.paged_attention_inputs(seed=0, **DECODE)
    times = []
    for i in range(args.warmup + args.steps):
        dt, nbytes = cpu_attention(host)
        if i >= args.warmup:
            times.append(dt)
    dt = sum(times) / len(times)
    value = nbytes / dt / 1e9
    line = {"impl": "reference", "metric": "paged_attn_decode_GBps", "value": value, "unit": "GB/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "paged_attention_decode batch64 hq32 hkv8 d128 block128 ctx U[1024,8192] q_len1"},
            "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                             "sample": "64 of 64 sequences per step (all 8 KV heads), torch CPU oracle"},
            "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "tokens_per_s": DECODE["batch"] / dt}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode", "verify", "ffn", "layer", "moe"])
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end and CPU legs (profiler captures)")
    ap.add_argument("--small", action="store_true",
                    help="reduced case of the workload for profiler captures (a few GB on the device at most): "
                         "verify batch 16, moe 16 experts / 256 tokens; other workloads unchanged")
    args = ap.parse_args()
    if args.impl == "reference":
        args.steps = min(args.steps or 5, 5)      # each step is about a second of CPU work
        args.warmup = min(args.warmup, 1)
        run_reference(args)
        return
    if args.steps is None:
        args.steps = {"decode": 1000, "verify": 50, "ffn": 2000, "layer": 500, "moe": 20}[args.workload]
    if args.small:
        VERIFY.update(batch=16)
        MOE.update(tokens=256, n_experts=16)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    d = Dist().init()
    try:
        if args.workload in ("decode", "verify"):
            run_attention(args, d, args.workload)
        elif args.workload == "ffn":
            run_ffn(args, d)
        elif args.workload == "layer":
            run_layer(args, d)
        else:
            run_moe(args, d)
    finally:
        d.close()


if __name__ == "__main__":
    main()
