"""Benchmarks of the fused-operator hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload all|decode|verify|ffn|layer|moe|matmul_mx] [--kernel-only] [--small]

The headline line (always printed, one JSON line on rank 0) is paged-attention decode: batch 64 sequences
per GPU, 32 query heads / 8 KV heads, head_dim 128, KV blocks of 128 tokens, q_len 1, context lengths uniform
in [1024, 8192] (the same lengths on every rank, different values), block tables a random permutation of a
pool sized to need + 10 %, bf16 in / bf16 out, fp32 accumulation.  One step = one pass of the hot path over
one batch of synthetic input.  With N > 1 (torchrun, one rank per GPU) every rank decodes its own sequences:
the path shards by batch with no collective.

With ``--workload all`` (the default) the line also carries a ``workloads`` object with the other configs at
the same N, each with value / unit / ms_per_step / roofline / cpu_baseline / e2e:
  verify     speculative-verify attention: batch 256 in total split by batch over the ranks,
             q_len 4 causal, 64/8 heads, ctx U[8192, 32768]                 (strong scaling)
  moe        DeepSeek-V3-shaped MoE layer, 4096 tokens, 256+1 experts FP8, top-8; expert-parallel
             over the ranks, dispatch and combine through the library's NCCL communicator
             (strong scaling; per-phase times and, at N = 1, a token sweep)
  ffn        SwiGLU FFN x[128,1024] fp32, W N(0, 0.02^2), plus an M sweep   (replicas: N = 1 only)
  layer      Llama-style decoder layer, decode step, batch 32, 4096-token paged caches (N = 1 only)
  matmul_mx  MX block-scaled FP8 matmul 8192^3 on the hardware block-scale path (N = 1 only)
``--workload X`` prints X alone in the same schema (profiler captures use it with ``--kernel-only``).

``value`` is device throughput with inputs resident in HBM: W >= 3 warm-up steps, then rounds of exactly K
steps each between CUDA events, every round bracketed by a barrier and a synchronize; enough rounds for
0.3 s of device work, the median round reported, max over ranks.  ``e2e`` is the same metric through the
public call with HOST tensors, copies inside the timed region.  ``peaks`` holds what the roofline fractions
divide by: the driver-measured HBM and bf16 figures and, measured here, an fp8 tensor peak
(``torch._scaled_mm`` 8192^3, best of 10) and at N > 1 an all-to-all bandwidth.

``--impl reference`` times the CPU golden restatement (``oracle/``) of the headline workload on all host
threads; under torchrun only rank 0 works.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time
import traceback

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

DECODE = dict(batch=64, num_heads=32, kv_heads=8, head_dim=128, block_size=128, ctx_lo=1024, ctx_hi=8192, q_len=1)
VERIFY = dict(batch=256, num_heads=64, kv_heads=8, head_dim=128, block_size=128, ctx_lo=8192, ctx_hi=32768, q_len=4)
LAYER = dict(batch=32, hidden=4096, num_heads=32, kv_heads=8, head_dim=128, inter=14336, ctx=4096)
FFN = dict(m=128, k=1024, inter=4096)
MOE = dict(tokens=4096, hidden=7168, inter=2048, n_experts=256, topk=8)
MX = dict(m=8192, n=8192, k=8192)

DECODE_DESC = "paged_attention_decode batch64/GPU hq32 hkv8 d128 block128 ctx U[1024,8192] q_len1"
MIN_DEVICE_SECONDS = 0.3       # device work per measurement (rounds of K steps until this much has run)
DEFAULT_STEPS = {"decode": 200, "verify": 20, "ffn": 500, "layer": 200, "moe": 10, "matmul_mx": 10}

# DRAM bytes (read + write) of one launch of the dominant kernel, from single captures under the profiler of the
# same command with --kernel-only (a smaller case scaled by the units processed where the full size is too large
# to capture; None where no capture exists)
NCU_TRAFFIC = {"decode": 1406460304,            # pa_decode_kernel<1>
               "ffn": 26022144,                 # ffn_fused_kernel at M = 128 (the weights, read once)
               "layer": 240724480 + 6793216,    # gate/up gemm_bf16_kernel launch of the layer
               "moe": (488558848 + 9664768) * 16,   # gate/up moe_gemm_fp8_kernel, 16-expert capture x 16
               "matmul_mx": 260926464 + 238253312 + 4204032,    # matmul_mx_pair_kernel + mx_pack_scales_kernel at 8192^3
               "matmul_mx_one_cta": 359288320 + 232929024}     # matmul_mx_kernel (PTO_MX_PAIR=0) at 8192^3
# pa_decode_kernel<2> on `--workload verify --small` (batch 16): DRAM bytes per byte of K/V that the step reads
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
        self._comm = None

    def init(self):
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=self.dev)
        return self

    def comm(self):
        """The library's communicator (created once; torch.distributed only carries its 128-byte id)."""
        if self._comm is None and self.world > 1:
            from pypto_b200.comm import Communicator
            self._comm = Communicator.from_torch_distributed(device=self.local)
        return self._comm

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
        if self._comm is not None:
            self._comm.close()
        if self.world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


def timed(step, d: Dist, steps: int, warmup: int):
    """W warm-up steps; then rounds of exactly K steps between CUDA events on the current stream, each round
    bracketed by barrier + synchronize, until MIN_DEVICE_SECONDS of device work has run (3 rounds at least).
    Returns (ms of the median round on this rank, clock record, number of rounds)."""
    sampler = ClockSampler(d.local).start()
    for _ in range(max(warmup, 3)):
        step()
    rounds_ms = []
    total, target = 0.0, MIN_DEVICE_SECONDS * 1e3
    while len(rounds_ms) < 3 or (total < target and len(rounds_ms) < 200):
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
        ms = e0.elapsed_time(e1)
        # every rank must run the same number of rounds: decide on the slowest rank's time
        ms_all, = d.reduce([ms], "MAX")
        rounds_ms.append(ms)
        total += ms_all
    d.barrier()
    return statistics.median(rounds_ms), sampler.stop(), len(rounds_ms)


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


def event_time(fn, n, warm=3):
    """Seconds per call of fn over n calls (CUDA events, current stream)."""
    for _ in range(warm):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(n):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / n / 1e3


_measured: dict = {}


def fp8_peak_tflops(dev, refresh=False):
    """Dense FP8 tensor throughput of this GPU, measured the way the bf16 peak is: a library GEMM
    (``torch._scaled_mm`` e4m3 x e4m3 -> bf16, 8192^3), best of 10.  None if that call is unavailable.
    ``refresh`` measures again and keeps the LARGER figure: a burst measured right after seconds of power-capped work
    reads hundreds of TFLOP/s low, and a peak that is too low flatters every fraction taken of it."""
    if "fp8" in _measured and (not refresh or _measured["fp8"] is None):
        return _measured["fp8"]
    before = _measured.get("fp8")
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()       # column-major right operand
        one = torch.ones((), device=dev)

        def mm():
            return torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            mm()
        best = min(event_time(mm, 1, warm=0) for _ in range(10))
        _measured["fp8"] = max(2 * n ** 3 / best / 1e12, before or 0.0)
    except Exception:
        _measured["fp8"] = before
    return _measured["fp8"]


def all_to_all_gbs(d: Dist):
    """Bytes leaving one GPU per second in an equal-split all-to-all of 64 MiB per rank pair and direction, through
    the library's communicator (NCCL send/recv grouped into one launch); max time over ranks."""
    if d.world == 1:
        return None
    if "a2a" in _measured:
        return _measured["a2a"]
    per_peer = 64 << 20
    send = torch.empty(d.world * per_peer, dtype=torch.uint8, device=d.dev)
    recv = torch.empty_like(send)
    comm = d.comm()
    sec = event_time(lambda: comm.all_to_all(send, recv), 10)
    sec, = d.reduce([sec], "MAX")
    _measured["a2a"] = (d.world - 1) * per_peer / sec / 1e9
    return _measured["a2a"]


def line(args, d: Dist, *, metric, unit, value, sec_per_step, scaling, dtype, config, launches, clocks, roofline,
         cpu_baseline, e2e, extra=None):
    out = {"metric": metric, "value": value, "unit": unit, "n_gpus": d.world, "steps": args.steps_for[metric],
           "warmup": max(args.warmup, 3), "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
           "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic", "config": config,
           "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu_baseline,
           "e2e": e2e}
    out.update(extra or {})
    return out


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


def decode_inputs(seed):
    """The headline workload: context lengths from seed 0 (every rank draws the same lengths, so the ranks of a
    weak-scaling run carry equal work), block table and Q / K / V values from ``seed``."""
    from oracle import inputs
    g = torch.Generator().manual_seed(0)
    ctx = torch.randint(DECODE["ctx_lo"], DECODE["ctx_hi"] + 1, (DECODE["batch"],), generator=g, dtype=torch.int32)
    kw = {k: v for k, v in DECODE.items() if k not in ("batch", "ctx_lo", "ctx_hi")}
    return inputs.paged_attention_inputs(seed=seed, context_lens=ctx, **kw)


def run_attention(args, d: Dist, which: str):
    from pypto_b200 import ir, ops
    from pypto_b200.runtime import ChipWorker, RunConfig, fused_programs
    pk = peaks()
    steps = args.steps_for[which]
    if which == "decode":
        host = decode_inputs(seed=d.rank)
        g = {k: (v.to(d.dev) if isinstance(v, torch.Tensor) else v) for k, v in host.items()}
        scaling, metric, desc = "weak", "paged_attn_decode_GBps", DECODE_DESC
    else:
        w = dict(VERIFY)
        if w["batch"] % d.world:
            raise ValueError("the verify batch must divide evenly over the ranks")
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

    ms, clocks, rounds = timed(step, d, steps, args.warmup)
    ops.check_device_status()
    kv_b, alg_b = attn_bytes(g)
    ms_max, = d.reduce([ms], "MAX")
    tot_b, tot_seq = d.reduce([float(alg_b), float(g["batch"])], "SUM")
    sec = ms_max / 1e3 / steps
    value = tot_b / sec / 1e9
    rank_gbs = alg_b / (ms / 1e3 / steps) / 1e9
    gbs_min, = d.reduce([rank_gbs], "MIN")
    gbs_sum, = d.reduce([rank_gbs], "SUM")

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
                res_sec = wall(lambda: handle(*b), 100)
            res_sec, = d.reduce([res_sec], "MAX")
            e2e = {"value": tot_b / all_sec / 1e9, "unit": "GB/s",
                   "h2d_bytes_per_step": small_b + cfg_t.numel() * 8 + 2 * host["key_cache"].numel() * 2,
                   "d2h_bytes_per_step": host_out.numel() * 2,
                   "note": "CompiledProgram call with every tensor on the host, KV pools included (PCIe-bound)",
                   "resident_kv_cache_value": tot_b / res_sec / 1e9,
                   "resident_kv_cache_us_per_call": res_sec * 1e6}
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
    achieved = alg_b / (ms / 1e3 / steps) / 1e9
    return line(args, d, metric=metric, unit="GB/s", value=value, sec_per_step=sec, scaling=scaling, dtype="bf16",
                config={"workload": desc, "l2": "inputs larger than L2", "kv_bytes_per_step_per_gpu": kv_b,
                        "context_lengths": "the same on every rank" if which == "decode" else "per rank",
                        "rounds": rounds},
                launches=2 * steps, clocks=clocks,
                roofline={"bound": "hbm", "achieved": achieved, "peak": pk["hbm"], "unit": "GB/s",
                          "frac": achieved / pk["hbm"],
                          "traffic": NCU_TRAFFIC[which] if which == "decode" else int(VERIFY_TRAFFIC_PER_KV_BYTE * kv_b),
                          "peak_source": pk["source"],
                          "note": "algorithmic bytes of one step / CUDA-event time of the step (pa_decode_kernel + "
                                  "pa_merge_kernel), rank 0"},
                cpu_baseline=cpu, e2e=e2e,
                extra={"tokens_per_s": tot_seq * g["q_len"] / sec,
                       "per_rank_GBps": {"min": gbs_min, "mean": gbs_sum / d.world}})


# --------------------------------------------------------------------------------------
# SwiGLU FFN
# --------------------------------------------------------------------------------------

def run_ffn(args, d: Dist):
    from oracle import ffn as offn
    from oracle import inputs
    from pypto_b200 import ops
    from pypto_b200.layers import SwiGLUFFN
    pk = peaks()
    steps = args.steps_for["ffn"]
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

    ms, clocks, rounds = timed(step, d, steps, args.warmup)
    ops.check_device_status()
    ms_max, = d.reduce([ms], "MAX")
    sec = ms_max / 1e3 / steps
    flops = offn.ffn_flops(m, k, inter)
    alg_b = 3 * k * inter * 2 + m * k * 4 * 2        # packed bf16 weights + fp32 x and y
    sweep = []
    e2e = cpu = None
    if not args.kernel_only:
        if d.rank == 0:
            for ms_ in (128, 512, 2048, 8192):
                xs = torch.randn(ms_, k, device=d.dev).bfloat16()
                o = torch.empty(ms_, k, dtype=torch.float32, device=d.dev)
                reps = [graphed(lambda f=f: f(xs, out=o)) for f in ffns]   # graphs: eager launches would be timed
                j = [0]                                                     # instead of the kernels at small M

                def st():
                    reps[j[0] % copies]()
                    j[0] += 1
                t = event_time(st, 20)
                tf = offn.ffn_flops(ms_, k, inter) / t / 1e12
                sweep.append({"M": ms_, "K": k, "I": inter, "us": t * 1e6, "tflops": tf, "frac_bf16_peak": tf / pk["bf16"]})
            # the decoder layer's FFN shape (hidden 4096, intermediate 14336) at prefill size
            gk, gi, gm = LAYER["hidden"], LAYER["inter"], 8192
            gen = torch.Generator(device=d.dev).manual_seed(1)
            big = SwiGLUFFN(*[(torch.randn(a, b, device=d.dev, generator=gen) * 0.02).bfloat16()
                              for a, b in ((gk, gi), (gk, gi), (gi, gk))])
            xs = torch.randn(gm, gk, device=d.dev, generator=gen).bfloat16()
            o = torch.empty(gm, gk, dtype=torch.float32, device=d.dev)
            t = event_time(lambda: big(xs, out=o), 10)
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
    t_rank = ms / 1e3 / steps
    return line(args, d, metric="ffn_swiglu_TFLOPs", unit="TFLOP/s", value=d.world * flops / sec / 1e12,
                sec_per_step=sec, scaling="weak", dtype="bf16",
                config={"workload": "swiglu_ffn x[128,1024] fp32 N(0,1), W N(0,0.02^2), bf16 operands fp32 accumulate",
                        "l2": "8 packed weight copies (201 MB) rotated between steps", "parallelism": "replicas only",
                        "launch": "CUDA graph of the step's kernels", "rounds": rounds},
                launches=SwiGLUFFN.launches_per_call * steps, clocks=clocks,
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
    steps = args.steps_for["layer"]
    t, geom = inputs.decoder_layer_inputs(**LAYER)
    dev_t = {k: v.to(d.dev) for k, v in t.items()}
    layer = DecoderLayer(dev_t, **geom)
    a = (dev_t["hidden"], dev_t["seq_lens"], dev_t["block_table"], dev_t["k_cache"], dev_t["v_cache"])
    keep = []
    replay = graphed(lambda: keep.append(layer.step(*a)))
    ms, clocks, rounds = timed(replay, d, steps, args.warmup)
    ops.check_device_status()
    ms_max, = d.reduce([ms], "MAX")
    sec = ms_max / 1e3 / steps
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
    t_rank = ms / 1e3 / steps
    return line(args, d, metric="decoder_layer_GBps", unit="GB/s", value=d.world * alg_b / sec / 1e9, sec_per_step=sec,
                scaling="weak", dtype="bf16",
                config={"workload": "llama_decoder_layer decode batch32 hidden4096 hq32 hkv8 d128 ffn14336 ctx4096 "
                                    "block128", "l2": "weights + KV (973 MB) larger than L2",
                        "parallelism": "replicas only", "launch": "one CUDA graph of the layer's kernels",
                        "rounds": rounds},
                launches=DecoderLayer.launches_per_step * steps, clocks=clocks,
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
    from pypto_b200.moe import MoELayer, PhaseTimer
    pk = peaks()
    steps = args.steps_for["moe"]
    T, H, I, E, K = MOE["tokens"], MOE["hidden"], MOE["inter"], MOE["n_experts"], MOE["topk"]
    L, tl = E // d.world, T // d.world
    gen = torch.Generator(device=d.dev).manual_seed(d.rank)
    gshared = torch.Generator(device=d.dev).manual_seed(12345)       # replicated pieces: same on all ranks
    gate_w = (torch.randn(H, E, device=d.dev, generator=gshared) * 0.02).bfloat16()
    bias = torch.rand(E, device=d.dev, generator=gshared) * 0.2 - 0.1
    layer = MoELayer.from_packed(ops.pack_weight(gate_w), bias, synthetic_experts(d.dev, gen, L, H, I),
                                 synthetic_experts(d.dev, gshared, 1, H, I), K, n_experts=E, comm=d.comm())
    x = torch.randn(tl, H, device=d.dev, generator=gen).bfloat16()

    ms, clocks, rounds = timed(lambda: layer.forward(x), d, steps, args.warmup)
    ops.check_device_status()
    if layer.status()[0]:
        raise RuntimeError(f"the MoE layer's kernels reported an error: {layer.status()}")
    ms_max, = d.reduce([ms], "MAX")
    sec = ms_max / 1e3 / steps
    flops = omoe.moe_flops(T, H, I, E, K)
    w_bytes = sum(v.numel() * v.element_size() for v in layer.routed.values()) + \
        sum(v.numel() * v.element_size() for v in layer.shared.values())
    # per-phase device times of one step (CUDA events the layer records between its phases on the main stream; the
    # shared expert runs beside them on its own stream), max over ranks
    ph = {}
    for _ in range(2):
        timer = PhaseTimer()
        layer.forward(x, timer=timer)
        ph = timer.result()
    names = sorted(ph)
    phases = dict(zip(names, d.reduce([ph[n] for n in names], "MAX")))
    fp8 = fp8_peak_tflops(d.dev)
    a2a = all_to_all_gbs(d)
    sweep = []
    e2e = cpu = None
    if not args.kernel_only:
        if d.world == 1 and not args.small:
            # token sweep on one GPU: the same 256 + 1 experts, T tokens; tensor-bound once T is large
            for tt in (4096, 8192, 16384, 32768):
                xt = torch.randn(tt, H, device=d.dev, generator=gen).bfloat16()
                t_s = event_time(lambda: layer.forward(xt), 3, warm=2)
                tf = omoe.moe_flops(tt, H, I, E, K) / t_s / 1e12
                sweep.append({"T": tt, "ms": t_s * 1e3, "tflops": tf, "frac_fp8_peak": tf / fp8 if fp8 else None,
                              "weights_GBps": w_bytes / t_s / 1e9})
                del xt
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
    t_rank = ms / 1e3 / steps
    value = flops / sec / 1e12
    # bytes that leave one GPU per exchange: a route's payload row out, a bf16 result row back
    routes_out = tl * K * (d.world - 1) / d.world
    return line(args, d, metric="moe_layer_TFLOPs", unit="TFLOP/s", value=value, sec_per_step=sec,
                scaling="strong", dtype="fp8_e4m3",
                config={"workload": f"deepseek_v3_moe tokens{T} hidden{H} experts{E}+1 inter{I} top{K} fp8 block128; "
                                    f"{L} routed experts and {tl} tokens per GPU",
                        "l2": f"expert weights per GPU {w_bytes / 1e9:.2f} GB, larger than L2",
                        "parallelism": f"ep{d.world}" if d.world > 1 else "single GPU, all experts local",
                        "rounds": rounds},
                launches=(17 if d.world > 1 else 15) * steps, clocks=clocks,
                roofline={"bound": "hbm", "achieved": w_bytes / t_rank / 1e9, "peak": pk["hbm"], "unit": "GB/s",
                          "frac": w_bytes / t_rank / 1e9 / pk["hbm"], "traffic": NCU_TRAFFIC["moe"],
                          "peak_source": pk["source"],
                          "note": "weight-bandwidth bound at ~128 tokens per expert: expert weight bytes of this GPU / "
                                  "time of the whole layer step"},
                cpu_baseline=cpu, e2e=e2e,
                extra={"tokens_per_s": T / sec, "phases_ms": phases, "sweep": sweep,
                       "frac_fp8_peak": value / d.world / fp8 if fp8 else None,
                       "exchange": {"bytes_out_per_gpu": int(routes_out * (H + H // 128 * 4 + 16)),
                                    "bytes_back_per_gpu": int(routes_out * H * 2),
                                    "back_path": "peer memory (own kernel + flags)" if layer.peer_exchange else
                                                 ("all-to-all-v" if d.world > 1 else "none"),
                                    "out_path": "peer memory (own kernel + flags)" if layer.peer_exchange_level >= 2 else
                                                ("all-to-all-v" if d.world > 1 else "none"),
                                    "all_to_all_GBps_measured": a2a}})


# --------------------------------------------------------------------------------------
# MX block-scaled FP8 matmul
# --------------------------------------------------------------------------------------

def run_matmul_mx(args, d: Dist):
    from oracle import matmul_mx as omx
    from pypto_b200 import ops
    steps = args.steps_for["matmul_mx"]
    m, n, k = (1024, 1024, 1024) if args.small else (MX["m"], MX["n"], MX["k"])
    gen = torch.Generator(device=d.dev).manual_seed(5)
    a = torch.randint(-3, 4, (m, k), device=d.dev, generator=gen).float().to(torch.float8_e4m3fn)
    b_t = torch.randint(-3, 4, (n, k), device=d.dev, generator=gen).float().to(torch.float8_e4m3fn)
    sa = torch.randint(120, 134, (m, k // 32), device=d.dev, generator=gen).to(torch.uint8)
    sb = torch.randint(120, 134, (k // 32, n), device=d.dev, generator=gen).to(torch.uint8)
    out = torch.empty(m, n, dtype=torch.float32, device=d.dev)
    fp8_peak_tflops(d.dev, refresh=True)        # the denominator: the largest of the figures taken before and after
    ms, clocks, rounds = timed(lambda: ops.matmul_mx(a, sa, b_t, sb, out=out), d, steps, args.warmup)
    ops.check_device_status()
    ms_max, = d.reduce([ms], "MAX")
    sec = ms_max / 1e3 / steps
    flops = 2.0 * m * n * k
    fp8 = fp8_peak_tflops(d.dev, refresh=True)
    cpu = e2e = None
    if not args.kernel_only:
        ah, bh = a.cpu().pin_memory(), b_t.cpu().pin_memory()
        sah, sbh = sa.cpu().pin_memory(), sb.cpu().pin_memory()
        oh = torch.empty(m, n).pin_memory()

        def call():
            o = ops.matmul_mx(ah.to(d.dev, non_blocking=True), sah.to(d.dev, non_blocking=True),
                              bh.to(d.dev, non_blocking=True), sbh.to(d.dev, non_blocking=True))
            oh.copy_(o, non_blocking=True)
            torch.cuda.synchronize()
        e2e_sec, = d.reduce([wall(call, 3)], "MAX")
        e2e = {"value": d.world * flops / e2e_sec / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": m * k + n * k + m * k // 32 + n * k // 32, "d2h_bytes_per_step": m * n * 4,
               "note": "operands and scale codes from pinned host memory, fp32 result back"}
        if d.rank == 0:
            cm = min(m, 512)        # the fp64 golden on a slab of rows
            ac, bc = a[:cm].cpu(), b_t.cpu().view(torch.uint8).t().contiguous().view(torch.float8_e4m3fn)
            sac, sbc = sa[:cm].cpu(), sb.cpu()
            t0 = time.perf_counter()
            omx.matmul_mx(ac, sac, bc, sbc)
            cdt = time.perf_counter() - t0
            cpu = {"value": 2.0 * cm * n * k / cdt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                   "kind": "port", "sample": f"{cm} of {m} rows, the reference's dequantise + fp64 matmul golden"}
    value = d.world * flops / sec / 1e12
    t_rank = ms / 1e3 / steps
    # problems of this size run on SM pairs (the launcher's rule): a kernel that packs the scale blocks, then the matmul
    sms = torch.cuda.get_device_properties(d.dev).multi_processor_count
    pair = (os.environ.get("PTO_MX_PAIR", "1") != "0" and m >= 512 and n >= 448 and k >= 1024
            and -(-m // 256) * -(-n // 224) >= sms)
    return line(args, d, metric="matmul_mx_TFLOPs", unit="TFLOP/s", value=value, sec_per_step=sec, scaling="weak",
                dtype="fp8_e4m3 x E8M0 scale per 32",
                config={"workload": f"matmul_mx m{m} n{n} k{k} e4m3 operands, E8M0 scale per 32-wide K group, fp32 out",
                        "l2": "operands 2 x 67 MB, output 268 MB: larger than L2", "parallelism": "replicas only",
                        "rounds": rounds},
                launches=steps * (2 if pair else 1), clocks=clocks,
                roofline={"bound": "tensor", "achieved": flops / t_rank / 1e12, "peak": fp8, "unit": "TFLOP/s",
                          "frac": flops / t_rank / 1e12 / fp8 if fp8 else None,
                          "traffic": (NCU_TRAFFIC["matmul_mx"] if pair else NCU_TRAFFIC["matmul_mx_one_cta"])
                          if (m, n, k) == (MX["m"], MX["n"], MX["k"]) else None,
                          "peak_source": "measured here: torch._scaled_mm e4m3 8192^3, best of 10, largest of the run's measurements",
                          "note": "2*m*n*k / CUDA-event time of the call: mx_pack_scales_kernel + matmul_mx_pair_kernel"
                                  if pair else "2*m*n*k / CUDA-event time of matmul_mx_kernel"},
                cpu_baseline=cpu, e2e=e2e)


# --------------------------------------------------------------------------------------
# CPU arm
# --------------------------------------------------------------------------------------

def run_reference(args):
    """The oracle (a port of the reference's torch golden) on the host cores, all threads.  The workload is one
    GPU's share of the repo arm's step (64 sequences, the same context lengths); the host's throughput does not
    depend on how many such shares a job holds, so the same figure stands beside every N."""
    d = Dist()
    if d.rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    host = decode_inputs(seed=0)
    steps = args.steps if args.steps is not None else 5
    cap_s, t_start = 150.0, time.perf_counter()       # wall-time cap of the whole run
    times, warm_done = [], 0
    nbytes = 0
    while len(times) < steps:
        dt, nbytes = cpu_attention(host)
        if warm_done < args.warmup:
            warm_done += 1
        else:
            times.append(dt)
        if time.perf_counter() - t_start > cap_s and times:
            break
    dt = sum(times) / len(times)
    value = nbytes / dt / 1e9
    out = {"impl": "reference", "metric": "paged_attn_decode_GBps", "value": value, "unit": "GB/s",
           "n_gpus": args.gpus, "steps": len(times), "warmup": warm_done, "ms_per_step": dt * 1e3,
           "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
           "config": {"workload": DECODE_DESC},
           "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                            "sample": "64 sequences per step (one GPU's share of a step, all 8 KV heads), torch CPU "
                                      f"oracle; {len(times)} of {steps} requested steps within the {cap_s:.0f} s cap"},
           "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
           "tokens_per_s": DECODE["batch"] / dt}
    print(json.dumps(out), flush=True)


RUNNERS = {"decode": lambda a, d: run_attention(a, d, "decode"), "verify": lambda a, d: run_attention(a, d, "verify"),
           "ffn": run_ffn, "layer": run_layer, "moe": run_moe, "matmul_mx": run_matmul_mx}
METRIC_OF = {"decode": "paged_attn_decode_GBps", "verify": "paged_attn_verify_GBps", "ffn": "ffn_swiglu_TFLOPs",
             "layer": "decoder_layer_GBps", "moe": "moe_layer_TFLOPs", "matmul_mx": "matmul_mx_TFLOPs"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all"] + list(RUNNERS))
    ap.add_argument("--kernel-only", action="store_true", help="skip the end-to-end and CPU legs (profiler captures)")
    ap.add_argument("--small", action="store_true",
                    help="reduced case of the workload for profiler captures (a few GB on the device at most): "
                         "verify batch 16, moe 16 experts / 256 tokens, matmul_mx 1024^3; other workloads unchanged")
    args = ap.parse_args()
    # stdout carries the JSON line and nothing else: NCCL's "NCCL version ..." banner (NCCL_DEBUG=VERSION) would sit
    # in front of it.  An explicit higher level (INFO, TRACE) is left alone.
    if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
        os.environ["NCCL_DEBUG"] = "WARN"
    if args.impl == "reference":
        run_reference(args)
        return
    if args.small:
        VERIFY.update(batch=16)
        MOE.update(tokens=256, n_experts=16)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    head = "decode" if args.workload == "all" else args.workload
    # --steps applies to the line that is printed as the headline; the other workloads keep their own counts
    args.steps_for = {}
    for w, m in METRIC_OF.items():
        args.steps_for[w] = args.steps_for[m] = args.steps if (args.steps is not None and w == head) else DEFAULT_STEPS[w]
    args.steps = args.steps_for[head]
    d = Dist().init()
    try:
        out = RUNNERS[head](args, d)
        if args.workload == "all":
            others = ["verify", "moe"] + (["ffn", "layer", "matmul_mx"] if d.world == 1 else [])
            workloads = {}
            for w in others:
                try:
                    torch.cuda.empty_cache()
                    r = RUNNERS[w](args, d)
                    for key in ("n_gpus", "warmup", "higher_is_better", "vs_baseline", "data"):
                        r.pop(key, None)
                    workloads[w] = r
                except Exception as e:       # a failing extra workload must not take the headline line with it
                    if d.world > 1:
                        raise                # ranks would diverge: fail loudly instead
                    workloads[w] = {"error": f"{type(e).__name__}: {e}", "trace": traceback.format_exc(limit=3)}
            out["workloads"] = workloads
            fp8 = fp8_peak_tflops(d.dev)
            pk = peaks()
            out["peaks"] = {"hbm_GBps": pk["hbm"], "bf16_TFLOPs": pk["bf16"], "bf16_TFLOPs_sustained": pk["bf16_sustained"],
                            "source": pk["source"], "fp8_TFLOPs": fp8,
                            "fp8_source": "measured here: torch._scaled_mm e4m3 8192^3, best of 10",
                            "all_to_all_GBps_out_per_gpu": all_to_all_gbs(d)}
        if d.rank == 0:
            print(json.dumps(out), flush=True)
    finally:
        d.close()


if __name__ == "__main__":
    main()
