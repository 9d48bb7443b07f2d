"""Benchmark of the paged-attention decode path (the workload the headline metric is quoted on).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of paged-attention decode over one batch of synthetic input:
batch 64 sequences per GPU, 32 query heads / 8 KV heads, head_dim 128, KV blocks of 128
tokens, q_len 1, context lengths uniform in [1024, 8192], block tables a random
permutation of a pool sized to need + 10 %, bf16 in / bf16 out, fp32 accumulation.
With N > 1 (torchrun, one rank per GPU) every rank decodes its own 64 sequences --
the path shards by batch with no collective -- so scaling is weak and ``value`` is the
sum over ranks of the KV bytes read, divided by the slowest rank's device time.

Prints ONE JSON line (rank 0).  ``value`` is kernel throughput with inputs resident in
HBM; ``e2e`` is the same metric through the launch surface (`run` with HOST tensors:
every input copied host->device and the output copied back inside the timed region).
``--impl reference`` times the CPU golden restatement (``oracle/``) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOAD = dict(batch=64, num_heads=32, kv_heads=8, head_dim=128, block_size=128, ctx_lo=1024,
                ctx_hi=8192, q_len=1)
METRIC, UNIT = "paged_attn_decode_GBps", "GB/s"
# dram bytes (read + write) of one pa_decode_kernel launch on this workload, from the ncu
# capture summarised in profiles/ (None until captured)
NCU_TRAFFIC_BYTES = 1406460304  # 1.398522e9 read + 7.938304e6 write, profiles/pa_decode_kernel_*.md


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.02):
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self.active = False

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:  # NVML missing: report that no clocks were read
            return self
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    _NAMES = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
              0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
              0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            if self.active:
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                    for bit, name in self._NAMES.items():
                        if mask & bit and name != "gpu_idle":
                            self.reasons.add(name)
                except Exception:
                    pass
            time.sleep(self.period)

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def make_inputs(seed: int):
    from oracle import inputs
    return inputs.paged_attention_inputs(seed=seed, **WORKLOAD)


def kv_bytes_of(d) -> int:
    from oracle import paged_attention as opa
    return opa.kv_bytes(d["context_lens"], d["kv_heads"], d["head_dim"])


def algorithmic_bytes(d) -> int:
    """KV rows of every visible token (K and V), plus Q, the output and the tables."""
    extra = d["query"].numel() * 2 * 2 + d["block_table"].numel() * 4 + d["context_lens"].numel() * 4
    return kv_bytes_of(d) + extra


def cpu_oracle_time(d, n_seq: int, repeats: int = 1):
    """Time the CPU golden restatement on the first n_seq sequences; returns (seconds, bytes)."""
    from oracle import paged_attention as opa
    sub = dict(d)
    sub["block_table"] = d["block_table"][:n_seq]
    sub["context_lens"] = d["context_lens"][:n_seq]
    rows = n_seq * d["q_len"] * d["num_heads"]
    sub["query"] = d["query"][:rows]

    def once():
        return opa.paged_attention(sub["query"], d["key_cache"], d["value_cache"], sub["block_table"],
                                   sub["context_lens"], num_heads=d["num_heads"], head_dim=d["head_dim"],
                                   block_size=d["block_size"], scale=d["scale"], kv_heads=d["kv_heads"],
                                   q_len=d["q_len"])

    once()  # warm-up (thread pool, allocator)
    t0 = time.perf_counter()
    for _ in range(repeats):
        once()
    dt = (time.perf_counter() - t0) / repeats
    return dt, opa.kv_bytes(sub["context_lens"], d["kv_heads"], d["head_dim"])


def run_reference(args):
    """CPU arm: the oracle (a port of the reference golden) on the host cores."""
    rank, world, _ = dist_env()
    if rank != 0:
        return
    d = make_inputs(0)
    n_seq = WORKLOAD["batch"]
    times = []
    for i in range(args.warmup + args.steps):
        dt, nbytes = cpu_oracle_time(d, n_seq)
        if i >= args.warmup:
            times.append(dt)
    dt = sum(times) / len(times)
    value = nbytes / dt / 1e9
    sample = f"{n_seq} of {WORKLOAD['batch']} sequences per step (all 8 KV heads), torch CPU"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "paged_attention_decode batch64 hq32 hkv8 d128 block128 ctx U[1024,8192] q_len1"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "tokens_per_s": n_seq / dt,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from pypto_b200 import ops

    d = make_inputs(rank)  # every rank decodes its own sequences
    g = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in d.items()}
    out = torch.empty(d["query"].shape, dtype=torch.bfloat16, device=dev)
    kw = dict(num_heads=d["num_heads"], kv_heads=d["kv_heads"], head_dim=d["head_dim"],
              block_size=d["block_size"], scale=d["scale"], q_len=d["q_len"], out=out)

    def step():
        ops.paged_attention(g["query"], g["key_cache"], g["value_cache"], g["block_table"],
                            g["context_lens"], **kw)

    def barrier():
        if world > 1:
            dist.barrier(device_ids=[local])
        torch.cuda.synchronize()

    sampler = ClockSampler(local).start()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.active = True
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    sampler.active = False
    ms = ev0.elapsed_time(ev1)
    ops.check_device_status()
    barrier()
    clocks = sampler.stop()

    my_bytes = algorithmic_bytes(d)
    stats = torch.tensor([ms, float(my_bytes), float(d["batch"])], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        ms_max, total_bytes, total_seq = mx[0].item(), sm[1].item(), sm[2].item()
    else:
        ms_max, total_bytes, total_seq = ms, float(my_bytes), float(d["batch"])
    sec_per_step = ms_max / 1e3 / args.steps
    value = total_bytes / sec_per_step / 1e9

    e2e_value = e2e_res = None
    h2d = d2h = 0
    if not args.kernel_only:
        e2e_value, e2e_res, h2d, d2h = end_to_end(args, d, dev, local, world, total_bytes, barrier)

    if rank == 0:
        emit(args, d, ms, my_bytes, value, sec_per_step, total_seq, world, clocks, e2e_value, e2e_res, h2d, d2h)
    if world > 1:
        dist.destroy_process_group()


def end_to_end(args, d, dev, local, world, total_bytes, barrier):
    """The same metric through the launch surface with HOST tensors."""
    import torch.distributed as dist

    from pypto_b200.runtime import RunConfig, fused_programs
    prog = fused_programs.paged_attention_program(d["batch"], d["num_heads"], d["head_dim"], d["block_size"],
                                                  d["max_blocks"], kv_heads=d["kv_heads"], q_len=d["q_len"],
                                                  out_dtype=torch.bfloat16)
    host = {k: d[k].pin_memory() for k in ("query", "key_cache", "value_cache", "block_table", "context_lens")}
    host_out = torch.empty(d["query"].shape, dtype=torch.bfloat16).pin_memory()
    cfg_t = fused_programs.pack_config(d)
    from pypto_b200 import ir
    compiled = ir.compile(prog, platform="b200")
    run_cfg = RunConfig(platform="b200", device_id=local)
    e2e_steps = max(2, min(args.steps, 5))
    compiled(host["query"], host["key_cache"], host["value_cache"], host["block_table"].flatten(),
             host["context_lens"], host_out, cfg_t, config=run_cfg)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        compiled(host["query"], host["key_cache"], host["value_cache"], host["block_table"].flatten(),
                 host["context_lens"], host_out, cfg_t, config=run_cfg)
    torch.cuda.synchronize()
    e2e_sec = (time.perf_counter() - t0) / e2e_steps
    e2e_stats = torch.tensor([e2e_sec], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(e2e_stats, op=dist.ReduceOp.MAX)
    e2e_value = total_bytes / e2e_stats[0].item() / 1e9
    h2d = sum(t.numel() * t.element_size() for t in host.values()) + cfg_t.numel() * 8
    d2h = host_out.numel() * host_out.element_size()
    # the resident-cache variant: KV pools stay on the device as DeviceTensors
    e2e_res = None
    try:
        e2e_res = fused_programs.time_resident(compiled, d, host, host_out, cfg_t, e2e_steps * 20, dev)
        res_stats = torch.tensor([e2e_res], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(res_stats, op=dist.ReduceOp.MAX)
        e2e_res = total_bytes / res_stats[0].item() / 1e9
    except Exception as e:  # reported, never hidden
        e2e_res = f"failed: {e}"
    return e2e_value, e2e_res, h2d, d2h


def emit(args, d, ms, my_bytes, value, sec_per_step, total_seq, world, clocks, e2e_value, e2e_res, h2d, d2h):
    peak, which = peaks()
    kernel_bytes = my_bytes  # one launch of the dominant kernel processes one rank's batch
    achieved = kernel_bytes / (ms / 1e3 / args.steps) / 1e9
    n_seq = WORKLOAD["batch"]
    cpu = None
    if not args.kernel_only:
        cpu_dt, cpu_bytes = cpu_oracle_time(d, n_seq, repeats=5)
        cpu = {"value": cpu_bytes / cpu_dt / 1e9, "unit": UNIT, "cores": torch.get_num_threads(),
               "kind": "port", "sample": f"{n_seq} of 64 sequences, mean of 5 passes, torch CPU oracle",
               "host_cpus": os.cpu_count()}
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "paged_attention_decode batch64/GPU hq32 hkv8 d128 block128 "
                               "ctx U[1024,8192] q_len1", "l2": "inputs (1.2 GB/GPU) larger than L2",
                   "kv_bytes_per_step_per_gpu": kv_bytes_of(d)},
        "tokens_per_s": total_seq / sec_per_step,
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": NCU_TRAFFIC_BYTES, "peak_source": which,
                     "note": "achieved = algorithmic bytes of one step / CUDA-event time of the step "
                             "(pa_decode_kernel + pa_merge_kernel), rank 0"},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "note": "run()-style call with every tensor on the host, KV pools included",
                "resident_kv_cache_value": e2e_res},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernel-only", action="store_true",
                    help="skip the end-to-end and CPU legs (used for profiler captures)")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps > 5:
            args.steps = 5  # each step is seconds of CPU work
        args.warmup = min(args.warmup, 1)
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
