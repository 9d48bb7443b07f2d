"""``run``, ``validate_golden`` and ``benchmark`` (python/pypto/runtime/runner.py:628-682,
python/pypto/runtime/device_runner.py:850-899, python/pypto/runtime/bench.py:1267-1340)."""

from __future__ import annotations

from dataclasses import dataclass, field

import torch

from .run_config import RunConfig


@dataclass
class RunResult:
    passed: bool
    error: str | None = None
    execution_time: float | None = None

    def __str__(self):
        return "PASS" if self.passed else f"FAIL: {self.error}"


def run(program, *tensors, config: RunConfig | None = None):
    """Compile ``program`` and, when tensors are given, execute it.  Returns the
    ``CompiledProgram`` so that it can be called again."""
    from .. import ir
    config = config or RunConfig()
    compiled = ir.compile(program, output_dir=config.save_kernels_dir, strategy=config.strategy,
                          backend_type=config.backend_type, platform=config.platform)
    if tensors and not config.codegen_only:
        compiled(*tensors, config=config)
    return compiled


def validate_golden(outputs: dict, golden: dict, rtol: float = 1e-5, atol: float = 1e-5) -> None:
    """``torch.isclose`` comparison; NaN in the golden marks a don't-care element
    (device_runner.py:874-876).  Raises AssertionError naming the first failing tensor."""
    for name, exp in golden.items():
        if name not in outputs:
            raise AssertionError(f"output '{name}' missing")
        got = outputs[name]
        if got.shape != exp.shape:
            raise AssertionError(f"output '{name}' has shape {tuple(got.shape)}, expected {tuple(exp.shape)}")
        e, g = exp.to(torch.float64), got.to(torch.float64)
        care = ~torch.isnan(e)
        ok = torch.isclose(g[care], e[care], rtol=rtol, atol=atol)
        if not bool(ok.all()):
            bad = int((~ok).sum())
            diff = (g[care] - e[care]).abs().max().item()
            raise AssertionError(f"output '{name}' does not match the golden: {bad} of {int(care.sum())} elements "
                                 f"outside rtol={rtol} atol={atol}; max abs diff {diff:.6g}")


@dataclass
class BenchmarkStats:
    """Per-launch device times in microseconds (bench.py:452)."""
    device_wall_us: list[float] = field(default_factory=list)

    @property
    def rounds(self):
        return len(self.device_wall_us)

    @property
    def mean_us(self):
        return sum(self.device_wall_us) / max(1, len(self.device_wall_us))

    @property
    def min_us(self):
        return min(self.device_wall_us) if self.device_wall_us else float("nan")

    @property
    def median_us(self):
        s = sorted(self.device_wall_us)
        return s[len(s) // 2] if s else float("nan")


def benchmark(compiled, args, *, rounds: int = 20, warmup: int = 3, worker=None) -> BenchmarkStats:
    """Register once, loop the bound handle, time each launch on the device with CUDA events
    on the worker's stream.  ``args`` should be DeviceTensors (resident inputs) so that the
    numbers are kernel time; host tensors are accepted and then include their copies."""
    from .worker import ChipWorker
    own = worker is None
    w = worker or ChipWorker(RunConfig(platform=compiled.platform))
    stats = BenchmarkStats()
    try:
        handle = w.register(compiled)
        stream = torch.cuda.ExternalStream(w.stream, device=torch.device("cuda", w.device_id))
        for _ in range(warmup):
            handle(*args)
        for _ in range(rounds):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            handle(*args)
            e1.record(stream)
            e1.synchronize()
            stats.device_wall_us.append(e0.elapsed_time(e1) * 1e3)
    finally:
        if own:
            w.close()
    return stats
