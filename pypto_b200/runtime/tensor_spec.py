"""Runtime tensor specification (python/pypto/runtime/tensor_spec.py:25-88)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch


@dataclass
class TensorSpec:
    name: str
    shape: list[int]
    dtype: torch.dtype
    init_value: int | float | torch.Tensor | Callable | None = field(default=None)
    is_output: bool = False

    def create_tensor(self) -> torch.Tensor:
        v = self.init_value
        if v is None:
            return torch.zeros(self.shape, dtype=self.dtype)
        if isinstance(v, (int, float)):
            return torch.full(self.shape, v, dtype=self.dtype)
        if isinstance(v, torch.Tensor):
            return v.to(dtype=self.dtype)
        if callable(v):
            if v in (torch.randn, torch.rand, torch.zeros, torch.ones):
                return v(self.shape, dtype=self.dtype)
            result: Any = v()
            return torch.as_tensor(result, dtype=self.dtype)
        raise TypeError(f"Unsupported init_value type {type(v)!r} for tensor {self.name!r}")
