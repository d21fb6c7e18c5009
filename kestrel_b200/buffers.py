"""Paired host/device staging buffers.

Same role and surface as ``CpuGpuBuffer`` in the reference
(``kestrel/utils/buffers.py:67-137``): a pinned host tensor, its device twin, a
NumPy view of the host side and non-blocking copies in both directions.
"""

from __future__ import annotations

import math

import torch


class CpuGpuBuffer:
    """Host tensor + device tensor of one shape; copies are asynchronous on CUDA."""

    def __init__(self, *size: int, dtype: torch.dtype, device: torch.device,
                 pin_memory: bool, with_numpy: bool = True, zero: bool = True) -> None:
        device = torch.device(device)
        pinned = bool(pin_memory) and device.type == "cuda"
        make = torch.zeros if zero else torch.empty
        self.cpu = make(*size, dtype=dtype, device="cpu", pin_memory=pinned)
        self.gpu = make(*size, dtype=dtype, device=device)
        if with_numpy:
            if dtype == torch.bfloat16:
                raise ValueError(
                    "bfloat16 torch tensors cannot be represented as NumPy arrays. "
                    "Instantiate CpuGpuBuffer(..., with_numpy=False) instead."
                )
            self.np = self.cpu.numpy()

    def copy_to_gpu(self, n: int | None = None) -> torch.Tensor:
        """Host -> device, whole buffer or the first ``n`` rows."""
        if n is None:
            return self.gpu.copy_(self.cpu, non_blocking=True)
        return self.gpu[:n].copy_(self.cpu[:n], non_blocking=True)

    def copy_to_cpu(self, n: int | None = None) -> torch.Tensor:
        """Device -> host (the caller synchronises before reading)."""
        if n is None:
            return self.cpu.copy_(self.gpu, non_blocking=True)
        return self.cpu[:n].copy_(self.gpu[:n], non_blocking=True)

    def cpu_view(self, shape: tuple[int, ...]) -> torch.Tensor:
        return self.cpu[: math.prod(shape)].view(shape)

    def gpu_view(self, shape: tuple[int, ...]) -> torch.Tensor:
        return self.gpu[: math.prod(shape)].view(shape)

    def copy_view_to_gpu(self, shape: tuple[int, ...]) -> torch.Tensor:
        dst = self.gpu_view(shape)
        dst.copy_(self.cpu_view(shape), non_blocking=True)
        return dst
