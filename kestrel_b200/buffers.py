"""Pinned host tensor + device twin: what the page table keeps its block table in.

The page table only needs the part of the reference's ``CpuGpuBuffer`` (``kestrel/utils/buffers.py:67-137``)
that its deferred commits use: the two tensors, a NumPy view of the host side for in-place edits, and a
non-blocking host-to-device copy of the first rows.
"""

from __future__ import annotations

import torch


class CpuGpuBuffer:
    """``cpu`` (pinned when the device is CUDA), ``gpu`` and ``np`` views of one zero-filled buffer."""

    def __init__(self, *size: int, dtype: torch.dtype, device: torch.device, pin_memory: bool = True) -> None:
        device = torch.device(device)
        self.cpu = torch.zeros(*size, dtype=dtype, device="cpu", pin_memory=bool(pin_memory) and device.type == "cuda")
        self.gpu = torch.zeros(*size, dtype=dtype, device=device)
        self.np = self.cpu.numpy()

    def copy_to_gpu(self, n: int | None = None) -> torch.Tensor:
        """Host -> device on the current stream: the whole buffer or its first ``n`` rows."""
        if n is None:
            return self.gpu.copy_(self.cpu, non_blocking=True)
        return self.gpu[:n].copy_(self.cpu[:n], non_blocking=True)
