"""Op backends.  ``get_ops(device)`` returns the PyTorch reference backend for CPU tensors
and the sm_100a kernel backend for CUDA tensors.  There is no other dispatch: on a GPU the
native extension must be present, and its absence is an error rather than a silent fallback."""
from __future__ import annotations

import torch

from .reference import TORCH_OPS, TorchOps

_CUDA_OPS = None


def get_ops(device: torch.device | str):
    device = torch.device(device)
    if device.type == "cpu":
        return TORCH_OPS
    global _CUDA_OPS
    if _CUDA_OPS is None:
        from .cuda import CudaOps  # raises if the extension is not built
        _CUDA_OPS = CudaOps()
    return _CUDA_OPS


__all__ = ["get_ops", "TorchOps", "TORCH_OPS"]
