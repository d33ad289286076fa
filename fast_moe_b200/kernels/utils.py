"""Backend selector kept for signature compatibility with the reference
(kernels/utils.py:13-17). The sm_100a library is the only implementation in this package: every
operator accepts ``kernel=`` and ignores its value."""
from __future__ import annotations

from enum import Enum, unique
from typing import Tuple

import torch


@unique
class KernelType(Enum):
    TRITON = "TRITON"
    PYTORCH = "PYTORCH"
    TRITON_CC = "TRITON_CC"


gpu_unavailable: Tuple[bool, str] = (
    not torch.cuda.is_available() or torch.cuda.device_count() == 0,
    "CUDA is not available or no Nvidia GPUs detected",
)


def to_fp32_if_pytorch_kernel(x: torch.Tensor, kernel: KernelType = KernelType.PYTORCH) -> torch.Tensor:
    """Same helper as the reference's (kernels/utils.py:28-33); used by tests that build an fp32
    comparison input."""
    if kernel == KernelType.PYTORCH:
        return x.to(torch.float32)
    return x
