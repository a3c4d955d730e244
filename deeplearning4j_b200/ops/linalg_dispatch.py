"""matmul dispatch: the hand-written tcgen05 GEMM for bf16/fp16 CUDA operands whose layouts a
TMA descriptor can address, torch otherwise (fp32/fp64, CPU, odd strides)."""
from __future__ import annotations

import torch


def matmul(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    if a.is_cuda and a.dim() == 2 and b.dim() == 2 and a.dtype in (torch.bfloat16, torch.float16) and a.dtype == b.dtype:
        from . import native
        if native.gemm_supported(a, b):
            return native.gemm(a, b)
    return torch.matmul(a, b)
