"""bfloat16 matrix products y = x W^T with 32-bit accumulation.

The reference's engine runs every projection through a library matrix product (nn.Linear on
cuBLAS: utils/attention.py:119-124,181; utils/layers.py:205-217; utils/model.py:170).  This module
chooses, per call, between that library product and this package's own kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from .library import KernelError


def linear_bf16(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16:
        raise KernelError(f"linear_bf16 takes bfloat16 operands, got {x.dtype} and {weight.dtype}")
    out_dtype = out_dtype or torch.bfloat16
    if out_dtype == torch.bfloat16:
        if out is not None:
            return torch.matmul(x, weight.t(), out=out)
        return torch.matmul(x, weight.t())
    result = torch.matmul(x, weight.t()).to(out_dtype)
    if out is not None:
        out.copy_(result)
        return out
    return result
