"""Matrix product ``y = x @ W^T`` with a weight kept as ``[out, in]``.

In float32 the product runs through the package's own 32-bit kernel (a fixed K-ordered
chain per output element).  In bfloat16 it runs through the library GEMM with 32-bit
accumulation, where the reference also calls a library (src/cuda/cublas.rs:49-92:
bfloat16 in and out, 32-bit compute, the weight transposed).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import kernels
from .base import Runtime


class Linear:
    def __init__(self, weight: torch.Tensor, runtime: Runtime):
        self.runtime = runtime
        self.weight = runtime.matrix(weight)
        self.out_features, self.in_features = self.weight.shape

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None,
                float32_out: bool = False) -> torch.Tensor:
        if x.shape[-1] != self.in_features:
            raise ValueError(f"linear expects width {self.in_features}, got {x.shape[-1]}")
        rows = x.shape[0]
        if self.runtime.is_float32:
            if out is None:
                out = torch.empty((rows, self.out_features), dtype=torch.float32, device=x.device)
            return kernels.gemm_f32_nt(x, self.weight, out)
        if not x.is_cuda:
            raise RuntimeError("tesseract_b200 has no CPU path; tensors must be on a CUDA device")
        if float32_out:
            result = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
            if out is not None:
                out.copy_(result)
                return out
            return result
        if out is None:
            return torch.mm(x, self.weight.t())
        return torch.mm(x, self.weight.t(), out=out)
