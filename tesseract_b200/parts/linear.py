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
        if rows <= kernels.DECODE_LINEAR_MAX_ROWS and x.stride(1) == 1 and kernels.decode_linear_supported(rows, self.out_features,
                                                                               self.in_features):
            # decode-sized batches: the package's own weight-streaming kernel
            if out is None:
                out = torch.empty((rows, self.out_features), device=x.device,
                                  dtype=torch.float32 if float32_out else self.runtime.dtype)
            return kernels.decode_linear(self.weight, out, x=x,
                                         epilogue=kernels.EPI_F32 if float32_out else kernels.EPI_BF16)
        if float32_out:
            result = torch.mm(x, self.weight.t(), out_dtype=torch.float32)
            if out is not None:
                out.copy_(result)
                return out
            return result
        if out is None:
            return torch.mm(x, self.weight.t())
        return torch.mm(x, self.weight.t(), out=out)

    def forward_normed(self, deferred, float32_out: bool = False, epilogue: Optional[int] = None) -> torch.Tensor:
        """``norm(residual [+ update]) @ W^T`` with the norm folded into the product's kernel, or ``None`` when that
        is not possible (needs bfloat16, at most 16 rows, an RMSNorm, sizes the kernel takes): the caller then lets
        the norm run on its own."""
        from .norm import RMSNorm

        rows = deferred.rows
        if epilogue is None:
            epilogue = kernels.EPI_F32 if float32_out else kernels.EPI_BF16
        prologue = kernels.PRO_NORM if deferred.update is None else kernels.PRO_ADD_NORM
        fusable = (not self.runtime.is_float32 and isinstance(deferred.norm, RMSNorm) and not deferred.done
                   and rows <= kernels.DECODE_LINEAR_NORMED_MAX_ROWS and deferred.residual.is_contiguous()
                   and kernels.decode_linear_supported(rows, self.out_features, self.in_features, prologue))
        if not fusable:
            return None
        width = self.out_features // 2 if epilogue == kernels.EPI_SWIGLU else self.out_features
        out = torch.empty((rows, width), device=deferred.residual.device,
                          dtype=torch.float32 if epilogue == kernels.EPI_F32 else self.runtime.dtype)
        new_residual = torch.empty_like(deferred.residual) if deferred.update is not None else None
        kernels.decode_linear(self.weight, out, residual=deferred.residual, update=deferred.update,
                              norm_weight=deferred.norm.weight, eps=deferred.norm.eps, residual_out=new_residual,
                              epilogue=epilogue)
        deferred.fused(new_residual)
        return out
